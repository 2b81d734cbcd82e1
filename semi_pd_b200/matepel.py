"""Matepel wiring — a hybrid decoder family behind the same ModelRunner / ForwardBatch / AttentionBackend surface as
llama.py, rimidra.py and nupovik.py.  Every size and constant comes from the model's config
(`ModelConfig.layer_specs`, one entry per layer).

    X_s = norm(embed[token]) · w_embed              for every stream s < S: the residual is S fp32 copies
    a sublayer q of a layer reads   u = Σ_s in_q[s] X_s,   y = sublayer(norm_q(u))
    and writes                      X'_t = Σ_s mix_q[s, t] X_s + mult · out_q[t] · y      (all streams at once)
    logits = head · norm(Σ_s X_s)

mixers
  lightning  decayed linear attention on SiLU-activated q, k, v: S_t = decay_h S_(t-1) + k_t v_tᵀ, o_t = S_tᵀ q_t; the
             heads' outputs are RMS-normed together (one weight over all heads), times sigmoid(W_g u), then W_o
             (csrc/retention.cu with the activation applied as the kernel reads its inputs).
  parallel   two branches on the same input, left_scale · left + right_scale · right:
             left   GQA softmax attention with biased q / k projections and NO value projection — the values are the
                    keys before rotation; partial rotate-half rotary positions whose frequencies are rescaled in two
                    regimes (fast-turning channels keep theirs, slow ones are divided by a factor, a ramp between;
                    cos and sin carry a magnitude 0.1 ln(factor) + 1); the softmax denominator holds one extra unit
                    (csrc/stream_ops.cu: bias + rotation + KV write in one kernel; csrc/attn_general*.cu with a sink of
                    score 0);
             right  an exponentially gated matrix memory (csrc/matrix_memory.cu): log input gate cap·tanh(·/cap), log
                    forget gate logsigmoid(cap·tanh(·/cap)), a running maximum that starts at 0; per-head unit RMS norm,
                    a weight over all heads, sigmoid(W_g u), then W_o.
feed-forward: W_down (g · sigmoid(1.702 g) · (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, ±limit).

Kernels: tcgen05 GEMMs (ops.linear) for 16-bit aligned shapes, the CUDA-core GEMM otherwise (float32 models, odd sizes);
every projection that reads one input is ONE GEMM (lightning: q ‖ k ‖ v ‖ g; parallel: both branches' eight
projections); the stream write of sublayer i, the stream read of sublayer i + 1 and its norm are one kernel, which also
combines the two branch outputs, their scales and the output bias in fp32.  Residual streams, norms, softmax, gates,
recurrent state and everything inside the recurrences are fp32 in every dtype.  Single GPU.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, Optional, Tuple

import torch

from . import ops
from .attention_backend import RadixAttention
from .forward_batch_info import ForwardBatch, LogitsProcessorOutput
from .layers import LogitsProcessor

GATE_SLOPE = 1.702  # the feed-forward's sigmoid slope: fixed by the design


class _W:
    """A weight holder (same role as layers.LinearBase, without TP sharding)."""

    def __init__(self):
        self.weight: torch.Tensor = None


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def scaled_rotary_table(rot_dims: int, base: float, scaling: Optional[dict], max_positions: int, device
                        ) -> Optional[torch.Tensor]:
    """fp32 [positions, rot_dims] = magnitude · (cos ‖ sin) of p · f_i, built in float64.  f_i = base^(-2 i / rot_dims);
    with scaling {factor, original, fast, slow}: c(t) = rot_dims · ln(original / (2 π t)) / (2 ln base) is the channel
    that turns t times within `original` positions; channels below lo = max(⌊c(fast)⌋, 0) keep f_i, channels above
    hi = min(⌈c(slow)⌉, rot_dims − 1) get f_i / factor, with a linear ramp between; magnitude = 0.1 ln(factor) + 1."""
    if rot_dims <= 0:
        return None
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / rot_dims)
    magnitude = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def channel(turns: float) -> float:
            return rot_dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(channel(float(scaling["fast"]))), 0)
        hi = min(math.ceil(channel(float(scaling["slow"]))), rot_dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        magnitude = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * freq[None, :]
    return (torch.cat([ang.cos(), ang.sin()], dim=-1) * magnitude).to(torch.float32).to(device).contiguous()


class StreamCoefficients:
    """The three coefficient sets of one sublayer's stream read / write: in [S], mix [S, S] (from, to), out [S]; fp32."""

    def __init__(self):
        self.w_in: torch.Tensor = None
        self.mix: torch.Tensor = None
        self.out: torch.Tensor = None


class SublayerOutput:
    """What a sublayer hands the stream write: y = sa · a + sb · b + sbias · bias (b, bias optional)."""

    __slots__ = ("a", "b", "bias", "sa", "sb", "sbias")

    def __init__(self, a, b=None, bias=None, sa=1.0, sb=1.0, sbias=1.0):
        self.a, self.b, self.bias, self.sa, self.sb, self.sbias = a, b, bias, sa, sb, sbias


class MatepelLightning:
    """Lightning-attention mixer.  q ‖ k ‖ v ‖ g are one GEMM; the recurrence kernel applies SiLU to q, k, v as it reads
    them and returns o in fp32; norm over all heads + sigmoid gate are one kernel in front of the output projection."""

    in_act = "silu"
    rotary_dim = 0
    cos_sin_cache = None
    k_scale = 1.0

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, device):
        self.layer_id, self.eps = layer_id, eps
        self.num_heads, self.head_dim, self.v_head_dim = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.decay = torch.tensor([float(d) for d in m["decay"]], dtype=torch.float32, device=device)
        self.in_proj, self.norm, self.o_proj = _W(), _W(), _W()

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> SublayerOutput:
        y = ops.linear_any(h, self.in_proj.weight)
        sizes = [self.qk_size, self.qk_size, self.v_size, self.v_size]
        q, k, v, g = y[:, : sum(sizes)].split(sizes, dim=-1)  # the GEMM's rows are padded to a multiple of 8
        o = forward_batch.attn_backend.forward_retention(q, k, v, self, forward_batch)
        y = ops.headnorm_gate(o, g, 1, self.v_size, self.eps, weight=self.norm.weight, gate_act="sigmoid")
        return SublayerOutput(ops.linear_any(y, self.o_proj.weight))

    __call__ = forward


class _MatrixMemory:
    """Descriptor of the gated matrix memory branch that the backend receives."""

    def __init__(self, m: dict, layer_id: int):
        self.layer_id = layer_id
        self.num_heads, self.head_dim, self.v_head_dim = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
        self.gate_cap = float(m.get("gate_cap") or 0.0)
        self.q_scale = self.head_dim ** -0.5
        self.i_bias: torch.Tensor = None  # fp32 [heads]
        self.f_bias: torch.Tensor = None


class MatepelParallel:
    """Softmax attention and gated matrix memory side by side.  All eight projections that read the mixer's input are
    one GEMM (rows padded to a multiple of 8): left q ‖ left k ‖ right q ‖ k ‖ v ‖ g ‖ i ‖ f."""

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, max_positions: int, device):
        self.layer_id, self.eps = layer_id, eps
        a, b = m["left"], m["right"]
        self.heads, self.kv_heads, self.dim = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"])
        rot = a.get("rot") or {}
        self.rot_dims = int(rot.get("dims") or 0)
        self.cos_sin = scaled_rotary_table(self.rot_dims, float(rot.get("base", 10000.0)), rot.get("scaling"),
                                           max_positions, device)
        # one more unit in the softmax denominator = a sink whose score is 0 for every head
        self.attn = RadixAttention(self.heads, self.dim, float(a["scale"]), num_kv_heads=self.kv_heads, layer_id=layer_id,
                                   v_head_dim=self.dim, general=True,
                                   sinks=torch.zeros(self.heads, dtype=torch.float32, device=device))
        self.memory = _MatrixMemory(b, layer_id)
        mm = self.memory
        self.left_scale, self.right_scale = float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))
        self.sizes = [self.heads * self.dim, self.kv_heads * self.dim, mm.num_heads * mm.head_dim,
                      mm.num_heads * mm.head_dim, mm.num_heads * mm.v_head_dim, mm.num_heads * mm.v_head_dim,
                      mm.num_heads, mm.num_heads]
        self.in_proj, self.left_o, self.right_o, self.right_norm = _W(), _W(), _W(), _W()
        self.q_bias: torch.Tensor = None     # fp32
        self.k_bias: torch.Tensor = None
        self.left_o_bias: torch.Tensor = None

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> SublayerOutput:
        backend, mm = forward_batch.attn_backend, self.memory
        y = ops.linear_any(h, self.in_proj.weight)
        lq, lk, rq, rk, rv, rg, zi, zf = y[:, : sum(self.sizes)].split(self.sizes, dim=-1)
        q = backend.forward_rotary_store(lq, lk, None, self.attn, forward_batch, q_bias=self.q_bias, k_bias=self.k_bias,
                                         cos_sin=self.cos_sin, rot_dims=self.rot_dims)
        left = ops.linear_any(self.attn(q, None, None, forward_batch, save_kv_cache=False), self.left_o.weight)
        o = backend.forward_matrix_memory(rq, rk, rv, zi, zf, mm, forward_batch)
        yr = ops.headnorm_gate(o, rg, mm.num_heads, mm.v_head_dim, self.eps, weight=self.right_norm.weight,
                               gate_act="sigmoid")
        right = ops.linear_any(yr, self.right_o.weight)
        return SublayerOutput(left, right, self.left_o_bias, self.left_scale, self.right_scale, self.left_scale)

    __call__ = forward


class MatepelMLP:
    """gate ‖ up are one GEMM; the clamps, the sigmoid-linear unit and the (u + 1) factor are one kernel."""

    def __init__(self, hidden: int, m: dict):
        self.ff = int(m["ff"])
        self.limit = float(m["limit"]) if m.get("limit") is not None else float("inf")  # no limit: nothing is clamped
        self.gate_up_proj, self.down_proj = _W(), _W()

    def forward(self, h: torch.Tensor) -> SublayerOutput:
        gate_up = ops.linear_any(h, self.gate_up_proj.weight)
        act = ops.act_and_mul(gate_up, "clamped_swish", limit=self.limit, slope=GATE_SLOPE)
        return SublayerOutput(ops.linear_any(act, self.down_proj.weight))

    __call__ = forward


class MatepelDecoderLayer:
    def __init__(self, config, layer_id: int, device):
        spec = config.layer_specs[layer_id]
        H = config.hidden_size
        self.layer_id, self.kind = layer_id, spec["type"]
        self.norm1, self.norm2 = _W(), _W()
        self.hc1, self.hc2 = StreamCoefficients(), StreamCoefficients()
        if self.kind == "lightning":
            self.mixer = MatepelLightning(H, spec["mixer"], layer_id, config.rms_norm_eps, device)
        else:
            self.mixer = MatepelParallel(H, spec["mixer"], layer_id, config.rms_norm_eps,
                                         config.max_position_embeddings, device)
        self.mlp = MatepelMLP(H, spec["mlp"]) if spec.get("mlp") is not None else None


class MatepelForCausalLM:
    def __init__(self, config, dtype=torch.bfloat16, device="cuda"):
        if config.layer_specs is None:
            raise ValueError("MatepelForCausalLM needs ModelConfig.layer_specs")
        self.config, self.dtype, self.device = config, dtype, device
        self.eps = config.rms_norm_eps
        self.mult = float(config.residual_mult)
        self.has_streams = config.num_streams is not None
        self.num_streams = int(config.num_streams) if self.has_streams else 1
        self.embed_tokens, self.embed_norm, self.final_norm, self.lm_head = _W(), _W(), _W(), _W()
        self.layers = [MatepelDecoderLayer(config, i, device) for i in range(config.num_hidden_layers)]
        self.logits_processor = LogitsProcessor(config)

    def cache_shapes(self):
        """(kv shapes, matrix-state shapes, vector-state sizes) per layer — what ModelRunner sizes the pools with.  A
        parallel layer owns keys and values per token (its attention branch) AND a matrix state plus the normaliser /
        running-maximum vector per request (its memory branch); a lightning layer owns a matrix state only."""
        kv, st, vec = [], [], []
        for layer in self.layers:
            m = layer.mixer
            if layer.kind == "parallel":
                mm = m.memory
                kv.append((m.kv_heads, m.dim, m.dim))
                st.append((mm.num_heads, mm.head_dim, mm.v_head_dim))
                vec.append(ops.matrix_memory_vector_dim(mm.num_heads, mm.head_dim, mm.v_head_dim))
            else:
                kv.append(None)
                st.append((m.num_heads, m.head_dim, m.v_head_dim))
                vec.append(None)
        return kv, st, vec

    def _write_args(self, y: Optional[SublayerOutput], hc: Optional[StreamCoefficients]) -> dict:
        if y is None:
            return {}
        return dict(a=y.a, b=y.b, bias=y.bias, sa=y.sa, sb=y.sb, sbias=y.sbias, mix=hc.mix, out_w=hc.out, mult=self.mult)

    @torch.no_grad()
    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        X = ops.embed_norm_streams(self.embed_tokens.weight, input_ids, self.embed_norm.weight, self.eps, self.num_streams)
        y = hc = None  # the sublayer output that is still to be written into the streams, and its coefficients
        hook = getattr(self, "_layer_hook", None)
        for layer in self.layers:
            # write of the previous sublayer + read and norm of this one — one kernel
            h = ops.streams_mix_norm(X, layer.norm1.weight, self.eps, in_w=layer.hc1.w_in, **self._write_args(y, hc))
            y, hc = layer.mixer(h, forward_batch), layer.hc1
            if layer.mlp is not None:
                h = ops.streams_mix_norm(X, layer.norm2.weight, self.eps, in_w=layer.hc2.w_in, **self._write_args(y, hc))
                y, hc = layer.mlp(h), layer.hc2
            if hook is not None:  # debugging / tests: the residual (sum of the streams) after this layer
                ops.streams_mix_norm(X, None, self.eps, **self._write_args(y, hc))
                y = hc = None
                hook(layer.layer_id, X.sum(1))
        rows = self.logits_processor.logit_rows(forward_batch)
        if rows is not None and rows.numel() == 0:  # a portion whose logits nobody asked for (nor the last write)
            return LogitsProcessorOutput(next_token_logits=torch.empty(
                (0, self.config.vocab_size), device=X.device, dtype=torch.float32))
        if rows is None:
            hs = ops.streams_mix_norm(X, self.final_norm.weight, self.eps, **self._write_args(y, hc))
        else:
            if y is not None:
                ops.streams_mix_norm(X, None, self.eps, **self._write_args(y, hc))
            hs = ops.streams_mix_norm(X, self.final_norm.weight, self.eps, rows=rows)
        logits = ops.linear_any(hs, self.lm_head.weight, out_f32=True)
        return LogitsProcessorOutput(next_token_logits=logits)

    __call__ = forward

    # ------------------------------------------------------------------------------------------
    # parameters.  Checkpoint names: embed, embed.norm, head, final.norm, l<i>.norm1, l<i>.norm2,
    # l<i>.hc<q>.{in,mix,out}, l<i>.mix.{q,k,v,g,o,norm} (lightning),
    # l<i>.mix.left.{q,q.b,k,k.b,o,o.b}, l<i>.mix.right.{q,k,v,g,o,norm,i,i.b,f,f.b} (parallel), l<i>.mlp.{gate,up,down}
    # ------------------------------------------------------------------------------------------
    def full_shapes(self) -> Dict[str, Tuple[int, ...]]:
        cfg = self.config
        H, S = cfg.hidden_size, self.num_streams
        shapes: Dict[str, Tuple[int, ...]] = {"embed": (cfg.vocab_size, H), "embed.norm": (H,)}
        for i, spec in enumerate(cfg.layer_specs):
            p, m = f"l{i}.", spec["mixer"]
            shapes[p + "norm1"] = (H,)
            if spec["type"] == "lightning":
                nh, dk, dv = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
                shapes.update({p + "mix.q": (nh * dk, H), p + "mix.k": (nh * dk, H), p + "mix.v": (nh * dv, H),
                               p + "mix.g": (nh * dv, H), p + "mix.o": (H, nh * dv), p + "mix.norm": (nh * dv,)})
            else:
                a, b = m["left"], m["right"]
                nh, g, dk = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"])
                shapes.update({p + "mix.left.q": (nh * dk, H), p + "mix.left.q.b": (nh * dk,),
                               p + "mix.left.k": (g * dk, H), p + "mix.left.k.b": (g * dk,),
                               p + "mix.left.o": (H, nh * dk), p + "mix.left.o.b": (H,)})
                nh, dk, dv = int(b["heads"]), int(b["dim"]), int(b.get("vdim", b["dim"]))
                shapes.update({p + "mix.right.q": (nh * dk, H), p + "mix.right.k": (nh * dk, H),
                               p + "mix.right.v": (nh * dv, H), p + "mix.right.g": (nh * dv, H),
                               p + "mix.right.o": (H, nh * dv), p + "mix.right.norm": (nh * dv,),
                               p + "mix.right.i": (nh, H), p + "mix.right.i.b": (nh,),
                               p + "mix.right.f": (nh, H), p + "mix.right.f.b": (nh,)})
            subs = ["hc1"]
            mlp = spec.get("mlp")
            if mlp is not None:
                ff = int(mlp["ff"])
                shapes.update({p + "norm2": (H,), p + "mlp.gate": (ff, H), p + "mlp.up": (ff, H), p + "mlp.down": (H, ff)})
                subs.append("hc2")
            if self.has_streams:
                for q in subs:
                    shapes.update({f"{p}{q}.in": (S,), f"{p}{q}.out": (S,), f"{p}{q}.mix": (S, S)})
        shapes["final.norm"] = (H,)
        shapes["head"] = (cfg.vocab_size, H)
        return shapes

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        w = {k: v for k, v in weights}
        shapes = self.full_shapes()
        missing = set(shapes) - set(w)
        if missing:
            raise KeyError(f"missing parameters: {sorted(missing)[:4]} …")
        for name, shape in shapes.items():
            if tuple(w[name].shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(w[name].shape)} does not match the config's {tuple(shape)}")

        def put(t):
            return t.to(self.dtype).to(self.device).contiguous()

        def put32(t):
            return t.to(torch.float32).to(self.device).contiguous()

        def rows8(parts):
            t = torch.cat(parts, 0)
            pad = _pad8(t.shape[0]) - t.shape[0]
            return put(torch.cat([t, t.new_zeros((pad, t.shape[1]))], 0) if pad else t)

        def coefficients(hc: StreamCoefficients, prefix: str):
            if self.has_streams:
                hc.w_in, hc.mix, hc.out = put32(w[prefix + ".in"]), put32(w[prefix + ".mix"]), put32(w[prefix + ".out"])
            else:  # one plain residual: x += mult · y
                hc.w_in = torch.ones(1, dtype=torch.float32, device=self.device)
                hc.mix, hc.out = hc.w_in.view(1, 1), hc.w_in

        self.embed_tokens.weight = put(w["embed"])
        self.embed_norm.weight = put(w["embed.norm"])
        self.final_norm.weight = put(w["final.norm"])
        self.lm_head.weight = put(w["head"])
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            layer.norm1.weight = put(w[p + "norm1"])
            coefficients(layer.hc1, p + "hc1")
            mx = layer.mixer
            if layer.kind == "lightning":
                mx.in_proj.weight = rows8([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"]])
                mx.norm.weight = put(w[p + "mix.norm"])
                mx.o_proj.weight = put(w[p + "mix.o"])
            else:
                a, b = p + "mix.left.", p + "mix.right."
                mx.in_proj.weight = rows8([w[a + "q"], w[a + "k"], w[b + "q"], w[b + "k"], w[b + "v"], w[b + "g"],
                                           w[b + "i"], w[b + "f"]])
                mx.q_bias, mx.k_bias, mx.left_o_bias = put32(w[a + "q.b"]), put32(w[a + "k.b"]), put32(w[a + "o.b"])
                mx.left_o.weight = put(w[a + "o"])
                mx.right_o.weight = put(w[b + "o"])
                mx.right_norm.weight = put(w[b + "norm"])
                mx.memory.i_bias, mx.memory.f_bias = put32(w[b + "i.b"]), put32(w[b + "f.b"])
            if layer.mlp is not None:
                layer.norm2.weight = put(w[p + "norm2"])
                coefficients(layer.hc2, p + "hc2")
                layer.mlp.gate_up_proj.weight = put(torch.cat([w[p + "mlp.gate"], w[p + "mlp.up"]], 0))
                layer.mlp.down_proj.weight = put(w[p + "mlp.down"])

    def dummy_full_weights(self, seed: int = 1234) -> Dict[str, torch.Tensor]:
        """Random weights by checkpoint name: projections N(0, 1/fan_in), norm weights around 1, biases N(0, 0.1²) (the
        forget gate's shifted up), stream coefficients around an even read and an identity-like mixing; rounded to
        bfloat16 like a stored checkpoint; one generator per parameter."""
        out = {}
        for idx, (name, shape) in enumerate(self.full_shapes().items()):
            g = torch.Generator().manual_seed(seed + idx)
            if ".hc" in name and name.endswith(".mix"):
                t = torch.eye(shape[0]) * 0.8 + 0.2 / shape[0] + torch.randn(shape, generator=g) * 0.05
            elif ".hc" in name:
                t = (1.0 / shape[0] if name.endswith(".in") else 1.0) + torch.randn(shape, generator=g) * 0.05
            elif len(shape) == 1 and "norm" in name:
                t = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif name.endswith(".f.b"):
                t = 3.0 + torch.randn(shape, generator=g) * 0.1
            elif len(shape) == 1:
                t = torch.randn(shape, generator=g) * 0.1
            elif name == "embed":
                t = torch.randn(shape, generator=g)
            else:
                t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            out[name] = t.to(torch.bfloat16)
        return out

    def init_dummy_weights(self, seed: int = 1234):
        w = self.dummy_full_weights(seed)
        self.load_weights(w.items())
        return w
