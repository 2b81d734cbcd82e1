"""Rimidra wiring — a hybrid decoder family behind the same ModelRunner / ForwardBatch /
AttentionBackend surface as llama.py.  Every size and constant is per layer and comes from the
model's config (`ModelConfig.layer_specs`); a layer is

    h = norm(x) ;  x <- x + (mixer(h) + ff(h))          (parallel: one norm feeds both sublayers)

with an RMS norm whose weight is stored around zero (scale = 1 + w), an fp32 residual stream x,
and one of two mixers:

  attention  GQA softmax attention without rotation: a sliding window, a learned per-head sink in
             the denominator, a linear distance bias with slope 2^(-8 (h + 1) / H), and a query
             temperature that grows with the logarithm of the position block
             (csrc/attn_general.cu over the paged KV pool);
  retention  decayed linear attention, S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, with partial
             rotate-half rotary positions on q and k, per-head RMS normalisation of o and a SiLU
             output gate (csrc/retention.cu over the per-request recurrent state pool);

and one of two feed-forwards: dense gated (tanh-form GELU) or a mixture of experts with sigmoid
routing scores, top-k WITHOUT renormalisation, experts that weight their INPUT, and a shared
expert scaled by a per-token sigmoid gate.  A layer may borrow another layer's weights
(`weights_of`) while keeping a cache / state of its own.

Kernels: tcgen05 GEMMs (ops.linear / linear_grouped_rows) for 16-bit aligned shapes, the CUDA-core
GEMM otherwise (float32 models, odd sizes); the fp32 residual-add + norm of layer i + 1 is fused with
the residual update of layer i (one kernel per layer boundary).  Softmax, norms, routing, the
residual stream, and everything inside the recurrence are fp32 in every dtype.  Single GPU.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from . import ops
from .attention_backend import RadixAttention
from .forward_batch_info import ForwardBatch, LogitsProcessorOutput
from .layers import LogitsProcessor


class _W:
    """A weight holder (same role as layers.LinearBase, without TP sharding)."""

    def __init__(self):
        self.weight: torch.Tensor = None


def _rotary_table(rot_dims: int, base: float, max_positions: int, device, factor: float = 1.0) -> Optional[torch.Tensor]:
    """fp32 [positions, rot_dims] = cos || sin of p · base^(-2 i / rot_dims) / factor, computed in float64 so
    the table holds the correctly rounded values even at large positions."""
    if rot_dims <= 0:
        return None
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / rot_dims) / float(factor)
    ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()


_ROTARY_TABLES: Dict[tuple, torch.Tensor] = {}


def _get_rotary_table(rot_dims, base, max_positions, device, factor: float = 1.0):
    """Tables are shared by the layers (and layer runs) with the same rotation."""
    key = (int(rot_dims), float(base), int(max_positions), str(device), float(factor))
    if key not in _ROTARY_TABLES:
        _ROTARY_TABLES[key] = _rotary_table(rot_dims, base, max_positions, device, factor)
    return _ROTARY_TABLES[key]


class RimidraAttention:
    """Windowed sink attention mixer.  Projections q ‖ k ‖ v are one GEMM; q, k, v are strided
    views of its output."""

    def __init__(self, hidden: int, m: dict, layer_id: int, device):
        self.heads, self.kv_heads = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
        self.dim, self.vdim = int(m["dim"]), int(m.get("vdim", m["dim"]))
        self.q_size, self.k_size, self.v_size = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.qkv_proj, self.o_proj, self.sink = _W(), _W(), _W()
        window = int((m.get("mask") or {}).get("size") or -1)
        qt = m.get("q_temp") or None
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / self.heads) for h in range(self.heads)],
                              dtype=torch.float32, device=device)
        self.attn = RadixAttention(self.heads, self.dim, float(m["scale"]), num_kv_heads=self.kv_heads,
                                   layer_id=layer_id, v_head_dim=self.vdim, sliding_window_size=window,
                                   distance_slopes=slopes,
                                   query_temperature=(float(qt["coef"]), int(qt["every"])) if qt else None,
                                   general=True)

    def share(self, other: "RimidraAttention"):
        self.qkv_proj, self.o_proj, self.sink = other.qkv_proj, other.o_proj, other.sink

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        self.attn.sinks = self.sink.weight  # fp32 [heads] (None: a plain softmax)
        qkv = ops.linear_any(h, self.qkv_proj.weight)
        q, k, v = qkv.split([self.q_size, self.k_size, self.v_size], dim=-1)
        o = self.attn(q, k, v, forward_batch, save_kv_cache=True)
        return ops.linear_any(o, self.o_proj.weight)

    __call__ = forward


class RimidraRetention:
    """Retention mixer.  Projections q ‖ k ‖ v ‖ g are one GEMM; the kernel rotates q / k, scales k
    by dim^-1/2, runs the recurrence over the request's state slot and returns o in fp32; the per-head
    RMS norm and the SiLU gate are one kernel in front of the output projection."""

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, max_positions: int, device):
        self.layer_id = layer_id
        self.num_heads = int(m["heads"])
        self.head_dim, self.v_head_dim = int(m["dim"]), int(m.get("vdim", m["dim"]))
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.eps = eps
        self.k_scale = self.head_dim ** -0.5
        rot = m.get("rot") or {}
        self.rotary_dim = int(rot.get("dims") or 0)
        self.cos_sin_cache = _get_rotary_table(self.rotary_dim, float(rot.get("base", 10000.0)), max_positions, device)
        decay = [float(d) for d in m["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError(f"layer {layer_id}: {len(decay)} decays for {self.num_heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        self.qkvg_proj, self.o_proj = _W(), _W()

    def share(self, other: "RimidraRetention"):
        self.qkvg_proj, self.o_proj = other.qkvg_proj, other.o_proj

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        qkvg = ops.linear_any(h, self.qkvg_proj.weight)
        q, k, v, g = qkvg.split([self.qk_size, self.qk_size, self.v_size, self.v_size], dim=-1)
        o = forward_batch.attn_backend.forward_retention(q, k, v, self, forward_batch)
        y = ops.headnorm_gate(o, g, self.num_heads, self.v_head_dim, self.eps)
        return ops.linear_any(y, self.o_proj.weight)

    __call__ = forward


class RimidraDenseMLP:
    def __init__(self, hidden: int, m: dict, act: str = "gelu_tanh"):
        self.ff = int(m["ff"])
        self.act = act
        self.gate_up_proj, self.down_proj = _W(), _W()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        if self.act == "silu":
            return ops.linear_any(ops.linear_silu_mul_any(h, self.gate_up_proj.weight), self.down_proj.weight)
        gate_up = ops.linear_any(h, self.gate_up_proj.weight)
        return ops.linear_any(ops.act_and_mul(gate_up, self.act), self.down_proj.weight)

    __call__ = forward


class RimidraMoE:
    """Sigmoid-routed experts that weight their input + a gated shared expert.  Router and shared
    gate are one fp32-output GEMM ([experts (+ 1), hidden]); the experts' gate ‖ up and down weights
    are stacked for the grouped GEMMs over expert-aligned 128-row tiles."""

    def __init__(self, hidden: int, m: dict):
        self.hidden = hidden
        self.num_experts, self.top_k = int(m["router"]["experts"]), int(m["router"]["top"])
        self.ff = int(m["expert"]["ff"])
        self.router = _W()            # [E (+ 1), hidden]: router rows, then the shared gate's row
        self.w_gate_up = _W()         # [E * 2 ff, hidden]
        self.w_down = _W()            # [E * hidden, ff]
        self.shared = RimidraDenseMLP(hidden, m["shared"], act="silu") if m.get("shared") else None

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        T, E = h.shape[0], self.num_experts
        z = ops.linear_any(h, self.router.weight, out_f32=True)
        ids, w = ops.moe_route_scores(z, E, self.top_k, score_func="sigmoid", renormalize=False)
        row_token, inv_pos, tile_group = ops.moe_align(ids, E)
        xs = ops.moe_gather_scaled(h, row_token, inv_pos, w)
        act = ops.linear_grouped_any(xs, self.w_gate_up.weight, tile_group, E, self.ff, silu_mul=True)
        y = ops.linear_grouped_any(act, self.w_down.weight, tile_group, E, self.hidden)
        shared = self.shared(h) if self.shared is not None else None
        return ops.moe_combine_gated(y, inv_pos, T, self.top_k, topk_w=None, shared=shared,
                                     shared_gate=z[:, E:] if self.shared is not None else None)

    __call__ = forward


class RimidraDecoderLayer:
    def __init__(self, config, layer_id: int, device):
        spec = config.layer_specs[layer_id]
        H = config.hidden_size
        self.layer_id = layer_id
        self.kind = spec["type"]
        self.weights_of = spec.get("weights_of")
        self.norm1 = _W()
        if self.kind == "attention":
            self.mixer = RimidraAttention(H, spec["mixer"], layer_id, device)
        else:
            self.mixer = RimidraRetention(H, spec["mixer"], layer_id, config.rms_norm_eps,
                                          config.max_position_embeddings, device)
        mlp = spec.get("mlp")
        if mlp is None:
            self.mlp = None
        elif mlp["kind"] == "dense":
            self.mlp = RimidraDenseMLP(H, mlp)
        elif mlp["kind"] == "moe":
            self.mlp = RimidraMoE(H, mlp)
        else:
            raise ValueError(f"layer {layer_id}: unknown feed-forward kind {mlp['kind']!r}")

    def share(self, other: "RimidraDecoderLayer"):
        """Use `other`'s tensors (norm, mixer, feed-forward); cache / state stay this layer's own."""
        self.norm1 = other.norm1
        self.mixer.share(other.mixer)
        self.mlp = other.mlp


class RimidraForCausalLM:
    def __init__(self, config, dtype=torch.bfloat16, device="cuda"):
        if config.layer_specs is None:
            raise ValueError("RimidraForCausalLM needs ModelConfig.layer_specs")
        self.config, self.dtype, self.device = config, dtype, device
        self.eps = config.rms_norm_eps
        self.embed_tokens, self.final_norm, self.lm_head = _W(), _W(), _W()
        self.layers = [RimidraDecoderLayer(config, i, device) for i in range(config.num_hidden_layers)]
        for layer in self.layers:
            if layer.weights_of is not None:
                layer.share(self.layers[layer.weights_of])
        self.logits_processor = LogitsProcessor(config)

    def cache_shapes(self):
        """(kv_shapes, state_shapes): per layer (kv_heads, k_dim, v_dim) or None, and (heads, k_dim,
        v_dim) of the recurrent state or None — what ModelRunner sizes the pools with."""
        kv, st = [], []
        for layer in self.layers:
            m = layer.mixer
            if layer.kind == "attention":
                kv.append((m.kv_heads, m.dim, m.vdim))
                st.append(None)
            else:
                kv.append(None)
                st.append((m.num_heads, m.head_dim, m.v_head_dim))
        return kv, st

    @torch.no_grad()
    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        x = ops.embed_f32(self.embed_tokens.weight, input_ids)  # fp32 residual stream
        mix = ff = None
        for layer in self.layers:
            # x += (mix + ff) of the previous layer, then this layer's norm — one kernel
            h = ops.residual_rmsnorm(x, layer.norm1.weight, self.eps, a=mix, b=ff, weight_offset=1.0)
            mix = layer.mixer(h, forward_batch)
            ff = layer.mlp(h) if layer.mlp is not None else None
            hook = getattr(self, "_layer_hook", None)
            if hook is not None:  # debugging / tests: the residual stream after this layer
                hook(layer.layer_id, x.clone() + (mix.float() + (ff.float() if ff is not None else 0)))
        rows = self.logits_processor.logit_rows(forward_batch)
        if rows is not None and rows.numel() == 0:  # a portion whose logits nobody asked for
            return LogitsProcessorOutput(next_token_logits=torch.empty(
                (0, self.config.vocab_size), device=x.device, dtype=torch.float32))
        if rows is None:
            xs = x
            hs = ops.residual_rmsnorm(xs, self.final_norm.weight, self.eps, a=mix, b=ff, weight_offset=1.0)
        else:
            ops.residual_rmsnorm(x, None, self.eps, a=mix, b=ff)
            xs = ops.embed_f32(x, rows)  # fp32 row gather
            hs = ops.residual_rmsnorm(xs, self.final_norm.weight, self.eps, weight_offset=1.0)
        logits = ops.linear_any(hs, self.lm_head.weight, out_f32=True)
        return LogitsProcessorOutput(next_token_logits=logits)

    __call__ = forward

    # ------------------------------------------------------------------------------------------
    # parameters.  Checkpoint names: embed, head, final.norm, l<i>.norm1, l<i>.mix.{q,k,v,o,sink,g},
    # l<i>.mlp.{gate,up,down} (dense), l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}
    # ------------------------------------------------------------------------------------------
    def full_shapes(self) -> Dict[str, Tuple[int, ...]]:
        cfg = self.config
        H = cfg.hidden_size
        shapes: Dict[str, Tuple[int, ...]] = {"embed": (cfg.vocab_size, H)}
        for i, spec in enumerate(cfg.layer_specs):
            if spec.get("weights_of") is not None:
                continue
            p, m = f"l{i}.", spec["mixer"]
            shapes[p + "norm1"] = (H,)
            dk, dv = int(m["dim"]), int(m.get("vdim", m["dim"]))
            if spec["type"] == "attention":
                nh, g = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
                shapes.update({p + "mix.q": (nh * dk, H), p + "mix.k": (g * dk, H), p + "mix.v": (g * dv, H),
                               p + "mix.sink": (nh,), p + "mix.o": (H, nh * dv)})
            else:
                nh = int(m["heads"])
                shapes.update({p + "mix.q": (nh * dk, H), p + "mix.k": (nh * dk, H), p + "mix.v": (nh * dv, H),
                               p + "mix.g": (nh * dv, H), p + "mix.o": (H, nh * dv)})
            mlp = spec.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                shapes.update({p + "mlp.gate": (ff, H), p + "mlp.up": (ff, H), p + "mlp.down": (H, ff)})
            else:
                ff = int(mlp["expert"]["ff"])
                for e in range(int(mlp["router"]["experts"])):
                    shapes.update({f"{p}mlp.e{e}.gate": (ff, H), f"{p}mlp.e{e}.up": (ff, H), f"{p}mlp.e{e}.down": (H, ff)})
                shapes[p + "mlp.router"] = (int(mlp["router"]["experts"]), H)
                if mlp.get("shared"):
                    sf = int(mlp["shared"]["ff"])
                    shapes.update({p + "mlp.shared.gate": (sf, H), p + "mlp.shared.up": (sf, H),
                                   p + "mlp.shared.down": (H, sf), p + "mlp.shared.sg": (1, H)})
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

        self.embed_tokens.weight = put(w["embed"])
        self.final_norm.weight = put(w["final.norm"])
        self.lm_head.weight = put(w["head"])
        for i, layer in enumerate(self.layers):
            if layer.weights_of is not None:
                continue
            p = f"l{i}."
            layer.norm1.weight = put(w[p + "norm1"])
            mx = layer.mixer
            if layer.kind == "attention":
                mx.qkv_proj.weight = put(torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"]], 0))
                mx.sink.weight = put32(w[p + "mix.sink"])
            else:
                mx.qkvg_proj.weight = put(torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"]], 0))
            mx.o_proj.weight = put(w[p + "mix.o"])
            mlp = layer.mlp
            if isinstance(mlp, RimidraDenseMLP):
                mlp.gate_up_proj.weight = put(torch.cat([w[p + "mlp.gate"], w[p + "mlp.up"]], 0))
                mlp.down_proj.weight = put(w[p + "mlp.down"])
            elif isinstance(mlp, RimidraMoE):
                E = mlp.num_experts
                mlp.w_gate_up.weight = put(torch.cat(
                    [t for e in range(E) for t in (w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"])], 0))
                mlp.w_down.weight = put(torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(E)], 0))
                router = [w[p + "mlp.router"]]
                if mlp.shared is not None:
                    router.append(w[p + "mlp.shared.sg"].reshape(1, -1))
                    mlp.shared.gate_up_proj.weight = put(torch.cat([w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"]], 0))
                    mlp.shared.down_proj.weight = put(w[p + "mlp.shared.down"])
                mlp.router.weight = put(torch.cat(router, 0))

    def dummy_full_weights(self, seed: int = 1234) -> Dict[str, torch.Tensor]:
        """Random weights by checkpoint name: projections N(0, 1/fan_in), norms and sinks N(0, 0.1²),
        rounded to bfloat16 like a stored checkpoint; one generator per parameter."""
        out = {}
        for idx, (name, shape) in enumerate(self.full_shapes().items()):
            g = torch.Generator().manual_seed(seed + idx)
            if len(shape) == 1:
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
