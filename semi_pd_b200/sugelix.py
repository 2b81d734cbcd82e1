"""Sugelix wiring — an attention-only decoder family behind the same ModelRunner / ForwardBatch / AttentionBackend
surface as llama.py, rimidra.py, nupovik.py and matepel.py.  Every size and constant comes from the model's config
(`ModelConfig.layer_specs`, one entry per layer RUN).

    x  = embed[token] · scale + pair[(previous · a + token · b) mod buckets]      fp32 residual stream, x0 = this x
    a block of layers may be repeated back to back, re-using its tensors (every repetition keeps a cache to itself);
    pass t of the block opens with  x += x0 (t > 0),  x += step[t]
    layer:  x += mixer(norm1(x));  x += ff(norm2(x))        norm(x) = tanh(alpha x) · w + b, no statistics
    logits = head · norm(x)

mixers (each ends with  W_o (heads ⊙ sigmoid(W_g u)),  the gate elementwise over the concatenated heads)
  attention         GQA softmax attention, biased q / k / v projections, rotation of channel pairs (2 i, 2 i + 1)
                    over the first rot.dims channels, scores capped by cap · tanh(· / cap), no window.
  attention_2       two softmax maps per head over the same values inside a sliding window; half-split rotation
                    with linearly scaled frequencies per map; o = unit_rms(a1 − lambda a2) · (1 − diff) with
                    lambda = exp(lq1 · lk1) − exp(lq2 · lk2) + diff, one number per layer.  The maps run as 2 H
                    query heads over 2 G key heads (rows reordered map-major when the weights are loaded, so the
                    grouped-query rule holds) whose value head is the key head modulo G.
  latent_attention  queries through a normed latent; the cache holds [normed key/value latent ‖ one rotated key
                    slice shared by the heads] per token.  Absorbed form: q_h is carried into the latent space
                    (W_uk_hᵀ q_h) beside its rotated slice, the general attention kernel scores it against the
                    cache rows with every head sharing the one "head", the values are the rows' latent columns,
                    and W_uv_h lifts the result; sliding window and a per-head sink.
feed-forward: mixture of experts, top-k by router logit with softmax weights over the chosen, each expert
W_down (g · sigmoid(1.702 g) · (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, ±limit); a shared expert of
the same form (own size and limit) is added for every token.

Kernels: tcgen05 GEMMs (ops.linear*, grouped and block-diagonal forms) for 16-bit aligned shapes, the CUDA-core GEMM
otherwise (float32 models, odd sizes); every projection that reads one input is ONE GEMM; csrc/mixer_ops.cu for the
pair embedding, the residual add fused with the tanh norm (and the pass opening), bias + rotation + cache write of
q / k / v in one launch, and the gate (with the difference of the maps and its norm); csrc/attn_general*.cu for all
three attentions.  Residual stream, norms, softmax, routing, positions and angles are fp32 in every dtype.  Single GPU.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, Optional, Tuple

import torch

from . import ops
from .attention_backend import RadixAttention
from .forward_batch_info import ForwardBatch, LogitsProcessorOutput
from .layers import LogitsProcessor
from .rimidra import _get_rotary_table

SWISH_SLOPE = 1.702  # the experts' sigmoid slope: fixed by the design


class _W:
    """A weight holder (same role as layers.LinearBase, without TP sharding)."""

    def __init__(self):
        self.weight: torch.Tensor = None


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class TanhNorm:
    """tanh(alpha x) · weight + bias with a scalar alpha."""

    def __init__(self):
        self.weight: torch.Tensor = None
        self.bias: torch.Tensor = None
        self.alpha: float = 1.0


class SugelixAttention:
    """Capped grouped-query attention.  q ‖ k ‖ v ‖ g are one GEMM; one launch adds the biases, rotates q and k and
    writes k and v into the cache."""

    paired, maps = True, 1

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, max_positions: int, device):
        self.layer_id, self.eps = layer_id, eps
        self.heads, self.kv_heads = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
        self.dim, self.vdim = int(m["dim"]), int(m.get("vdim", m["dim"]))
        n = self.maps
        self.sizes = [n * self.heads * self.dim, n * self.kv_heads * self.dim, self.kv_heads * self.vdim,
                      self.heads * self.vdim]
        rot = m.get("rot") or {}
        self.rot_dims = int(rot.get("dims") or 0)
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        self.cos_sin = _get_rotary_table(self.rot_dims, float(rot.get("base", 10000.0)), max_positions, device, factor)
        window = int((m.get("mask") or {}).get("size") or -1)
        self.attn = RadixAttention(n * self.heads, self.dim, float(m["scale"]), num_kv_heads=n * self.kv_heads,
                                   layer_id=layer_id, v_head_dim=self.vdim, sliding_window_size=window,
                                   logit_cap=float(m.get("softcap") or 0.0), general=True, num_v_heads=self.kv_heads)
        self.in_proj, self.o_proj = _W(), _W()
        self.q_bias: torch.Tensor = None  # fp32
        self.k_bias: torch.Tensor = None
        self.v_bias: torch.Tensor = None

    _TENSORS = ("in_proj", "o_proj", "q_bias", "k_bias", "v_bias")

    def share(self, other):
        for n in self._TENSORS:
            setattr(self, n, getattr(other, n))

    def cache_shape(self):
        return (self.maps * self.kv_heads, self.dim, self.vdim, self.kv_heads)

    def attend(self, h: torch.Tensor, forward_batch: ForwardBatch):
        """→ (attention output [T, maps · heads · vdim], the gate's view of the merged projection)."""
        y = ops.linear_any(h, self.in_proj.weight)
        q, k, v, g = y[:, : sum(self.sizes)].split(self.sizes, dim=-1)  # the GEMM's rows are padded to a multiple of 8
        n, a = self.maps, self.attn
        k_buf, v_buf = forward_batch.token_to_kv_pool.get_kv_buffer(self.layer_id)
        q_rot = torch.empty((h.shape[0], self.sizes[0]), device=h.device, dtype=h.dtype)
        forward_batch.attn_backend.forward_rotary_segments([
            ops.rotary_segment(q, q_rot, n * self.heads, self.dim, self.rot_dims, bias=self.q_bias),
            ops.rotary_segment(k, k_buf.view(k_buf.shape[0], -1), n * self.kv_heads, self.dim, self.rot_dims,
                               bias=self.k_bias, to_pool=True),
            ops.rotary_segment(v, v_buf.view(v_buf.shape[0], -1), self.kv_heads, self.vdim, 0, bias=self.v_bias,
                               to_pool=True),
        ], forward_batch, self.cos_sin, h.dtype, paired=self.paired)
        return a(q_rot, None, None, forward_batch, save_kv_cache=False), g

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        o, g = self.attend(h, forward_batch)
        return ops.linear_any(ops.heads_gate(o, g, self.heads, self.vdim), self.o_proj.weight)

    __call__ = forward


class SugelixDifferenceAttention(SugelixAttention):
    """Two maps per head; their difference at unit RMS per head, scaled, gated.  The merged projection's q and k rows
    are map-major ([map][head][dim]), so the attention output is [map 1's heads ‖ map 2's heads]."""

    paired, maps = False, 2

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, max_positions: int, device):
        super().__init__(hidden, m, layer_id, eps, max_positions, device)
        self.diff = float(m["diff"])
        self.lam: float = 0.0  # exp(lq1 · lk1) − exp(lq2 · lk2) + diff, set when the weights are loaded

    _TENSORS = SugelixAttention._TENSORS + ("lam",)

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        o, g = self.attend(h, forward_batch)
        n = self.heads * self.vdim
        y = ops.heads_gate(o[:, :n], g, self.heads, self.vdim, a2=o[:, n:], lam=self.lam, eps=self.eps,
                           post=1.0 - self.diff)
        return ops.linear_any(y, self.o_proj.weight)

    __call__ = forward


class SugelixLatentAttention:
    """Latent attention with a rotated key slice, a window and a sink.  The query latent, the key/value latent with
    its rotated slice and the gate are one GEMM (rows padded to a multiple of 8)."""

    def __init__(self, hidden: int, m: dict, layer_id: int, eps: float, max_positions: int, device):
        self.layer_id, self.eps = layer_id, eps
        self.heads, self.dim, self.rot_dim, self.vdim = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
        self.q_rank, self.rank = int(m["q_rank"]), int(m["kv_rank"])
        self.row = self.rank + self.rot_dim  # a cache row: latent ‖ rotated key slice
        self.sizes = [self.q_rank, self.row, self.heads * self.vdim]
        rot = m.get("rot") or {}
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        self.cos_sin = _get_rotary_table(self.rot_dim, float(rot.get("base", 10000.0)), max_positions, device, factor)
        window = int((m.get("mask") or {}).get("size") or -1)
        # every query head reads the one row per token: keys are the row, values its first `rank` columns
        self.attn = RadixAttention(self.heads, self.row, float(m["scale"]), num_kv_heads=1, layer_id=layer_id,
                                   v_head_dim=self.rank, sliding_window_size=window, general=True, num_v_heads=1,
                                   v_slot_stride=self.row)
        self.in_proj, self.q_norm, self.uq, self.c_norm, self.uk_t, self.uv, self.o_proj, self.sink = (_W() for _ in range(8))

    _TENSORS = ("in_proj", "q_norm", "uq", "c_norm", "uk_t", "uv", "o_proj", "sink")

    def share(self, other):
        for n in self._TENSORS:
            setattr(self, n, getattr(other, n))

    def cache_shape(self):
        return (1, self.row, 0)

    def forward(self, h: torch.Tensor, forward_batch: ForwardBatch) -> torch.Tensor:
        self.attn.sinks = self.sink.weight  # fp32 [heads] (None: a plain softmax)
        T, H = h.shape[0], self.heads
        y = ops.linear_any(h, self.in_proj.weight)
        cq_raw, ckv, g = y[:, : sum(self.sizes)].split(self.sizes, dim=-1)
        q = ops.linear_any(ops.rmsnorm_store(cq_raw, self.q_norm.weight, self.eps, want_out=True), self.uq.weight)
        pool = forward_batch.token_to_kv_pool.get_key_buffer(self.layer_id)
        pool = pool.view(pool.shape[0], -1)
        ops.rmsnorm_store(ckv[:, : self.rank], self.c_norm.weight, self.eps, pool=pool, loc=forward_batch.out_cache_loc)
        # q in the cache's coordinates: per head [W_ukᵀ q_unrotated (rank) ‖ rotated slice]
        q_lat = torch.empty((T, H * self.row), device=h.device, dtype=h.dtype)
        ops.linear_block_diag_any(q, self.uk_t.weight, H, self.dim, self.rank, x_group_stride=self.dim + self.rot_dim,
                                  out=q_lat, out_group_stride=self.row)
        forward_batch.attn_backend.forward_rotary_segments([
            ops.rotary_segment(q[:, self.dim:], q_lat[:, self.rank:], H, self.rot_dim, self.rot_dim,
                               src_head=self.dim + self.rot_dim, dst_head=self.row),
            ops.rotary_segment(ckv[:, self.rank:], pool[:, self.rank:], 1, self.rot_dim, self.rot_dim, to_pool=True),
        ], forward_batch, self.cos_sin, h.dtype, paired=False)
        o_lat = self.attn(q_lat, None, None, forward_batch, save_kv_cache=False)
        o = ops.linear_block_diag_any(o_lat, self.uv.weight, H, self.rank, self.vdim)
        return ops.linear_any(ops.heads_gate(o, g, H, self.vdim), self.o_proj.weight)

    __call__ = forward


class SugelixExpert:
    """A dense feed-forward of the experts' form (the shared expert): gate ‖ up are one GEMM."""

    def __init__(self, hidden: int, m: dict):
        self.ff = int(m["ff"])
        self.limit = float(m["limit"]) if m.get("limit") is not None else float("inf")
        self.gate_up_proj, self.down_proj = _W(), _W()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        act = ops.act_and_mul(ops.linear_any(h, self.gate_up_proj.weight), "clamped_swish", limit=self.limit,
                              slope=SWISH_SLOPE)
        return ops.linear_any(act, self.down_proj.weight)

    __call__ = forward


class SugelixMoE:
    """Top-k experts by router logit, weights = softmax over the chosen logits; the experts' gate ‖ up and down
    weights are stacked for the grouped GEMMs over expert-aligned 128-row tiles; the routing weights multiply the
    experts' outputs in the combine, which also adds the shared expert."""

    def __init__(self, hidden: int, m: dict):
        self.hidden = hidden
        self.num_experts, self.top_k = int(m["router"]["experts"]), int(m["router"]["top"])
        self.ff = int(m["expert"]["ff"])
        self.limit = float(m["expert"]["limit"]) if m["expert"].get("limit") is not None else float("inf")
        self.router, self.w_gate_up, self.w_down = _W(), _W(), _W()  # [E, hidden], [E · 2 ff, hidden], [E · hidden, ff]
        self.shared = SugelixExpert(hidden, m["shared"]) if m.get("shared") else None

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        T, E = h.shape[0], self.num_experts
        z = ops.linear_any(h, self.router.weight, out_f32=True)
        # softmax over all experts, renormalised over the chosen = softmax over the chosen logits
        ids, w = ops.moe_route_scores(z, E, self.top_k, score_func="softmax", renormalize=True)
        row_token, inv_pos, tile_group = ops.moe_align(ids, E)
        xs = ops.moe_gather_scaled(h, row_token, inv_pos, None)
        gate_up = ops.linear_grouped_any(xs, self.w_gate_up.weight, tile_group, E, 2 * self.ff)
        act = ops.act_and_mul(gate_up, "clamped_swish", limit=self.limit, slope=SWISH_SLOPE)
        y = ops.linear_grouped_any(act, self.w_down.weight, tile_group, E, self.hidden)
        shared = self.shared(h) if self.shared is not None else None
        return ops.moe_combine_gated(y, inv_pos, T, self.top_k, topk_w=w, shared=shared)

    __call__ = forward


_MIXERS = {"attention": SugelixAttention, "attention_2": SugelixDifferenceAttention,
           "latent_attention": SugelixLatentAttention}


class SugelixDecoderLayer:
    """One layer RUN: its own cache (layer_id), tensors of its own or of the first run of the layer."""

    def __init__(self, config, layer_id: int, device):
        spec = config.layer_specs[layer_id]
        H = config.hidden_size
        self.layer_id, self.kind = layer_id, spec["type"]
        self.name_index = int(spec.get("layer", layer_id))  # index in the checkpoint's tensor names
        self.weights_of = spec.get("weights_of")
        self.pass_index = spec.get("pass_index")            # number of the loop pass this run opens, or None
        self.norm1, self.norm2 = TanhNorm(), TanhNorm()
        self.mixer = _MIXERS[self.kind](H, spec["mixer"], layer_id, config.rms_norm_eps,
                                        config.max_position_embeddings, device)
        self.mlp = SugelixMoE(H, spec["mlp"]) if spec.get("mlp") is not None else None

    def share(self, other: "SugelixDecoderLayer"):
        self.norm1, self.norm2 = other.norm1, other.norm2
        self.mixer.share(other.mixer)
        self.mlp = other.mlp


class SugelixForCausalLM:
    def __init__(self, config, dtype=torch.bfloat16, device="cuda"):
        if config.layer_specs is None:
            raise ValueError("SugelixForCausalLM needs ModelConfig.layer_specs")
        self.config, self.dtype, self.device = config, dtype, device
        self.eps = config.rms_norm_eps
        self.embed_scale = float(config.embedding_scale)
        self.pair = config.pair_embedding
        self.loop_times = int(config.loop_times)
        self.has_passes = any(s.get("pass_index") is not None for s in config.layer_specs)
        self.embed_tokens, self.pair_table, self.lm_head = _W(), _W(), _W()
        self.loop_step: torch.Tensor = None  # fp32 [times, width]
        self.final_norm = TanhNorm()
        self.layers = [SugelixDecoderLayer(config, i, device) for i in range(config.num_hidden_layers)]
        for layer in self.layers:
            if layer.weights_of is not None:
                layer.share(self.layers[layer.weights_of])
        self.logits_processor = LogitsProcessor(config)

    def cache_shapes(self):
        """(kv shapes, matrix-state shapes, vector-state sizes, extras) per layer run — what ModelRunner sizes the
        pools with.  A run of the two grouped attentions owns (key heads, dim, vdim, value heads) per token, a latent
        run one row [latent ‖ rotated key slice] that is read as keys and as values; no run has a recurrent state,
        but the pair embedding keeps every request's last token."""
        n = len(self.layers)
        return ([layer.mixer.cache_shape() for layer in self.layers], [None] * n, [None] * n,
                {"token_state": self.pair is not None})

    @torch.no_grad()
    def forward(self, input_ids, positions, forward_batch: ForwardBatch, input_embeds=None) -> LogitsProcessorOutput:
        pair = self.pair or {}
        x = forward_batch.attn_backend.forward_pair_embedding(
            self.embed_tokens.weight, input_ids, forward_batch, scale=self.embed_scale, pair=self.pair_table.weight,
            buckets=pair.get("buckets", 0), mul_prev=pair.get("mul_prev", 0), mul_cur=pair.get("mul_cur", 0))
        x0 = x.clone() if self.loop_times > 1 else None  # x is updated in place from here on
        pending = None  # the sublayer output that is still to be added to x
        hook = getattr(self, "_layer_hook", None)
        for layer in self.layers:
            t = layer.pass_index
            # x += the previous sublayer (+ what opens a pass), then this layer's first norm — one kernel
            h = ops.residual_tanh_norm(x, layer.norm1.weight, layer.norm1.bias, layer.norm1.alpha, a=pending,
                                       x0=x0 if t is not None and t > 0 else None,
                                       vec=self.loop_step[t] if t is not None else None)
            pending = layer.mixer(h, forward_batch)
            if layer.mlp is not None:
                h = ops.residual_tanh_norm(x, layer.norm2.weight, layer.norm2.bias, layer.norm2.alpha, a=pending)
                pending = layer.mlp(h)
            if hook is not None:  # debugging / tests: the residual stream after this layer run
                ops.residual_tanh_norm(x, None, None, 1.0, a=pending)
                pending = None
                hook(layer.layer_id, x.clone())
        rows = self.logits_processor.logit_rows(forward_batch)
        if rows is not None and rows.numel() == 0:  # a portion whose logits nobody asked for
            return LogitsProcessorOutput(next_token_logits=torch.empty(
                (0, self.config.vocab_size), device=x.device, dtype=torch.float32))
        fn = self.final_norm
        if rows is None:
            hs = ops.residual_tanh_norm(x, fn.weight, fn.bias, fn.alpha, a=pending)
        else:
            if pending is not None:
                ops.residual_tanh_norm(x, None, None, 1.0, a=pending)
            hs = ops.residual_tanh_norm(x, fn.weight, fn.bias, fn.alpha, rows=rows)
        logits = ops.linear_any(hs, self.lm_head.weight, out_f32=True)
        return LogitsProcessorOutput(next_token_logits=logits)

    __call__ = forward

    # ------------------------------------------------------------------------------------------
    # parameters.  Checkpoint names: embed, bigram, loop.step, head, final.norm{,.b,.alpha}, l<i>.norm<j>{,.b,.alpha},
    # l<i>.mix.{q,q.b,k,k.b,v,v.b,g,o} (+ lq1,lk1,lq2,lk2 for attention_2),
    # l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o} (latent), l<i>.mlp.{router, e<j>.{gate,up,down},
    # shared.{gate,up,down}}
    # ------------------------------------------------------------------------------------------
    def full_shapes(self) -> Dict[str, Tuple[int, ...]]:
        cfg = self.config
        H = cfg.hidden_size
        shapes: Dict[str, Tuple[int, ...]] = {"embed": (cfg.vocab_size, H)}
        if self.pair is not None:
            shapes["bigram"] = (self.pair["buckets"] + 1, H)
        if self.has_passes:
            shapes["loop.step"] = (self.loop_times, H)

        def norm(name):
            shapes.update({name: (H,), name + ".b": (H,), name + ".alpha": ()})

        for spec in cfg.layer_specs:
            if spec.get("weights_of") is not None:
                continue
            p, m = f"l{spec['layer']}.", spec["mixer"]
            norm(p + "norm1")
            nh, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if spec["type"] == "latent_attention":
                dr, rq, rk = int(m["rot_dim"]), int(m["q_rank"]), int(m["kv_rank"])
                shapes.update({p + "mix.dq": (rq, H), p + "mix.dq.norm": (rq,), p + "mix.uq": (nh * (dk + dr), rq),
                               p + "mix.dkv": (rk + dr, H), p + "mix.dkv.norm": (rk,), p + "mix.uk": (nh * dk, rk),
                               p + "mix.uv": (nh * dv, rk), p + "mix.sink": (nh,), p + "mix.g": (nh * dv, H),
                               p + "mix.o": (H, nh * dv)})
            else:
                g, n = int(m.get("kv_heads", nh)), 2 if spec["type"] == "attention_2" else 1
                shapes.update({p + "mix.q": (n * nh * dk, H), p + "mix.q.b": (n * nh * dk,), p + "mix.k": (n * g * dk, H),
                               p + "mix.k.b": (n * g * dk,), p + "mix.v": (g * dv, H), p + "mix.v.b": (g * dv,),
                               p + "mix.g": (nh * dv, H), p + "mix.o": (H, nh * dv)})
                if n == 2:
                    shapes.update({p + "mix." + s: (dk,) for s in ("lq1", "lk1", "lq2", "lk2")})
            mlp = spec.get("mlp")
            if mlp is None:
                continue
            norm(p + "norm2")
            ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            for e in range(E):
                shapes.update({f"{p}mlp.e{e}.gate": (ff, H), f"{p}mlp.e{e}.up": (ff, H), f"{p}mlp.e{e}.down": (H, ff)})
            shapes[p + "mlp.router"] = (E, H)
            if mlp.get("shared"):
                sf = int(mlp["shared"]["ff"])
                shapes.update({p + "mlp.shared.gate": (sf, H), p + "mlp.shared.up": (sf, H), p + "mlp.shared.down": (H, sf)})
        norm("final.norm")
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

        def norm(n: TanhNorm, name: str):
            n.weight, n.bias, n.alpha = put(w[name]), put(w[name + ".b"]), float(w[name + ".alpha"].float())

        def map_major(t, heads, dim):
            """rows [head][map][dim] → [map][head][dim] (a vector or a matrix's rows)."""
            return t.reshape(heads, 2, dim, *t.shape[1:]).transpose(0, 1).reshape(t.shape)

        self.embed_tokens.weight = put(w["embed"])
        self.pair_table.weight = put(w["bigram"]) if self.pair is not None else None
        self.loop_step = put32(w["loop.step"]) if self.has_passes else None
        norm(self.final_norm, "final.norm")
        self.lm_head.weight = put(w["head"])
        for layer in self.layers:
            if layer.weights_of is not None:
                continue
            p = f"l{layer.name_index}."
            norm(layer.norm1, p + "norm1")
            mx = layer.mixer
            if layer.kind == "latent_attention":
                mx.in_proj.weight = rows8([w[p + "mix.dq"], w[p + "mix.dkv"], w[p + "mix.g"]])
                mx.q_norm.weight, mx.c_norm.weight = put(w[p + "mix.dq.norm"]), put(w[p + "mix.dkv.norm"])
                mx.uq.weight = put(w[p + "mix.uq"])
                # absorbed form: per head the transposed key lift [rank, dim], stacked; the value lift as stored
                uk = w[p + "mix.uk"].view(mx.heads, mx.dim, mx.rank)
                mx.uk_t.weight = put(uk.transpose(1, 2).reshape(mx.heads * mx.rank, mx.dim))
                mx.uv.weight = put(w[p + "mix.uv"])
                mx.sink.weight = put32(w[p + "mix.sink"])
            else:
                q, qb, k, kb = w[p + "mix.q"], w[p + "mix.q.b"], w[p + "mix.k"], w[p + "mix.k.b"]
                if layer.kind == "attention_2":
                    q, qb = map_major(q, mx.heads, mx.dim), map_major(qb, mx.heads, mx.dim)
                    k, kb = map_major(k, mx.kv_heads, mx.dim), map_major(kb, mx.kv_heads, mx.dim)
                    f = {s: w[p + "mix." + s].double() for s in ("lq1", "lk1", "lq2", "lk2")}
                    mx.lam = (math.exp(float((f["lq1"] * f["lk1"]).sum())) - math.exp(float((f["lq2"] * f["lk2"]).sum()))
                              + mx.diff)
                mx.in_proj.weight = rows8([q, k, w[p + "mix.v"], w[p + "mix.g"]])
                mx.q_bias, mx.k_bias, mx.v_bias = put32(qb), put32(kb), put32(w[p + "mix.v.b"])
            mx.o_proj.weight = put(w[p + "mix.o"])
            mlp = layer.mlp
            if mlp is None:
                continue
            norm(layer.norm2, p + "norm2")
            E = mlp.num_experts
            mlp.w_gate_up.weight = put(torch.cat(
                [t for e in range(E) for t in (w[f"{p}mlp.e{e}.gate"], w[f"{p}mlp.e{e}.up"])], 0))
            mlp.w_down.weight = put(torch.cat([w[f"{p}mlp.e{e}.down"] for e in range(E)], 0))
            mlp.router.weight = put(w[p + "mlp.router"])
            if mlp.shared is not None:
                mlp.shared.gate_up_proj.weight = put(torch.cat([w[p + "mlp.shared.gate"], w[p + "mlp.shared.up"]], 0))
                mlp.shared.down_proj.weight = put(w[p + "mlp.shared.down"])
        for layer in self.layers:  # later runs of a looped layer read the tensors (and constants) just loaded
            if layer.weights_of is not None:
                layer.share(self.layers[layer.weights_of])

    def dummy_full_weights(self, seed: int = 1234) -> Dict[str, torch.Tensor]:
        """Random weights by checkpoint name: projections N(0, 1/fan_in), norm weights around 1 with an alpha near
        0.5, the other vectors N(0, 0.1²), embedding rows of unit scale divided by the embedding's multiplier;
        rounded to bfloat16 like a stored checkpoint; one generator per parameter."""
        out = {}
        for idx, (name, shape) in enumerate(self.full_shapes().items()):
            g = torch.Generator().manual_seed(seed + idx)
            if name.endswith(".alpha"):
                t = 0.5 + torch.rand(shape, generator=g) * 0.2
            elif len(shape) == 1 and name.split(".")[-1] in ("norm", "norm1", "norm2"):
                t = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif len(shape) == 1:
                t = torch.randn(shape, generator=g) * 0.1
            elif name == "embed":
                t = torch.randn(shape, generator=g) / max(self.embed_scale, 1e-6)
            elif name in ("bigram", "loop.step"):
                t = torch.randn(shape, generator=g) * 0.5
            else:
                t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            out[name] = t.to(torch.bfloat16)
        return out

    def init_dummy_weights(self, seed: int = 1234):
        w = self.dummy_full_weights(seed)
        self.load_weights(w.items())
        return w
