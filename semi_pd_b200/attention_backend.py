"""Attention plug-in: the reference's `AttentionBackend` ABC
(python/sglang/srt/layers/attention/base_attn_backend.py:14-108), `RadixAttention`
(python/sglang/srt/layers/radix_attention.py:20-70) and ONE backend, `SpdAttnBackend`, in place
of FlashInferAttnBackend (layers/attention/flashinfer_backend.py:62-910).

What disappears relative to the flashinfer backend: there is no `plan()`.  The kernels read
`req_to_token`, `req_pool_indices`, `seq_lens` / `extend_*` directly on the device, pick their
KV split from the launch shape, and merge splits in-kernel — so `init_forward_metadata*` does no
host-device synchronisation and nothing has to be re-planned between CUDA-graph replays.
"""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from typing import Optional

import torch

from . import ops
from .forward_batch_info import ForwardBatch, ForwardMode


class AttentionBackend(ABC):
    """The base class of attention backends"""

    @abstractmethod
    def init_forward_metadata(self, forward_batch: ForwardBatch):
        raise NotImplementedError()

    def init_cuda_graph_state(self, max_bs: int):
        raise NotImplementedError()

    def init_forward_metadata_capture_cuda_graph(self, bs: int, num_tokens: int,
                                                 req_pool_indices: torch.Tensor,
                                                 seq_lens: torch.Tensor,
                                                 encoder_lens: Optional[torch.Tensor],
                                                 forward_mode: ForwardMode, spec_info=None):
        raise NotImplementedError()

    def init_forward_metadata_replay_cuda_graph(self, bs: int, req_pool_indices: torch.Tensor,
                                                seq_lens: torch.Tensor, seq_lens_sum: int,
                                                encoder_lens: Optional[torch.Tensor],
                                                forward_mode: ForwardMode, spec_info=None,
                                                seq_lens_cpu: Optional[torch.Tensor] = None):
        raise NotImplementedError()

    def get_cuda_graph_seq_len_fill_value(self):
        raise NotImplementedError()

    def forward(self, q, k, v, layer: "RadixAttention", forward_batch: ForwardBatch,
                save_kv_cache: bool = True):
        if forward_batch.forward_mode.is_decode():
            return self.forward_decode(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache)
        return self.forward_extend(q, k, v, layer, forward_batch, save_kv_cache=save_kv_cache)

    def forward_decode(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True):
        raise NotImplementedError()

    def forward_extend(self, q, k, v, layer, forward_batch, save_kv_cache: bool = True):
        raise NotImplementedError()


class RadixAttention:
    """The attention layer descriptor the backend receives (radix_attention.py:26-52)."""

    def __init__(self, num_heads: int, head_dim: int, scaling: float, num_kv_heads: int,
                 layer_id: int, logit_cap: float = 0.0, v_head_dim: int = -1,
                 sliding_window_size: int = -1, is_cross_attention: bool = False, prefix: str = "",
                 sinks: Optional[torch.Tensor] = None, distance_slopes: Optional[torch.Tensor] = None,
                 query_temperature: Optional[tuple] = None, general: bool = False, num_v_heads: int = 0,
                 v_slot_stride: int = 0):
        self.tp_q_head_num = num_heads
        self.tp_k_head_num = num_kv_heads
        self.tp_v_head_num = num_kv_heads
        self.head_dim = head_dim
        self.qk_head_dim = head_dim
        self.v_head_dim = v_head_dim if v_head_dim != -1 else head_dim
        self.scaling = scaling
        self.layer_id = layer_id
        self.logit_cap = logit_cap
        self.sliding_window_size = sliding_window_size or -1
        self.is_cross_attention = is_cross_attention
        # options only the general kernel (csrc/attn_general.cu) has: a learned per-head sink in the
        # softmax denominator (fp32 [heads]), a per-head slope of a linear distance bias (fp32
        # [heads]), a query temperature (coef, every): q · (1 + coef · ln(floor((pos + 1) / every) + 1)).
        # `general` routes the layer there; it is implied by any of them, by a window, and by
        # key size != value size.
        self.sinks = sinks
        self.distance_slopes = distance_slopes
        self.query_temperature = query_temperature
        # also the general kernel's: logit_cap (cap · tanh(score / cap)), value heads fewer than key heads (key head g
        # reads value head g mod num_v_heads), a slot stride of the value pool (values inside wider rows)
        self.num_v_heads = num_v_heads or num_kv_heads
        self.v_slot_stride = v_slot_stride
        self.tp_v_head_num = self.num_v_heads
        self.general = bool(general or sinks is not None or distance_slopes is not None or query_temperature
                            or self.sliding_window_size > 0 or self.v_head_dim != self.qk_head_dim)
        self.k_scale = None
        self.v_scale = None

    def forward(self, q, k, v, forward_batch: ForwardBatch, save_kv_cache: bool = True):
        if k is not None:
            assert v is not None
            k = k.view(-1, self.tp_k_head_num, self.qk_head_dim)
            v = v.view(-1, self.tp_v_head_num, self.v_head_dim)
        return forward_batch.attn_backend.forward(q, k, v, self, forward_batch, save_kv_cache)

    __call__ = forward


class SpdAttnBackend(AttentionBackend):
    """Ragged chunked-prefill attention + batched paged-decode attention in libspd."""

    def __init__(self, model_runner):
        super().__init__()
        self.device = model_runner.device
        self.num_q_heads = model_runner.model_config.num_attention_heads // model_runner.tp_size
        self.head_dim = model_runner.model_config.head_dim
        self.is_mla = getattr(model_runner.model_config, "model_type", "llama") == "deepseek_v2"
        self.mla_workspace = self.decode_workspace = None
        if getattr(model_runner.model_config, "layer_specs", None) is not None:
            # hybrid family: every layer runs the general kernel or a retention mixer, neither of
            # which needs a workspace or a host-side plan
            self.impl = "general"
            self.max_extend_len = 0
            return
        # "tc" = tcgen05 kernels (the product path, head_dim 128); "simt" exists for bring-up /
        # cross-checks and serves the head_dim-64 plumbing model (OPT-125m, BASELINE configs[0])
        self.impl = os.environ.get("SPD_ATTN_IMPL", "tc" if self.head_dim == 128 else "simt")
        self.max_extend_len = 0
        # Split-KV scratch of the decode kernel.  Captured CUDA graphs bake its address in, so it
        # is allocated exactly ONCE here and never replaced: the kernel only splits when
        # batch x kv_heads is below the SM count, i.e. for at most ceil(SMs / kv_heads) requests,
        # which bounds the scratch whatever batch size an eager step later runs with.
        if self.is_mla:
            # absorbed MLA: one latent "kv head"; the split-KV scratch of spd_attn_mla (bounded by
            # 2 x SMs query tokens, see csrc/attn_mla.cu) — allocated once, like the one below
            cfg = model_runner.model_config
            need = ops.lib.spd_attn_mla_workspace_bytes(self.num_q_heads, cfg.kv_lora_rank)
            self.mla_workspace = torch.zeros((need,), dtype=torch.uint8, device=self.device)
            self.decode_workspace = None
            return
        num_kv_heads = model_runner.model_config.get_num_kv_heads(model_runner.tp_size)
        sms = ops.device_sm_count(self.device.index or 0)
        self.split_rows = -(-sms // max(num_kv_heads, 1)) + 1
        need = ops.lib.spd_attn_decode_workspace_bytes(self.split_rows, self.num_q_heads, self.head_dim)
        self.decode_workspace = torch.zeros((need,), dtype=torch.uint8, device=self.device)

    def init_forward_metadata(self, forward_batch: ForwardBatch):
        if forward_batch.forward_mode.is_extend():
            self.max_extend_len = max(forward_batch.extend_seq_lens_cpu)

    def init_cuda_graph_state(self, max_bs: int):
        pass  # the one workspace exists since __init__ and is never reallocated

    def init_forward_metadata_capture_cuda_graph(self, bs, num_tokens, req_pool_indices, seq_lens,
                                                 encoder_lens, forward_mode, spec_info=None):
        assert forward_mode.is_decode(), "only DECODE is captured on the semi-PD path"

    def init_forward_metadata_replay_cuda_graph(self, bs, req_pool_indices, seq_lens, seq_lens_sum,
                                                encoder_lens, forward_mode, spec_info=None,
                                                seq_lens_cpu=None):
        # nothing to re-plan: the captured kernels read seq_lens / req_pool_indices from the
        # graph's static buffers
        pass

    def get_cuda_graph_seq_len_fill_value(self):
        return 1

    def _forward_general(self, q, layer: RadixAttention, forward_batch: ForwardBatch):
        """Window / sink / distance bias / query temperature / k_dim != v_dim / float32: the general
        kernel, decode and ragged extend alike, reading the batch's device-side metadata."""
        k_buf, v_buf = forward_batch.token_to_kv_pool.get_kv_buffer(layer.layer_id)
        coef, every = layer.query_temperature or (0.0, 0)
        common = dict(num_q_heads=layer.tp_q_head_num, num_kv_heads=layer.tp_k_head_num, head_dim=layer.qk_head_dim,
                      v_dim=layer.v_head_dim, sm_scale=layer.scaling, window=layer.sliding_window_size,
                      sinks=layer.sinks, slopes=layer.distance_slopes, qtemp_coef=coef, qtemp_every=every,
                      softcap=layer.logit_cap, num_v_heads=layer.num_v_heads, v_slot_stride=layer.v_slot_stride)
        r2t = forward_batch.req_to_token_pool.req_to_token
        if forward_batch.forward_mode.is_decode():
            return ops.attn_general(q, k_buf, v_buf, r2t, forward_batch.req_pool_indices,
                                    seq_lens=forward_batch.seq_lens, **common)
        return ops.attn_general(q, k_buf, v_buf, r2t, forward_batch.req_pool_indices,
                                prefix_lens=forward_batch.extend_prefix_lens, extend_lens=forward_batch.extend_seq_lens,
                                extend_start_loc=forward_batch.extend_start_loc, max_extend_len=self.max_extend_len,
                                **common)

    def forward_retention(self, q, k, v, layer, forward_batch: ForwardBatch):
        """Retention mixer (decayed linear attention) over the request's recurrent state slot;
        `layer` carries num_heads, head_dim, v_head_dim, decay (fp32 [heads]), cos_sin_cache, rotary_dim,
        k_scale and layer_id, optionally in_act ("silu": q, k, v are activated as the kernel reads them).
        → o fp32 [T, heads · v_head_dim]; the state is updated in place."""
        state = forward_batch.token_to_kv_pool.state_pool.get_state(layer.layer_id)
        common = dict(num_heads=layer.num_heads, head_dim=layer.head_dim, v_dim=layer.v_head_dim, decay=layer.decay,
                      cos_sin=layer.cos_sin_cache, rot_dims=layer.rotary_dim, k_scale=layer.k_scale,
                      in_act=getattr(layer, "in_act", None))
        if forward_batch.forward_mode.is_decode():
            return ops.retention(q, k, v, state, forward_batch.req_pool_indices, seq_lens=forward_batch.seq_lens,
                                 out_cache_loc=forward_batch.out_cache_loc, **common)
        return ops.retention(q, k, v, state, forward_batch.req_pool_indices,
                             prefix_lens=forward_batch.extend_prefix_lens, extend_lens=forward_batch.extend_seq_lens,
                             extend_start_loc=forward_batch.extend_start_loc, **common)

    def _batch_rows(self, forward_batch: ForwardBatch) -> dict:
        """The device-side description of a batch's rows that the recurrent kernels read."""
        if forward_batch.forward_mode.is_decode():
            return dict(seq_lens=forward_batch.seq_lens, out_cache_loc=forward_batch.out_cache_loc)
        return dict(prefix_lens=forward_batch.extend_prefix_lens, extend_lens=forward_batch.extend_seq_lens,
                    extend_start_loc=forward_batch.extend_start_loc)

    def forward_gated_recurrence(self, q, k, v, z, layer, forward_batch: ForwardBatch):
        """Linear-attention mixer with a per-token, per-key-channel decay over the request's state slot.
        `layer` carries num_heads, head_dim, v_head_dim, layer_id, form ("sigmoid_pow" | "double_exp"), q_scale,
        tau, z_bias and bonus (fp32 [heads · head_dim] or None).  → o fp32 [T, heads · v_head_dim]."""
        state = forward_batch.token_to_kv_pool.state_pool.get_state(layer.layer_id)
        return ops.gated_recurrence(q, k, v, z, state, forward_batch.req_pool_indices, num_heads=layer.num_heads,
                                    head_dim=layer.head_dim, v_dim=layer.v_head_dim, form=layer.form,
                                    q_scale=layer.q_scale, tau=layer.tau, z_bias=layer.z_bias, bonus=layer.bonus,
                                    **self._batch_rows(forward_batch))

    def forward_matrix_memory(self, q, k, v, zi, zf, layer, forward_batch: ForwardBatch):
        """Exponentially gated matrix memory over the request's state slot (matrix state + the layer's vector
        state, which holds the normaliser and the running maximum).  `layer` carries num_heads, head_dim,
        v_head_dim, layer_id, i_bias / f_bias (fp32 [heads] or None), gate_cap and q_scale; zi / zf [T, heads] are
        the raw gate projections.  → o fp32 [T, heads · v_head_dim]."""
        pool = forward_batch.token_to_kv_pool.state_pool
        return ops.matrix_memory(q, k, v, zi, zf, pool.get_state(layer.layer_id), pool.get_shift(layer.layer_id),
                                 forward_batch.req_pool_indices, num_heads=layer.num_heads, head_dim=layer.head_dim,
                                 v_dim=layer.v_head_dim, i_bias=layer.i_bias, f_bias=layer.f_bias, cap=layer.gate_cap,
                                 q_scale=layer.q_scale, **self._batch_rows(forward_batch))

    def forward_rotary_store(self, q, k, v, layer: RadixAttention, forward_batch: ForwardBatch, q_bias=None,
                             k_bias=None, cos_sin=None, rot_dims: int = 0):
        """Bias + partial rotation of q and k by the batch's positions, with the KV write fused: rotated keys into
        the layer's key pool, `v` (or, v None, the biased keys before the rotation) into its value pool.
        → rotated q; the attention call that follows passes save_kv_cache=False."""
        k_buf, v_buf = forward_batch.token_to_kv_pool.get_kv_buffer(layer.layer_id)
        return ops.rotary_bias_store(q, k, v, q_bias, k_bias, k_buf, v_buf, forward_batch.out_cache_loc,
                                     forward_batch.positions, cos_sin, rot_dims, layer.tp_q_head_num,
                                     layer.tp_k_head_num, layer.qk_head_dim, layer.v_head_dim)

    def forward_pair_embedding(self, table, input_ids, forward_batch: ForwardBatch, scale: float = 1.0, pair=None,
                               buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
        """Embedding rows times `scale` plus the row of a hashed (previous token, token) table; the previous token of
        a portion's first row comes from (and the portion's last token goes to) the request's slot of the state
        pool's `prev_token`.  → fp32 [T, dim]."""
        if pair is None:
            return ops.embed_pair(table, input_ids, scale)
        rows = self._batch_rows(forward_batch)
        return ops.embed_pair(table, input_ids, scale, pair=pair, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur,
                              prev_state=forward_batch.token_to_kv_pool.state_pool.prev_token,
                              req_pool_indices=forward_batch.req_pool_indices, **rows)

    def forward_rotary_segments(self, segments, forward_batch: ForwardBatch, cos_sin, dtype, paired: bool = False):
        """Bias + partial rotation by the batch's positions of up to four strided segments in one launch; segments
        made with to_pool=True are written at the batch's cache slots (ops.rotary_segment / rotary_segments)."""
        ops.rotary_segments(segments, forward_batch.positions, cos_sin, dtype, loc=forward_batch.out_cache_loc,
                            paired=paired)

    def forward_token_shift(self, h, mu, layer, forward_batch: ForwardBatch):
        """Token shift of a mixer's input: → [n_mix, T, dim] = h + (previous row − h) · mu[s]; the row before a
        request's first new one comes from (and its last row goes to) the layer's vector state slot."""
        shift = forward_batch.token_to_kv_pool.state_pool.get_shift(layer.layer_id)
        rows = self._batch_rows(forward_batch)
        if not forward_batch.forward_mode.is_decode():
            rows["max_extend_len"] = self.max_extend_len
        return ops.token_shift_mix(h, mu, shift, forward_batch.req_pool_indices, **rows)

    def forward_extend(self, q, k, v, layer: RadixAttention, forward_batch: ForwardBatch,
                       save_kv_cache: bool = True):
        pool = forward_batch.token_to_kv_pool
        if save_kv_cache:
            pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v)
        if layer.general:
            return self._forward_general(q, layer, forward_batch)
        k_buf, v_buf = pool.get_kv_buffer(layer.layer_id)
        return ops.attn_prefill(
            q, k_buf, v_buf, forward_batch.req_to_token_pool.req_to_token,
            forward_batch.req_pool_indices, forward_batch.extend_prefix_lens,
            forward_batch.extend_seq_lens, forward_batch.extend_start_loc, self.max_extend_len,
            layer.tp_q_head_num, layer.tp_k_head_num, layer.head_dim, layer.scaling, impl=self.impl)

    def forward_decode(self, q, k, v, layer: RadixAttention, forward_batch: ForwardBatch,
                       save_kv_cache: bool = True):
        pool = forward_batch.token_to_kv_pool
        if save_kv_cache:
            pool.set_kv_buffer(layer, forward_batch.out_cache_loc, k, v)
        if layer.general:
            return self._forward_general(q, layer, forward_batch)
        k_buf, v_buf = pool.get_kv_buffer(layer.layer_id)
        return ops.attn_decode(
            q, k_buf, v_buf, forward_batch.req_to_token_pool.req_to_token,
            forward_batch.req_pool_indices, forward_batch.seq_lens, layer.tp_q_head_num,
            layer.tp_k_head_num, layer.head_dim, layer.scaling, impl=self.impl,
            workspace=self.decode_workspace)

    def forward_mla(self, q_lat, layer: RadixAttention, forward_batch: ForwardBatch):
        """Absorbed MLA attention over the latent pool (DeepseekV2AttentionMLA.forward_absorb's
        attention call, models/deepseek_v2.py:684-700): q_lat [T, H * (kv_lora + rope)] →
        [T, H * kv_lora].  The latent rows of this batch are already in the pool."""
        pool = forward_batch.token_to_kv_pool
        kv = pool.get_key_buffer(layer.layer_id)
        rope = layer.head_dim - layer.v_head_dim
        common = dict(num_heads=layer.tp_q_head_num, kv_lora_rank=layer.v_head_dim, rope_dim=rope,
                      sm_scale=layer.scaling, workspace=self.mla_workspace)
        if forward_batch.forward_mode.is_decode():
            return ops.attn_mla(q_lat, kv, forward_batch.req_to_token_pool.req_to_token,
                                forward_batch.req_pool_indices, seq_lens=forward_batch.seq_lens, **common)
        return ops.attn_mla(q_lat, kv, forward_batch.req_to_token_pool.req_to_token,
                            forward_batch.req_pool_indices, prefix_lens=forward_batch.extend_prefix_lens,
                            extend_start_loc=forward_batch.extend_start_loc, **common)
