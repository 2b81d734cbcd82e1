"""Python operator surface over libspd.so.

Function names, argument meaning and error behaviour mirror the reference's `sgl_kernel` Python
API (sgl-kernel/python/sgl_kernel/elementwise.py:9-25,58-76,102-151) and the call sites in
`python/sglang/srt/layers/*`; each wrapper only unwraps `torch.Tensor`s into raw pointers and
launches on torch's current CUDA stream (as sgl-kernel/python/sgl_kernel/utils.py:21-22 does).
torch is plumbing here (device memory + streams); every computation runs in libspd.so.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib
from ._lib import SPD_EPI_NONE, SPD_EPI_SILU_MUL, check, lib

_DTYPE = {torch.bfloat16: _lib.SPD_BF16, torch.float16: _lib.SPD_F16}
# the 32-bit capable operators (hybrid model family) additionally take float32
_DTYPE_ANY = {**_DTYPE, torch.float32: _lib.SPD_F32}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPE[t.dtype]
    except KeyError:
        raise RuntimeError(f"libspd supports bfloat16/float16 tensors, got {t.dtype}") from None


def _dta(t: torch.Tensor) -> int:
    try:
        return _DTYPE_ANY[t.dtype]
    except KeyError:
        raise RuntimeError(f"libspd supports bfloat16/float16/float32 tensors here, got {t.dtype}") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "libspd ops need CUDA tensors: there is no CPU path (got a tensor on %s)" % t.device
            )


# ------------------------------------------------------------------------------------------------
# SM budget of the calling worker (set by the semi-PD engine per thread: prefill / decode partition)
# ------------------------------------------------------------------------------------------------
import threading

_tls = threading.local()


def set_sm_budget(n: int) -> None:
    """SMs the current thread's kernels may assume (0 = whole device).  Persistent kernels size
    their grids with it; the green-context stream enforces it."""
    _tls.sm_budget = int(n)


def get_sm_budget() -> int:
    return getattr(_tls, "sm_budget", 0)


# ------------------------------------------------------------------------------------------------
# elementwise
# ------------------------------------------------------------------------------------------------
def rmsnorm(input: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(input, weight)
    if out is None:
        out = torch.empty_like(input)
    d = input.shape[-1]
    x2 = input.view(-1, d) if input.is_contiguous() else input
    if x2.dim() != 2 or x2.stride(1) != 1:
        raise RuntimeError("rmsnorm: input must be 2-D with a contiguous last dimension")
    check(lib.spd_rmsnorm(out.data_ptr(), x2.data_ptr(), weight.data_ptr(), x2.shape[0], d,
                          x2.stride(0), out.view(-1, d).stride(0), float(eps), _dt(input), _stream()),
          "spd_rmsnorm")
    return out


def fused_add_rmsnorm(input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                      eps: float = 1e-6) -> None:
    _cuda(input, residual, weight)
    if not (input.is_contiguous() and residual.is_contiguous()):
        raise RuntimeError("fused_add_rmsnorm: input and residual must be contiguous")
    d = input.shape[-1]
    check(lib.spd_fused_add_rmsnorm(input.data_ptr(), residual.data_ptr(), weight.data_ptr(),
                                    input.numel() // d, d, float(eps), _dt(input), _stream()),
          "spd_fused_add_rmsnorm")


def silu_and_mul(input: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(input)
    if input.shape[-1] * input.dtype.itemsize % 16 != 0:
        raise ValueError("The pointers must be multiple of 16 bytes.")
    d = input.shape[-1] // 2
    if out is None:
        out = torch.empty(input.shape[:-1] + (d,), device=input.device, dtype=input.dtype)
    if not input.is_contiguous():
        raise RuntimeError("silu_and_mul: input must be contiguous")
    check(lib.spd_silu_and_mul(out.data_ptr(), input.data_ptr(), input.numel() // (2 * d), d,
                               _dt(input), _stream()), "spd_silu_and_mul")
    return out


def layernorm(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """torch.nn.LayerNorm over the last dimension (OPT; transformers modeling_opt.py)."""
    _cuda(input, weight, bias)
    d = input.shape[-1]
    x2 = input.view(-1, d)
    if x2.stride(1) != 1:
        raise RuntimeError("layernorm: input must have a contiguous last dimension")
    if out is None:
        out = torch.empty((x2.shape[0], d), device=input.device, dtype=input.dtype)
    check(lib.spd_layernorm(out.data_ptr(), x2.data_ptr(), weight.data_ptr(), bias.data_ptr(), x2.shape[0], d,
                            x2.stride(0), out.stride(0), float(eps), _dt(input), _stream()), "spd_layernorm")
    return out.view(input.shape)


def bias_act_residual(x: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      residual: Optional[torch.Tensor] = None, act: str = "none",
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(x + bias) + residual, act in {"none", "relu"}; x / residual contiguous."""
    _cuda(x)
    if not x.is_contiguous() or (residual is not None and not residual.is_contiguous()):
        raise RuntimeError("bias_act_residual: x and residual must be contiguous")
    d = x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    check(lib.spd_bias_act_residual(out.data_ptr(), x.data_ptr(), bias.data_ptr() if bias is not None else None,
                                    residual.data_ptr() if residual is not None else None, x.numel() // d, d,
                                    {"none": 0, "relu": 1}[act], _dt(x), _stream()), "spd_bias_act_residual")
    return out


def apply_rope_with_cos_sin_cache_inplace(positions: torch.Tensor, query: torch.Tensor,
                                          key: torch.Tensor, head_size: int,
                                          cos_sin_cache: torch.Tensor, is_neox: bool = True) -> None:
    _cuda(positions, query, key, cos_sin_cache)
    if cos_sin_cache.dtype != torch.float32:
        raise ValueError("cos_sin_cache should be float32")
    if positions.dtype != torch.int64:
        positions = positions.long()
    T = query.shape[0]
    q2, k2 = query.view(T, -1), key.view(T, -1)
    check(lib.spd_rope_inplace(q2.data_ptr(), k2.data_ptr(), cos_sin_cache.data_ptr(),
                               positions.data_ptr(), T, q2.shape[1] // head_size,
                               k2.shape[1] // head_size, head_size, cos_sin_cache.shape[1],
                               q2.stride(0), k2.stride(0), 0 if is_neox else 1, _dt(query), _stream()),
          "spd_rope_inplace")


def rope_kvwrite(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor,
                 value: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                 out_cache_loc: torch.Tensor, head_size: int, cos_sin_cache: torch.Tensor,
                 is_neox: bool = True) -> None:
    """RoPE(q, k) in place + k_pool[loc] = k, v_pool[loc] = v in one launch."""
    _cuda(positions, query, key, value, k_pool, v_pool, out_cache_loc, cos_sin_cache)
    if cos_sin_cache.dtype != torch.float32:
        raise ValueError("cos_sin_cache should be float32")
    if positions.dtype != torch.int64 or out_cache_loc.dtype != torch.int64:
        raise RuntimeError("rope_kvwrite: positions and out_cache_loc must be int64")
    T = query.shape[0]
    q2, k2, v2 = query.view(T, -1), key.view(T, -1), value.view(T, -1)
    check(lib.spd_rope_kvwrite(q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), k_pool.data_ptr(),
                               v_pool.data_ptr(), cos_sin_cache.data_ptr(), positions.data_ptr(),
                               out_cache_loc.data_ptr(), T, q2.shape[1] // head_size,
                               k2.shape[1] // head_size, head_size, cos_sin_cache.shape[1],
                               q2.stride(0), k2.stride(0), v2.stride(0), 0 if is_neox else 1,
                               _dt(query), _stream()), "spd_rope_kvwrite")


def kv_write(key: torch.Tensor, value: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
             loc: torch.Tensor) -> None:
    _cuda(key, value, k_pool, v_pool, loc)
    T = key.shape[0]
    if T == 0:
        return
    k2, v2 = key.view(T, -1), value.view(T, -1)
    if loc.dtype != torch.int64:
        loc = loc.long()
    check(lib.spd_kv_write(k2.data_ptr(), v2.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                           loc.data_ptr(), T, k2.shape[1], k2.stride(0), v2.stride(0), _dt(key),
                           _stream()), "spd_kv_write")


def gather_rows(table: torch.Tensor, idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(table, idx)
    if idx.dtype != torch.int64:
        idx = idx.long()
    n = idx.numel()
    if out is None:
        out = torch.empty((n, table.shape[1]), device=table.device, dtype=table.dtype)
    check(lib.spd_gather_rows(out.data_ptr(), table.data_ptr(), idx.data_ptr(), n, table.shape[1],
                              table.shape[0], _dt(table), _stream()), "spd_gather_rows")
    return out


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise RuntimeError("argmax: logits must be fp32 [B, V] with a contiguous last dimension")
    if out is None:
        out = torch.empty((logits.shape[0],), device=logits.device, dtype=torch.int32)
    check(lib.spd_argmax_f32(out.data_ptr(), logits.data_ptr(), logits.shape[0], logits.shape[1],
                             logits.stride(0), _stream()), "spd_argmax_f32")
    return out


def argmax_partial(logits: torch.Tensor, index_offset: int) -> torch.Tensor:
    """[B, 16] uint8 rows {f32 max, i32 index_offset + argmax, 0, 0} of one vocab shard."""
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise RuntimeError("argmax_partial: logits must be fp32 [B, V] with a contiguous last dimension")
    out = torch.empty((logits.shape[0], 16), device=logits.device, dtype=torch.uint8)
    check(lib.spd_argmax_partial_f32(out.data_ptr(), logits.data_ptr(), logits.shape[0], logits.shape[1],
                                     logits.stride(0), int(index_offset), _stream()),
          "spd_argmax_partial_f32")
    return out


def argmax_merge(pairs: torch.Tensor) -> torch.Tensor:
    """pairs [parts, B, 16] uint8 (argmax_partial rows of every shard) → ids [B] int32."""
    _cuda(pairs)
    parts, B = pairs.shape[0], pairs.shape[1]
    out = torch.empty((B,), device=pairs.device, dtype=torch.int32)
    check(lib.spd_argmax_merge(out.data_ptr(), pairs.data_ptr(), parts, B, _stream()), "spd_argmax_merge")
    return out


# ------------------------------------------------------------------------------------------------
# metadata
# ------------------------------------------------------------------------------------------------
def compute_positions(extend_prefix_lens: torch.Tensor, extend_seq_lens: torch.Tensor,
                      extend_num_tokens: int, want_token_req: bool = False):
    """(positions i64 [T], extend_start_loc i32 [bs][, token_req i32 [T]]) —
    compute_position_triton's contract (forward_batch_info.py:393-419)."""
    _cuda(extend_prefix_lens, extend_seq_lens)
    bs = extend_seq_lens.shape[0]
    dev = extend_seq_lens.device
    positions = torch.empty((extend_num_tokens,), dtype=torch.int64, device=dev)
    start = torch.empty((bs,), dtype=torch.int32, device=dev)
    treq = torch.empty((extend_num_tokens,), dtype=torch.int32, device=dev) if want_token_req else None
    has_prefix = extend_prefix_lens is not None and extend_prefix_lens.shape[0] == bs
    check(lib.spd_compute_positions(positions.data_ptr(), start.data_ptr(),
                                    treq.data_ptr() if treq is not None else None,
                                    extend_prefix_lens.data_ptr() if has_prefix else None,
                                    extend_seq_lens.data_ptr(), bs, _stream()),
          "spd_compute_positions")
    return (positions, start, treq) if want_token_req else (positions, start)


def clamp_position(seq_lens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(seq_lens)
    if seq_lens.dtype != torch.int64:
        seq_lens = seq_lens.long()
    if out is None:
        out = torch.empty_like(seq_lens)
    check(lib.spd_decode_positions(out.data_ptr(), seq_lens.data_ptr(), seq_lens.numel(), _stream()),
          "spd_decode_positions")
    return out


def create_kv_indices(req_to_token: torch.Tensor, req_pool_indices: torch.Tensor,
                      page_kernel_lens: torch.Tensor, kv_indptr: torch.Tensor,
                      kv_start_idx: Optional[torch.Tensor], kv_indices: torch.Tensor) -> None:
    """create_flashinfer_kv_indices_triton's contract (S/layers/attention/utils.py:5-39)."""
    _cuda(req_to_token, req_pool_indices, page_kernel_lens, kv_indptr, kv_indices)
    if req_pool_indices.dtype != torch.int64:
        req_pool_indices = req_pool_indices.long()
    if page_kernel_lens.dtype != torch.int32:
        page_kernel_lens = page_kernel_lens.int()
    check(lib.spd_build_kv_indices(kv_indices.data_ptr(), req_to_token.data_ptr(),
                                   req_pool_indices.data_ptr(), page_kernel_lens.data_ptr(),
                                   kv_indptr.data_ptr(),
                                   kv_start_idx.data_ptr() if kv_start_idx is not None else None,
                                   req_pool_indices.numel(), req_to_token.stride(0), _stream()),
          "spd_build_kv_indices")


def write_req_to_token_pool(req_to_token: torch.Tensor, req_pool_indices: torch.Tensor,
                            pre_lens: torch.Tensor, seq_lens: torch.Tensor,
                            extend_lens: torch.Tensor, out_cache_loc: torch.Tensor) -> None:
    """write_req_to_token_pool_triton's contract (S/managers/schedule_batch.py:1446-1480)."""
    _cuda(req_to_token, req_pool_indices, pre_lens, seq_lens, extend_lens, out_cache_loc)
    args = [t if t.dtype == torch.int64 else t.long()
            for t in (req_pool_indices, pre_lens, seq_lens, extend_lens, out_cache_loc)]
    check(lib.spd_write_req_to_token(req_to_token.data_ptr(), *[a.data_ptr() for a in args],
                                     args[0].numel(), req_to_token.stride(0), _stream()),
          "spd_write_req_to_token")


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------
_gemm_ws = {}


def _gemm_workspace(device: torch.device) -> torch.Tensor:
    """Split-K scratch, one per (device, stream) so the prefill and decode workers never share it."""
    key = (device.index, _stream())
    ws = _gemm_ws.get(key)
    if ws is None:
        ws = torch.zeros((lib.spd_gemm_workspace_bytes(),), dtype=torch.uint8, device=device)
        _gemm_ws[key] = ws
    return ws


def linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_f32: bool = False, epilogue: int = SPD_EPI_NONE, exact_f32: bool = False) -> torch.Tensor:
    """F.linear(x, weight) — x [M, K], weight [N, K] (or [2N, K] with SPD_EPI_SILU_MUL).  out_f32:
    the 16-bit product as fp32 (`.float()` of a 16-bit matmul); with exact_f32 the fp32 accumulator."""
    _cuda(x, weight)
    if x.dim() != 2 or weight.dim() != 2 or x.stride(1) != 1 or weight.stride(1) != 1:
        raise RuntimeError("linear: x and weight must be 2-D with contiguous last dimension")
    if x.dtype != weight.dtype:
        raise RuntimeError(f"linear: dtype mismatch {x.dtype} vs {weight.dtype}")
    M, K = x.shape
    N = weight.shape[0] // (2 if epilogue == SPD_EPI_SILU_MUL else 1)
    if weight.shape[1] != K:
        raise RuntimeError(f"linear: shape mismatch x{tuple(x.shape)} w{tuple(weight.shape)}")
    if out is None:
        out = torch.empty((M, N), device=x.device, dtype=torch.float32 if out_f32 else x.dtype)
    ws = _gemm_workspace(x.device)
    check(lib.spd_gemm(out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0),
                       weight.stride(0), out.stride(0), _dt(x), (2 if exact_f32 else 1) if out_f32 else 0, epilogue,
                       ws.data_ptr(), ws.numel(), get_sm_budget(), _stream()), "spd_gemm")
    return out


def linear_block_diag(x: torch.Tensor, weight: torch.Tensor, num_groups: int, k: int, n: int,
                      x_group_stride: int, out: Optional[torch.Tensor] = None,
                      out_group_stride: int = 0) -> torch.Tensor:
    """out[:, g*n:(g+1)*n] = x[:, g*x_group_stride : +k] @ weight[g*n:(g+1)*n, :k].T — the per-head
    products of the absorbed MLA form (torch.bmm(q_nope, w_kc), torch.bmm(attn_out, w_vc)) as one launch."""
    _cuda(x, weight)
    if x.dim() != 2 or weight.dim() != 2 or x.stride(1) != 1 or weight.stride(1) != 1 or x.dtype != weight.dtype:
        raise RuntimeError("linear_block_diag: x and weight must be 2-D, contiguous rows, same dtype")
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, num_groups * n), device=x.device, dtype=x.dtype)
    check(lib.spd_gemm_grouped(out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, n, k, x.stride(0),
                               weight.stride(0), out.stride(0), num_groups, None, x_group_stride, x.shape[1],
                               out_group_stride, 0, _dt(x), SPD_EPI_NONE, get_sm_budget(), _stream()),
          "spd_gemm_grouped")
    return out


def linear_grouped_rows(x_sorted: torch.Tensor, weight: torch.Tensor, tile_group: torch.Tensor, num_groups: int,
                        n: int, epilogue: int = SPD_EPI_NONE, k_concat: bool = False) -> torch.Tensor:
    """Rows of x_sorted are grouped by expert in 128-row tiles; weight = the experts' [n (or 2n), K]
    matrices stacked along the rows — or, k_concat, [n, E * K] concatenated along K.  → [rows, n]."""
    _cuda(x_sorted, weight, tile_group)
    M, K = x_sorted.shape
    out = torch.empty((M, n), device=x_sorted.device, dtype=x_sorted.dtype)
    check(lib.spd_gemm_grouped(out.data_ptr(), x_sorted.data_ptr(), weight.data_ptr(), M, n, K, x_sorted.stride(0),
                               weight.stride(0), out.stride(0), num_groups, tile_group.data_ptr(), 0, K, 0,
                               K if k_concat else 0, _dt(x_sorted), epilogue, get_sm_budget(), _stream()),
          "spd_gemm_grouped")
    return out


def moe_route(logits: torch.Tensor, top_k: int, scale: float = 1.0, renormalize: bool = False):
    """→ (topk_ids int32 [T, k], topk_weights fp32 [T, k])."""
    _cuda(logits)
    T, E = logits.shape
    ids = torch.empty((T, top_k), device=logits.device, dtype=torch.int32)
    w = torch.empty((T, top_k), device=logits.device, dtype=torch.float32)
    check(lib.spd_moe_route(ids.data_ptr(), w.data_ptr(), logits.contiguous().data_ptr(), T, E, top_k, float(scale),
                            1 if renormalize else 0, _dt(logits), _stream()), "spd_moe_route")
    return ids, w


def moe_align(topk_ids: torch.Tensor, num_experts: int):
    """→ (row_token [R], inv_pos [T*k], tile_group [R/128]) with R = spd_moe_align_rows()."""
    _cuda(topk_ids)
    T, k = topk_ids.shape
    R = lib.spd_moe_align_rows(T, k, num_experts)
    dev = topk_ids.device
    row_token = torch.empty((R,), device=dev, dtype=torch.int32)
    inv_pos = torch.empty((T * k,), device=dev, dtype=torch.int32)
    tile_group = torch.empty((R // 128,), device=dev, dtype=torch.int32)
    check(lib.spd_moe_align(row_token.data_ptr(), inv_pos.data_ptr(), tile_group.data_ptr(), topk_ids.data_ptr(),
                            T, k, num_experts, R, _stream()), "spd_moe_align")
    return row_token, inv_pos, tile_group


def moe_gather(x: torch.Tensor, row_token: torch.Tensor) -> torch.Tensor:
    _cuda(x, row_token)
    out = torch.empty((row_token.numel(), x.shape[1]), device=x.device, dtype=x.dtype)
    check(lib.spd_moe_gather(out.data_ptr(), x.data_ptr(), row_token.data_ptr(), row_token.numel(), x.shape[1],
                             x.stride(0), _dt(x), _stream()), "spd_moe_gather")
    return out


def moe_combine(y: torch.Tensor, inv_pos: torch.Tensor, topk_w: torch.Tensor,
                shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    _cuda(y, inv_pos, topk_w)
    T, k = topk_w.shape
    out = torch.empty((T, y.shape[1]), device=y.device, dtype=y.dtype)
    check(lib.spd_moe_combine(out.data_ptr(), y.data_ptr(), shared.data_ptr() if shared is not None else None,
                              inv_pos.data_ptr(), topk_w.data_ptr(), T, k, y.shape[1], _dt(y), _stream()),
          "spd_moe_combine")
    return out


def moe_dense_act(gate_up: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, num_experts: int,
                  inter: int) -> torch.Tensor:
    _cuda(gate_up, topk_ids, topk_w)
    T, k = topk_ids.shape
    out = torch.empty((T, num_experts * inter), device=gate_up.device, dtype=gate_up.dtype)
    check(lib.spd_moe_dense_act(out.data_ptr(), gate_up.data_ptr(), topk_ids.data_ptr(), topk_w.data_ptr(), T, k,
                                num_experts, inter, _dt(gate_up), _stream()), "spd_moe_dense_act")
    return out


def kv_write_single(rows: torch.Tensor, pool: torch.Tensor, loc: torch.Tensor) -> None:
    """pool[loc[t]] = rows[t] — MLATokenToKVPool.set_kv_buffer (one latent buffer per layer)."""
    _cuda(rows, pool, loc)
    T = rows.shape[0]
    if T == 0:
        return
    r2 = rows.view(T, -1)
    if loc.dtype != torch.int64:
        loc = loc.long()
    check(lib.spd_kv_write(r2.data_ptr(), None, pool.data_ptr(), None, loc.data_ptr(), T, r2.shape[1],
                           r2.stride(0), 0, _dt(rows), _stream()), "spd_kv_write")


def attn_mla(q: torch.Tensor, kv_pool: torch.Tensor, req_to_token, req_pool_indices, num_heads: int,
             kv_lora_rank: int, rope_dim: int, sm_scale: float, workspace: torch.Tensor, seq_lens=None,
             prefix_lens=None, extend_start_loc=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Absorbed MLA attention: decode (seq_lens) or ragged extend (prefix_lens + extend_start_loc).
    q [T, H * (kv_lora + rope)] → out [T, H * kv_lora]."""
    _cuda(q, kv_pool, req_to_token, req_pool_indices)
    T = q.shape[0]
    q2 = q.view(T, -1)
    if out is None:
        out = torch.empty((T, num_heads * kv_lora_rank), device=q.device, dtype=q.dtype)
    check(lib.spd_attn_mla(out.data_ptr(), q2.data_ptr(), kv_pool.data_ptr(), req_to_token.data_ptr(),
                           req_pool_indices.data_ptr(), seq_lens.data_ptr() if seq_lens is not None else None,
                           prefix_lens.data_ptr() if prefix_lens is not None else None,
                           extend_start_loc.data_ptr() if extend_start_loc is not None else None,
                           req_pool_indices.numel(), T, num_heads, kv_lora_rank, rope_dim, q2.stride(0),
                           out.stride(0), req_to_token.stride(0), float(sm_scale), _dt(q), workspace.data_ptr(),
                           workspace.numel(), get_sm_budget(), _stream()), "spd_attn_mla")
    return out


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
_attn_ws = {}


def _attn_workspace(device, batch: int, hq: int, d: int) -> torch.Tensor:
    need = lib.spd_attn_decode_workspace_bytes(batch, hq, d)
    key = (device.index, _stream())
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros((max(need, 1 << 20),), dtype=torch.uint8, device=device)
        _attn_ws[key] = ws
    return ws


def attn_decode(q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens, num_q_heads,
                num_kv_heads, head_dim, sm_scale, out=None, impl: str = "tc", workspace=None):
    _cuda(q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens)
    B = q.shape[0]
    q2 = q.view(B, -1)
    if out is None:
        out = torch.empty_like(q2)
    if req_pool_indices.dtype != torch.int64 or seq_lens.dtype != torch.int64:
        raise RuntimeError("attn_decode: req_pool_indices and seq_lens must be int64")
    ws = workspace if workspace is not None else _attn_workspace(q.device, B, num_q_heads, head_dim)
    if impl == "tc":
        check(lib.spd_attn_decode_paged(out.data_ptr(), q2.data_ptr(), k_pool.data_ptr(),
                                        v_pool.data_ptr(), req_to_token.data_ptr(),
                                        req_pool_indices.data_ptr(), seq_lens.data_ptr(), B,
                                        num_q_heads, num_kv_heads, head_dim, q2.stride(0),
                                        out.stride(0), req_to_token.stride(0), float(sm_scale),
                                        _dt(q), ws.data_ptr(), ws.numel(), get_sm_budget(), _stream()),
              "spd_attn_decode_paged")
    elif impl == "simt":
        check(lib.spd_attn_decode_simt(out.data_ptr(), q2.data_ptr(), k_pool.data_ptr(),
                                       v_pool.data_ptr(), req_to_token.data_ptr(),
                                       req_pool_indices.data_ptr(), seq_lens.data_ptr(), B,
                                       num_q_heads, num_kv_heads, head_dim, q2.stride(0),
                                       out.stride(0), req_to_token.stride(0), float(sm_scale),
                                       _dt(q), ws.data_ptr(), ws.numel(), _stream()),
              "spd_attn_decode_simt")
    else:
        raise ValueError(impl)
    return out


def attn_prefill(q, k_pool, v_pool, req_to_token, req_pool_indices, prefix_lens, extend_lens,
                 extend_start_loc, max_extend_len, num_q_heads, num_kv_heads, head_dim, sm_scale,
                 out=None, impl: str = "tc"):
    _cuda(q, k_pool, v_pool, req_to_token, req_pool_indices, prefix_lens, extend_lens, extend_start_loc)
    T = q.shape[0]
    q2 = q.view(T, -1)
    if out is None:
        out = torch.empty_like(q2)
    if req_pool_indices.dtype != torch.int64:
        raise RuntimeError("attn_prefill: req_pool_indices must be int64")
    for t in (prefix_lens, extend_lens, extend_start_loc):
        if t.dtype != torch.int32:
            raise RuntimeError("attn_prefill: prefix_lens / extend_lens / extend_start_loc must be int32")
    args = (out.data_ptr(), q2.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
            req_to_token.data_ptr(), req_pool_indices.data_ptr(), prefix_lens.data_ptr(),
            extend_lens.data_ptr(), extend_start_loc.data_ptr(), req_pool_indices.numel(), T,
            int(max_extend_len), num_q_heads, num_kv_heads, head_dim, q2.stride(0), out.stride(0),
            req_to_token.stride(0), float(sm_scale), _dt(q))
    if impl == "tc":
        check(lib.spd_attn_prefill_ragged(*args, get_sm_budget(), _stream()), "spd_attn_prefill_tc")
    else:
        check(lib.spd_attn_prefill_simt(*args, _stream()), "spd_attn_prefill_simt")
    return out


# ------------------------------------------------------------------------------------------------
# 32-bit capable operators (hybrid model family: fp32 residual stream, windowed attention with
# sinks, retention, sigmoid-routed experts that weight their input)
# ------------------------------------------------------------------------------------------------
def _ptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


def embed_f32(table: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """fp32 [n, dim] rows of a 16/32-bit embedding table (the start of an fp32 residual stream)."""
    _cuda(table, idx)
    if idx.dtype != torch.int64:
        idx = idx.long()
    out = torch.empty((idx.numel(), table.shape[1]), device=table.device, dtype=torch.float32)
    check(lib.spd_embed_f32(out.data_ptr(), table.data_ptr(), idx.data_ptr(), idx.numel(), table.shape[1],
                            table.shape[0], _dta(table), _stream()), "spd_embed_f32")
    return out


def residual_rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, a: Optional[torch.Tensor] = None,
                     b: Optional[torch.Tensor] = None, weight_offset: float = 0.0,
                     out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x (fp32, in place) += a (+ b); → x / sqrt(mean(x²) + eps) · (weight_offset + weight) in the
    weight's dtype (None when weight is None: residual add only)."""
    _cuda(x, weight, a, b)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise RuntimeError("residual_rmsnorm: the residual stream is contiguous fp32")
    for t in (a, b):
        if t is not None and (not t.is_contiguous() or t.shape != x.shape):
            raise RuntimeError("residual_rmsnorm: a / b must match x and be contiguous")
    ref = weight if weight is not None else a
    if a is not None and weight is not None and a.dtype != weight.dtype:
        raise RuntimeError("residual_rmsnorm: a / b and weight must share a dtype")
    d = x.shape[-1]
    out = torch.empty(x.shape, device=x.device, dtype=ref.dtype) if weight is not None else None
    check(lib.spd_residual_rmsnorm(_ptr(out), x.data_ptr(), _ptr(a), _ptr(b), _ptr(weight), x.numel() // d, d,
                                   float(eps), float(weight_offset), _dta(ref), _stream()), "spd_residual_rmsnorm")
    return out


def act_and_mul(x: torch.Tensor, act: str = "silu", limit: float = 0.0, slope: float = 1.0) -> torch.Tensor:
    """act(x[:, :I]) · x[:, I:], act in {"silu", "gelu_tanh"}; any of the three dtypes.  act "clamped_swish":
    with g = min(x[:, :I], limit) and u = clamp(x[:, I:], ±limit), g · sigmoid(slope · g) · (u + 1)."""
    _cuda(x)
    if x.dim() != 2 or not x.is_contiguous():
        raise RuntimeError("act_and_mul: x must be contiguous [rows, 2 I]")
    inter = x.shape[1] // 2
    out = torch.empty((x.shape[0], inter), device=x.device, dtype=x.dtype)
    check(lib.spd_act_and_mul(out.data_ptr(), x.data_ptr(), x.shape[0], inter,
                              {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}[act], float(limit), float(slope),
                              _dta(x), _stream()), "spd_act_and_mul")
    return out


def headnorm_gate(o: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int, eps: float,
                  weight: Optional[torch.Tensor] = None, gate_act: str = "silu") -> torch.Tensor:
    """o fp32 [T, heads·vdim] → per-head o / rms(o) [· weight] · act(gate), act SiLU or sigmoid, in gate's dtype.
    weight: [vdim] (shared by the heads) or [heads·vdim], in gate's dtype.  heads = 1 norms the whole row."""
    _cuda(o, gate, weight)
    w_stride = 0
    if weight is not None:
        if weight.dtype != gate.dtype or not weight.is_contiguous() or weight.numel() not in (vdim, heads * vdim):
            raise RuntimeError("headnorm_gate: weight is [vdim] or [heads * vdim] in the gate's dtype")
        w_stride = vdim if weight.numel() == heads * vdim and heads > 1 else 0
    if o.dtype != torch.float32 or not o.is_contiguous() or gate.stride(1) != 1:
        raise RuntimeError("headnorm_gate: o is contiguous fp32, gate has contiguous rows")
    T = o.shape[0]
    out = torch.empty((T, heads * vdim), device=o.device, dtype=gate.dtype)
    check(lib.spd_headnorm_gate(out.data_ptr(), o.data_ptr(), gate.data_ptr(), T, heads, vdim, gate.stride(0),
                                float(eps), _ptr(weight), w_stride, {"silu": 0, "sigmoid": 1}[gate_act], _dta(gate),
                                _stream()), "spd_headnorm_gate")
    return out


def linear_simt(x: torch.Tensor, weight: torch.Tensor, out_f32: bool = False,
                tile_group: Optional[torch.Tensor] = None, group_rows: int = 0, n: Optional[int] = None) -> torch.Tensor:
    """F.linear on the CUDA cores (any shape / dtype, fp32 accumulation in ascending k).  With
    tile_group, rows of x come in expert-aligned 128-row tiles and rows [g·group_rows, +n) of weight
    multiply group g's tiles."""
    _cuda(x, weight, tile_group)
    if x.dim() != 2 or weight.dim() != 2 or x.stride(1) != 1 or weight.stride(1) != 1 or x.dtype != weight.dtype:
        raise RuntimeError("linear_simt: x and weight must be 2-D, contiguous rows, same dtype")
    M, K = x.shape
    N = weight.shape[0] if n is None else n
    out = torch.empty((M, N), device=x.device, dtype=torch.float32 if out_f32 else x.dtype)
    check(lib.spd_linear_simt(out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, N, K, x.stride(0), weight.stride(0),
                              out.stride(0), _ptr(tile_group), int(group_rows), _dta(x), 1 if out_f32 else 0, _stream()),
          "spd_linear_simt")
    return out


def _tc_gemm_ok(x: torch.Tensor, weight: torch.Tensor, n: int) -> bool:
    """Shapes / dtypes the tcgen05 GEMMs take (16-bit, 16-byte rows and pointers)."""
    return (x.dtype in _DTYPE and x.shape[1] % 8 == 0 and n % 8 == 0 and x.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_any(x: torch.Tensor, weight: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    """F.linear for the hybrid family: the tcgen05 GEMMs where they apply (16-bit, aligned shapes),
    the CUDA-core GEMM otherwise (float32 models, odd sizes)."""
    if _tc_gemm_ok(x, weight, weight.shape[0]) and os.environ.get("SPD_HYBRID_GEMM", "tc") == "tc":
        return linear(x, weight, out_f32=out_f32, exact_f32=True)
    return linear_simt(x, weight, out_f32=out_f32)


def linear_grouped_any(x_sorted: torch.Tensor, weight: torch.Tensor, tile_group: torch.Tensor, num_groups: int,
                       n: int, silu_mul: bool = False) -> torch.Tensor:
    """Expert-grouped F.linear over 128-row tiles; weight = the experts' [n, K] matrices stacked.
    silu_mul: each expert's block is [gate; up] (2n rows) and the result is silu(gate) * up [rows, n] —
    the tensor-core GEMM applies it to its fp32 accumulators in the epilogue, the CUDA-core route runs
    the activation kernel on the product."""
    if (_tc_gemm_ok(x_sorted, weight, n) and x_sorted.shape[1] % 64 == 0
            and os.environ.get("SPD_HYBRID_GEMM", "tc") == "tc"):
        if silu_mul and os.environ.get("SPD_HYBRID_FUSED_ACT", "1") != "1":
            return act_and_mul(linear_grouped_rows(x_sorted, weight, tile_group, num_groups, 2 * n), "silu")
        return linear_grouped_rows(x_sorted, weight, tile_group, num_groups, n,
                                   epilogue=SPD_EPI_SILU_MUL if silu_mul else SPD_EPI_NONE)
    rows = 2 * n if silu_mul else n
    y = linear_simt(x_sorted, weight, tile_group=tile_group, group_rows=rows, n=rows)
    return act_and_mul(y, "silu") if silu_mul else y


def linear_silu_mul_any(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """silu(x W_gate^T) * (x W_up^T) for weight = [W_gate; W_up]: one tensor-core GEMM with the
    activation in its epilogue for prefill-sized 16-bit batches (the Llama MLP's route), GEMM +
    activation kernel otherwise."""
    n = weight.shape[0] // 2
    if (x.shape[0] >= 257 and _tc_gemm_ok(x, weight, n) and os.environ.get("SPD_HYBRID_GEMM", "tc") == "tc"
            and os.environ.get("SPD_HYBRID_FUSED_ACT", "1") == "1"):
        return linear(x, weight, epilogue=SPD_EPI_SILU_MUL)
    return act_and_mul(linear_any(x, weight), "silu")


def moe_route_scores(logits: torch.Tensor, num_experts: int, top_k: int, score_func: str = "sigmoid",
                     renormalize: bool = False, scale: float = 1.0, correction: Optional[torch.Tensor] = None,
                     num_groups: int = 1, keep_groups: int = 1):
    """fp32 logits [T, >= E] (row stride free) → (topk_ids int32 [T, k], topk_weights fp32 [T, k]).
    correction (fp32 [E]) biases the selection, never the weights; with num_groups > 1 the experts are cut into
    equal runs, each run is ranked by its top-2 biased scores added together, and selection is restricted to the
    keep_groups highest-ranked runs."""
    _cuda(logits, correction)
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != num_experts):
        raise RuntimeError("moe_route_scores: correction is fp32 [experts]")
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise RuntimeError("moe_route_scores: logits are fp32 with contiguous rows")
    T = logits.shape[0]
    ids = torch.empty((T, top_k), device=logits.device, dtype=torch.int32)
    w = torch.empty((T, top_k), device=logits.device, dtype=torch.float32)
    check(lib.spd_moe_route_scores(ids.data_ptr(), w.data_ptr(), logits.data_ptr(), logits.stride(0), T, num_experts,
                                   top_k, {"softmax": 0, "sigmoid": 1}[score_func], 1 if renormalize else 0,
                                   float(scale), _ptr(correction), int(num_groups), int(keep_groups), _stream()),
          "spd_moe_route_scores")
    return ids, w


def moe_gather_scaled(x: torch.Tensor, row_token: torch.Tensor, inv_pos: torch.Tensor,
                      topk_w: Optional[torch.Tensor]) -> torch.Tensor:
    """Expert-sorted rows of x, each multiplied by its routing weight (experts that weight their input)."""
    _cuda(x, row_token, inv_pos, topk_w)
    k = topk_w.shape[1] if topk_w is not None else inv_pos.numel() // max(x.shape[0], 1)
    out = torch.empty((row_token.numel(), x.shape[1]), device=x.device, dtype=x.dtype)
    check(lib.spd_moe_gather_scaled(out.data_ptr(), x.data_ptr(), row_token.data_ptr(), inv_pos.data_ptr(),
                                    _ptr(topk_w), row_token.numel(), k, x.shape[1], x.stride(0), _dta(x), _stream()),
          "spd_moe_gather_scaled")
    return out


def moe_combine_gated(y: torch.Tensor, inv_pos: torch.Tensor, tokens: int, top_k: int,
                      topk_w: Optional[torch.Tensor] = None, shared: Optional[torch.Tensor] = None,
                      shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Σ_j [w_j] y[row(t, j)] + [sigmoid(shared_gate[t])] shared[t]; shared_gate is an fp32 column
    (any row stride)."""
    _cuda(y, inv_pos, topk_w, shared, shared_gate)
    out = torch.empty((tokens, y.shape[1]), device=y.device, dtype=y.dtype)
    gs = shared_gate.stride(0) if shared_gate is not None else 0
    if shared_gate is not None and shared_gate.dtype != torch.float32:
        raise RuntimeError("moe_combine_gated: the shared gate logits are fp32")
    check(lib.spd_moe_combine_gated(out.data_ptr(), y.data_ptr(), inv_pos.data_ptr(), _ptr(topk_w), _ptr(shared),
                                    _ptr(shared_gate), gs, tokens, top_k, y.shape[1], _dta(y), _stream()),
          "spd_moe_combine_gated")
    return out


def residual_rmsnorm2(x: torch.Tensor, weight: torch.Tensor, weight2: Optional[torch.Tensor], eps: float,
                      a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None, weight_offset: float = 0.0):
    """x (fp32, in place) += a (+ b); → (norm(x) · (off + weight), norm(x) · (off + weight2) or None): one
    pass over the row for layers whose two sublayers have a norm weight each."""
    _cuda(x, weight, weight2, a, b)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise RuntimeError("residual_rmsnorm2: the residual stream is contiguous fp32")
    for t in (a, b):
        if t is not None and (not t.is_contiguous() or t.shape != x.shape or t.dtype != weight.dtype):
            raise RuntimeError("residual_rmsnorm2: a / b must match x, be contiguous and share the weight's dtype")
    if weight2 is not None and weight2.dtype != weight.dtype:
        raise RuntimeError("residual_rmsnorm2: the two weights share a dtype")
    d = x.shape[-1]
    out = torch.empty(x.shape, device=x.device, dtype=weight.dtype)
    out2 = torch.empty_like(out) if weight2 is not None else None
    check(lib.spd_residual_rmsnorm2(out.data_ptr(), _ptr(out2), x.data_ptr(), _ptr(a), _ptr(b), weight.data_ptr(),
                                    _ptr(weight2), x.numel() // d, d, float(eps), float(weight_offset), _dta(weight),
                                    _stream()), "spd_residual_rmsnorm2")
    return out, out2


def linear_block_diag_any(x: torch.Tensor, weight: torch.Tensor, num_groups: int, k: int, n: int,
                          x_group_stride: Optional[int] = None, out: Optional[torch.Tensor] = None,
                          out_group_stride: Optional[int] = None) -> torch.Tensor:
    """out[:, g n : (g + 1) n] = x[:, g k : (g + 1) k] @ weight[g n : (g + 1) n, :k].T for g < num_groups — the
    per-head products of an absorbed latent attention; tensor cores where the shapes tile, CUDA cores otherwise.
    x_group_stride / out_group_stride (default k / n): columns between two groups of x / out, for heads that carry
    more than the multiplied slice; `out` is then a caller's [M, >= num_groups · out_group_stride] buffer."""
    _cuda(x, weight, out)
    if x.dim() != 2 or weight.dim() != 2 or x.stride(1) != 1 or weight.stride(1) != 1 or x.dtype != weight.dtype:
        raise RuntimeError("linear_block_diag_any: x and weight must be 2-D, contiguous rows, same dtype")
    xg = k if x_group_stride is None else int(x_group_stride)
    og = n if out_group_stride is None else int(out_group_stride)
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, num_groups * og), device=x.device, dtype=x.dtype)
    elif out.dtype != x.dtype or out.stride(1) != 1 or out.shape[0] != M:
        raise RuntimeError("linear_block_diag_any: out is [M, ...] with contiguous rows in x's dtype")
    if (x.dtype in _DTYPE and n % 128 == 0 and k % 64 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and xg % 8 == 0 and og % 8 == 0 and out.stride(0) % 8 == 0
            and out.data_ptr() % 16 == 0 and os.environ.get("SPD_HYBRID_GEMM", "tc") == "tc"):
        return linear_block_diag(x, weight, num_groups, k, n, x_group_stride=xg, out=out, out_group_stride=og)
    check(lib.spd_linear_simt_block_diag(out.data_ptr(), x.data_ptr(), weight.data_ptr(), M, n, k, x.stride(0),
                                         weight.stride(0), out.stride(0), num_groups, xg, og, _dta(x), _stream()),
          "spd_linear_simt_block_diag")
    return out


def gated_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, state: torch.Tensor,
                     req_pool_indices, num_heads: int, head_dim: int, v_dim: int, form: str, q_scale: float = 1.0,
                     tau: float = 1.0, z_bias: Optional[torch.Tensor] = None, bonus: Optional[torch.Tensor] = None,
                     seq_lens=None, out_cache_loc=None, prefix_lens=None, extend_lens=None,
                     extend_start_loc=None) -> torch.Tensor:
    """Linear attention with a per-token decay per key channel over the per-request state (updated in place).
    form "sigmoid_pow": w = sigmoid(z + z_bias)^(1/tau), o_t reads the updated state; form "double_exp":
    w = exp(-exp(z + z_bias)), o_t reads the old state plus bonus · k_t v_tᵀ.  q / k / z [T, H·head_dim],
    v [T, H·v_dim] (row-strided views allowed) → o fp32 [T, H·v_dim]."""
    _cuda(q, k, v, z, state, req_pool_indices, z_bias, bonus)
    T = q.shape[0]
    if state.dtype != torch.float32 or not state.is_contiguous():
        raise RuntimeError("gated_recurrence: the state is contiguous fp32")
    if any(t.stride(1) != 1 for t in (q, k, v, z)) or not (q.dtype == k.dtype == v.dtype == z.dtype):
        raise RuntimeError("gated_recurrence: q / k / v / z need contiguous rows and one dtype")
    for t in (z_bias, bonus):
        if t is not None and (t.dtype != torch.float32 or t.numel() != num_heads * head_dim or not t.is_contiguous()):
            raise RuntimeError("gated_recurrence: z_bias and bonus are fp32 [heads * head_dim]")
    o = torch.empty((T, num_heads * v_dim), device=q.device, dtype=torch.float32)
    check(lib.spd_gated_recurrence(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), z.data_ptr(),
                                   state.data_ptr(), req_pool_indices.data_ptr(), _ptr(seq_lens), _ptr(out_cache_loc),
                                   _ptr(prefix_lens), _ptr(extend_lens), _ptr(extend_start_loc),
                                   req_pool_indices.numel(), num_heads, head_dim, v_dim, q.stride(0), k.stride(0),
                                   v.stride(0), z.stride(0), _ptr(z_bias), _ptr(bonus),
                                   {"sigmoid_pow": 0, "double_exp": 1}[form], float(q_scale), float(tau), _dta(q),
                                   _stream()), "spd_gated_recurrence")
    return o


def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, shift_state: torch.Tensor, req_pool_indices, seq_lens=None,
                    out_cache_loc=None, prefix_lens=None, extend_lens=None, extend_start_loc=None,
                    max_extend_len: int = 0) -> torch.Tensor:
    """→ [n_mix, T, dim]: h + (previous row − h) · mu[s]; a request's row before its first new one is kept in
    shift_state[slot] (fp32 [slots, dim], zeros at position 0), which then receives its last row."""
    _cuda(h, mu, shift_state, req_pool_indices)
    if h.dim() != 2 or not h.is_contiguous() or mu.dtype != h.dtype or not mu.is_contiguous() or mu.shape[1] != h.shape[1]:
        raise RuntimeError("token_shift_mix: h [T, dim] and mu [n_mix, dim] are contiguous and share a dtype")
    if shift_state.dtype != torch.float32 or not shift_state.is_contiguous():
        raise RuntimeError("token_shift_mix: the shift state is contiguous fp32")
    T, dim = h.shape
    out = torch.empty((mu.shape[0], T, dim), device=h.device, dtype=h.dtype)
    check(lib.spd_token_shift_mix(out.data_ptr(), h.data_ptr(), mu.data_ptr(), shift_state.data_ptr(),
                                  req_pool_indices.data_ptr(), _ptr(seq_lens), _ptr(out_cache_loc), _ptr(prefix_lens),
                                  _ptr(extend_lens), _ptr(extend_start_loc), req_pool_indices.numel(), T,
                                  int(max_extend_len), dim, mu.shape[0], _dta(h), _stream()), "spd_token_shift_mix")
    return out


def embed_sincos(table: torch.Tensor, idx: torch.Tensor, positions: torch.Tensor, freq_hi: torch.Tensor,
                 freq_lo: torch.Tensor) -> torch.Tensor:
    """fp32 [n, dim]: table rows plus the sinusoidal position vector (sin at even, cos at odd entries of
    position · (freq_hi + freq_lo)[i])."""
    _cuda(table, idx, positions, freq_hi, freq_lo)
    if idx.dtype != torch.int64:
        idx = idx.long()
    if positions.dtype != torch.int64:
        positions = positions.long()
    out = torch.empty((idx.numel(), table.shape[1]), device=table.device, dtype=torch.float32)
    check(lib.spd_embed_sincos(out.data_ptr(), table.data_ptr(), idx.data_ptr(), positions.data_ptr(),
                               freq_hi.data_ptr(), freq_lo.data_ptr(), idx.numel(), table.shape[1], table.shape[0],
                               _dta(table), _stream()), "spd_embed_sincos")
    return out


def cast_concat(a: torch.Tensor, b: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """[a | b] of two fp32 [T, dim] streams in `dtype` — the operand of a projection that reads both."""
    _cuda(a, b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape or not a.is_contiguous() \
            or not b.is_contiguous():
        raise RuntimeError("cast_concat: a and b are contiguous fp32 of one shape")
    out = torch.empty((a.shape[0], 2 * a.shape[1]), device=a.device, dtype=dtype)
    check(lib.spd_cast_concat(out.data_ptr(), a.data_ptr(), b.data_ptr(), a.shape[0], a.shape[1], _dta(out), _stream()),
          "spd_cast_concat")
    return out


_ACTS = {"silu": 0, "gelu_tanh": 1, "relu2": 2, "tanh": 3, "relu": 4}


def activation(x: torch.Tensor, act: str) -> torch.Tensor:
    """act(x) elementwise (silu, gelu_tanh, relu2 = relu squared, tanh, relu); x [rows, cols] with contiguous rows."""
    _cuda(x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise RuntimeError("activation: x must be [rows, cols] with contiguous rows")
    out = torch.empty(x.shape, device=x.device, dtype=x.dtype)
    check(lib.spd_activation(out.data_ptr(), x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), _ACTS[act], _dta(x),
                             _stream()), "spd_activation")
    return out


def rmsnorm_store(x: torch.Tensor, weight: torch.Tensor, eps: float, pool: Optional[torch.Tensor] = None,
                  loc: Optional[torch.Tensor] = None, want_out: bool = False) -> Optional[torch.Tensor]:
    """RMS norm of the rows of x (row-strided view allowed) times weight, written to pool[loc[t]] (a cache pool
    whose rows are at least as long) and / or returned."""
    _cuda(x, weight, pool, loc)
    if x.dim() != 2 or x.stride(1) != 1 or weight.dtype != x.dtype or (pool is not None and pool.dtype != x.dtype):
        raise RuntimeError("rmsnorm_store: x [T, dim] with contiguous rows; weight and pool in x's dtype")
    if pool is not None and loc.dtype != torch.int64:
        loc = loc.long()
    T, dim = x.shape
    out = torch.empty((T, dim), device=x.device, dtype=x.dtype) if want_out else None
    pool_stride = pool.stride(0) if pool is not None else 0
    check(lib.spd_rmsnorm_store(_ptr(pool), _ptr(out), x.data_ptr(), weight.data_ptr(), _ptr(loc), T, dim, x.stride(0),
                                pool_stride, float(eps), _dta(x), _stream()), "spd_rmsnorm_store")
    return out


def head_gate_sigmoid(o: torch.Tensor, g: torch.Tensor, heads: int, vdim: int) -> torch.Tensor:
    """o [T, heads·vdim] · sigmoid(g [T, heads]) per head (row-strided views allowed)."""
    _cuda(o, g)
    if o.stride(1) != 1 or g.stride(1) != 1 or o.dtype != g.dtype:
        raise RuntimeError("head_gate_sigmoid: o and g need contiguous rows and one dtype")
    T = o.shape[0]
    out = torch.empty((T, heads * vdim), device=o.device, dtype=o.dtype)
    check(lib.spd_head_gate_sigmoid(out.data_ptr(), o.data_ptr(), g.data_ptr(), T, heads, vdim, o.stride(0),
                                    g.stride(0), _dta(o), _stream()), "spd_head_gate_sigmoid")
    return out


def scale_f32_(x: torch.Tensor, alpha: float) -> torch.Tensor:
    """x *= alpha in place (contiguous fp32)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise RuntimeError("scale_f32_: x is contiguous fp32")
    check(lib.spd_scale_f32(x.data_ptr(), x.numel(), float(alpha), _stream()), "spd_scale_f32")
    return x


def kv_store(key: torch.Tensor, value: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
             loc: torch.Tensor) -> None:
    """k_pool[loc] = key rows, v_pool[loc] = value rows (row sizes may differ; any dtype)."""
    _cuda(key, value, k_pool, v_pool, loc)
    T = key.shape[0]
    if T == 0:
        return
    if value is None:  # one buffer holds keys and values (a latent cache)
        k2 = key.reshape(T, -1)
        if loc.dtype != torch.int64:
            loc = loc.long()
        check(lib.spd_kv_store(k2.data_ptr(), None, k_pool.data_ptr(), None, loc.data_ptr(), T, k2.shape[1], 0,
                               k2.stride(0), 0, _dta(key), _stream()), "spd_kv_store")
        return
    k2, v2 = key.reshape(T, -1), value.reshape(T, -1)  # views for row-strided slices of a merged projection
    if k2.dim() != 2 or v2.dim() != 2 or k2.stride(1) != 1 or v2.stride(1) != 1:
        raise RuntimeError("kv_store: key / value must be [T, row] with contiguous rows")
    if loc.dtype != torch.int64:
        loc = loc.long()
    check(lib.spd_kv_store(k2.data_ptr(), v2.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), loc.data_ptr(), T,
                           k2.shape[1], v2.shape[1], k2.stride(0), v2.stride(0), _dta(key), _stream()), "spd_kv_store")


def attn_general(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, req_to_token, req_pool_indices,
                 num_q_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, sm_scale: float, window: int = -1,
                 sinks: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None, qtemp_coef: float = 0.0,
                 qtemp_every: int = 0, seq_lens=None, prefix_lens=None, extend_lens=None, extend_start_loc=None,
                 max_extend_len: int = 0, softcap: float = 0.0, num_v_heads: int = 0,
                 v_slot_stride: int = 0) -> torch.Tensor:
    """Windowed / sink / distance-biased softmax attention over the paged pool; decode (seq_lens) or
    ragged extend (prefix_lens, extend_lens, extend_start_loc).  q [T, H·head_dim] → [T, H·v_dim].
    max_extend_len > 0 (a host-side bound of extend_lens) lets 16-bit prefill run on the tensor cores.
    softcap > 0 caps the scaled scores by softcap · tanh(· / softcap); num_v_heads < num_kv_heads: key head g
    reads value head g mod num_v_heads; v_slot_stride: elements between two slots of v_pool (values that are
    the first v_dim columns of wider rows)."""
    _cuda(q, k_pool, v_pool, req_to_token, req_pool_indices, sinks, slopes)
    T = q.shape[0]
    if q.dim() != 2 or q.stride(1) != 1:
        raise RuntimeError("attn_general: q must be [T, H * head_dim] with contiguous rows")
    if req_pool_indices.dtype != torch.int64 or (seq_lens is not None and seq_lens.dtype != torch.int64):
        raise RuntimeError("attn_general: req_pool_indices and seq_lens must be int64")
    for t in (prefix_lens, extend_lens, extend_start_loc):
        if t is not None and t.dtype != torch.int32:
            raise RuntimeError("attn_general: prefix_lens / extend_lens / extend_start_loc must be int32")
    for t in (sinks, slopes):
        if t is not None and t.dtype != torch.float32:
            raise RuntimeError("attn_general: sinks and slopes are fp32")
    out = torch.empty((T, num_q_heads * v_dim), device=q.device, dtype=q.dtype)
    check(lib.spd_attn_general_ex(out.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
                                  req_to_token.data_ptr(), req_pool_indices.data_ptr(), _ptr(seq_lens), _ptr(prefix_lens),
                                  _ptr(extend_lens), _ptr(extend_start_loc), req_pool_indices.numel(), T, num_q_heads,
                                  num_kv_heads, head_dim, v_dim, q.stride(0), out.stride(0), req_to_token.stride(0),
                                  float(sm_scale), int(window), _ptr(sinks), _ptr(slopes), float(qtemp_coef),
                                  int(qtemp_every), int(max_extend_len), float(softcap or 0.0), int(num_v_heads),
                                  int(v_slot_stride), _dta(q), _stream()), "spd_attn_general")
    return out


def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, req_pool_indices,
              num_heads: int, head_dim: int, v_dim: int, decay: torch.Tensor, cos_sin: Optional[torch.Tensor],
              rot_dims: int, k_scale: float, seq_lens=None, out_cache_loc=None, prefix_lens=None, extend_lens=None,
              extend_start_loc=None, in_act: Optional[str] = None) -> torch.Tensor:
    """Decayed linear attention over the per-request recurrent state (updated in place);
    q / k [T, H·head_dim], v [T, H·v_dim] (row-strided views allowed) → o fp32 [T, H·v_dim].  in_act "silu":
    q, k and v are the SiLU of what is passed (applied in fp32 inside the kernel)."""
    _cuda(q, k, v, state, req_pool_indices, decay, cos_sin)
    T = q.shape[0]
    if state.dtype != torch.float32 or decay.dtype != torch.float32 or not state.is_contiguous():
        raise RuntimeError("retention: state and decay are fp32")
    if any(t.stride(1) != 1 for t in (q, k, v)) or not (q.dtype == k.dtype == v.dtype):
        raise RuntimeError("retention: q / k / v need contiguous rows and one dtype")
    o = torch.empty((T, num_heads * v_dim), device=q.device, dtype=torch.float32)
    check(lib.spd_retention(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                            req_pool_indices.data_ptr(), _ptr(seq_lens), _ptr(out_cache_loc), _ptr(prefix_lens),
                            _ptr(extend_lens), _ptr(extend_start_loc), req_pool_indices.numel(), num_heads, head_dim,
                            v_dim, q.stride(0), k.stride(0), v.stride(0), decay.data_ptr(), _ptr(cos_sin), int(rot_dims),
                            cos_sin.shape[0] if cos_sin is not None else 0, float(k_scale),
                            {None: 0, "silu": 1}[in_act], _dta(q), _stream()),
          "spd_retention")
    return o


# ------------------------------------------------------------------------------------------------
# a residual kept as several streams, rotary positions with biased projections, gated matrix memory
# ------------------------------------------------------------------------------------------------
def embed_norm_streams(table: torch.Tensor, idx: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
                       streams: int) -> torch.Tensor:
    """fp32 [n, streams, dim]: every stream starts as the RMS-normed embedding row (weight None: the raw row)."""
    _cuda(table, idx, weight)
    if idx.dtype != torch.int64:
        idx = idx.long()
    if weight is not None and (weight.dtype != table.dtype or not weight.is_contiguous()):
        raise RuntimeError("embed_norm_streams: the norm weight shares the table's dtype")
    out = torch.empty((idx.numel(), int(streams), table.shape[1]), device=table.device, dtype=torch.float32)
    check(lib.spd_embed_norm_streams(out.data_ptr(), table.data_ptr(), idx.data_ptr(), _ptr(weight), idx.numel(),
                                     table.shape[1], table.shape[0], int(streams), float(eps), _dta(table), _stream()),
          "spd_embed_norm_streams")
    return out


def streams_mix_norm(X: torch.Tensor, weight: Optional[torch.Tensor], eps: float, a: Optional[torch.Tensor] = None,
                     b: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, sa: float = 1.0,
                     sb: float = 1.0, sbias: float = 1.0, mix: Optional[torch.Tensor] = None,
                     out_w: Optional[torch.Tensor] = None, mult: float = 1.0, in_w: Optional[torch.Tensor] = None,
                     rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """X fp32 [T, S, dim] in place.  With a: y = sa·a + sb·b + sbias·bias and X'[t] = Σ_s mix[s, t] X[s] + mult ·
    out_w[t] · y.  With weight: → norm(Σ_s in_w[s] X'[s]) · weight in the weight's dtype (in_w None: the plain sum);
    rows (int64) selects the tokens that are read (no write then)."""
    _cuda(X, weight, a, b, bias, mix, out_w, in_w, rows)
    if X.dtype != torch.float32 or not X.is_contiguous() or X.dim() != 3:
        raise RuntimeError("streams_mix_norm: the streams are contiguous fp32 [T, S, dim]")
    T, S, d = X.shape
    ref = weight if weight is not None else a
    for t in (a, b):
        if t is not None and (not t.is_contiguous() or tuple(t.shape) != (T, d) or t.dtype != ref.dtype):
            raise RuntimeError("streams_mix_norm: a / b are contiguous [T, dim] in one dtype")
    for t, n in ((bias, d), (mix, S * S), (out_w, S), (in_w, S)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n):
            raise RuntimeError("streams_mix_norm: bias and stream coefficients are contiguous fp32")
    n_out = T if rows is None else rows.numel()
    out = torch.empty((n_out, d), device=X.device, dtype=weight.dtype) if weight is not None else None
    check(lib.spd_streams_mix_norm(_ptr(out), X.data_ptr(), _ptr(a), _ptr(b), _ptr(bias), float(sa), float(sb),
                                   float(sbias), _ptr(mix), _ptr(out_w), float(mult), _ptr(in_w), _ptr(weight),
                                   _ptr(rows), n_out, d, S, float(eps), _dta(ref), _stream()), "spd_streams_mix_norm")
    return out


def rotary_bias_store(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor], q_bias: Optional[torch.Tensor],
                      k_bias: Optional[torch.Tensor], k_pool: torch.Tensor, v_pool: Optional[torch.Tensor],
                      loc: torch.Tensor, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], rot_dims: int,
                      num_q_heads: int, num_kv_heads: int, head_dim: int, v_dim: int) -> torch.Tensor:
    """→ rotated q + q_bias [T, Hq·head_dim]; the rotated k + k_bias go to k_pool[loc], the values to v_pool[loc]:
    v, or (v None) the biased keys before the rotation.  q / k / v may be row-strided views."""
    _cuda(q, k, v, q_bias, k_bias, k_pool, v_pool, loc, positions, cos_sin)
    T = q.shape[0]
    if any(t is not None and t.stride(1) != 1 for t in (q, k, v)):
        raise RuntimeError("rotary_bias_store: q / k / v need contiguous rows")
    for t in (q_bias, k_bias, cos_sin):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise RuntimeError("rotary_bias_store: biases and the cos / sin table are contiguous fp32")
    if loc.dtype != torch.int64 or positions.dtype != torch.int64:
        raise RuntimeError("rotary_bias_store: loc and positions are int64")
    if not k_pool.is_contiguous() or (v_pool is not None and not v_pool.is_contiguous()):
        raise RuntimeError("rotary_bias_store: the pools are contiguous")
    out = torch.empty((T, num_q_heads * head_dim), device=q.device, dtype=q.dtype)
    check(lib.spd_rotary_bias_store(out.data_ptr(), q.data_ptr(), k.data_ptr(), _ptr(v), _ptr(q_bias), _ptr(k_bias),
                                    k_pool.data_ptr(), _ptr(v_pool), loc.data_ptr(), positions.data_ptr(),
                                    _ptr(cos_sin), int(rot_dims), cos_sin.shape[0] if cos_sin is not None else 0, T,
                                    num_q_heads, num_kv_heads, head_dim, v_dim, q.stride(0), k.stride(0),
                                    v.stride(0) if v is not None else 0, out.stride(0), _dta(q), _stream()),
          "spd_rotary_bias_store")
    return out


def matrix_memory_vector_dim(num_heads: int, head_dim: int, v_dim: int) -> int:
    """Floats per request of the vector state that matrix_memory keeps beside the matrix state."""
    return int(lib.spd_matrix_memory_vector_dim(int(num_heads), int(head_dim), int(v_dim)))


def matrix_memory(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, zi: torch.Tensor, zf: torch.Tensor,
                  state: torch.Tensor, vec: torch.Tensor, req_pool_indices, num_heads: int, head_dim: int, v_dim: int,
                  i_bias: Optional[torch.Tensor], f_bias: Optional[torch.Tensor], cap: float, q_scale: float,
                  seq_lens=None, out_cache_loc=None, prefix_lens=None, extend_lens=None,
                  extend_start_loc=None) -> torch.Tensor:
    """Exponentially gated matrix memory over the per-request state (matrix state `state`, normaliser and running
    maximum in `vec`, both updated in place); zi / zf [T, H] are the raw gate projections.  → o fp32 [T, H·v_dim]."""
    _cuda(q, k, v, zi, zf, state, vec, req_pool_indices, i_bias, f_bias)
    T = q.shape[0]
    if state.dtype != torch.float32 or vec.dtype != torch.float32 or not state.is_contiguous() or vec.stride(1) != 1:
        raise RuntimeError("matrix_memory: the states are fp32")
    if any(t.stride(1) != 1 for t in (q, k, v, zi, zf)) or not (q.dtype == k.dtype == v.dtype == zi.dtype == zf.dtype):
        raise RuntimeError("matrix_memory: q / k / v / zi / zf need contiguous rows and one dtype")
    for t in (i_bias, f_bias):
        if t is not None and (t.dtype != torch.float32 or t.numel() != num_heads):
            raise RuntimeError("matrix_memory: gate biases are fp32 [heads]")
    o = torch.empty((T, num_heads * v_dim), device=q.device, dtype=torch.float32)
    check(lib.spd_matrix_memory(o.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), zi.data_ptr(), zf.data_ptr(),
                                state.data_ptr(), vec.data_ptr(), vec.stride(0), req_pool_indices.data_ptr(),
                                _ptr(seq_lens), _ptr(out_cache_loc), _ptr(prefix_lens), _ptr(extend_lens),
                                _ptr(extend_start_loc), req_pool_indices.numel(), num_heads, head_dim, v_dim,
                                q.stride(0), k.stride(0), v.stride(0), zi.stride(0), zf.stride(0), _ptr(i_bias),
                                _ptr(f_bias), float(cap), float(q_scale), _dta(q), _stream()), "spd_matrix_memory")
    return o


# ------------------------------------------------------------------------------------------------
# token-pair embedding, tanh norm, rotary positions over strided segments, gated attention heads
# ------------------------------------------------------------------------------------------------
def embed_pair(table: torch.Tensor, idx: torch.Tensor, scale: float = 1.0, pair: Optional[torch.Tensor] = None,
               buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, prev_state: Optional[torch.Tensor] = None,
               req_pool_indices=None, seq_lens=None, out_cache_loc=None, prefix_lens=None, extend_lens=None,
               extend_start_loc=None) -> torch.Tensor:
    """fp32 [n, dim] = table[idx] · scale + pair[(prev · mul_prev + idx · mul_cur) mod buckets] (row `buckets` for a
    request's first token).  prev: the row before of the same request, or prev_state[slot] (int32 [slots]) where a
    portion starts; prev_state[slot] then receives the request's last token.  Decode (seq_lens) or ragged extend."""
    _cuda(table, idx, pair, prev_state, req_pool_indices)
    if idx.dtype != torch.int64:
        idx = idx.long()
    if pair is not None:
        if pair.dtype != table.dtype or not pair.is_contiguous() or pair.shape[1] != table.shape[1] \
                or pair.shape[0] != buckets + 1:
            raise RuntimeError("embed_pair: the pair table is [buckets + 1, dim] in the table's dtype")
        if prev_state is None or prev_state.dtype != torch.int32 or not prev_state.is_contiguous():
            raise RuntimeError("embed_pair: the previous-token state is contiguous int32 [slots]")
        if req_pool_indices.dtype != torch.int64 or (seq_lens is not None and seq_lens.dtype != torch.int64):
            raise RuntimeError("embed_pair: req_pool_indices and seq_lens must be int64")
        for t in (prefix_lens, extend_lens, extend_start_loc):
            if t is not None and t.dtype != torch.int32:
                raise RuntimeError("embed_pair: prefix_lens / extend_lens / extend_start_loc must be int32")
    n = idx.numel()
    out = torch.empty((n, table.shape[1]), device=table.device, dtype=torch.float32)
    batch = req_pool_indices.numel() if req_pool_indices is not None else 0
    check(lib.spd_embed_pair(out.data_ptr(), table.data_ptr(), _ptr(pair), idx.data_ptr(), _ptr(prev_state),
                             _ptr(req_pool_indices), _ptr(seq_lens), _ptr(out_cache_loc), _ptr(prefix_lens),
                             _ptr(extend_lens), _ptr(extend_start_loc), batch, n, table.shape[1], table.shape[0],
                             float(scale), int(buckets), int(mul_prev), int(mul_cur), _dta(table), _stream()),
          "spd_embed_pair")
    return out


def residual_tanh_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], alpha: float,
                       a: Optional[torch.Tensor] = None, x0: Optional[torch.Tensor] = None,
                       vec: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """x (fp32, in place) += a + x0 + vec (each optional); → tanh(alpha · x) · weight + bias in the weight's dtype
    (None when weight is None: update only).  rows (int64) selects the rows that are normed (nothing is added)."""
    _cuda(x, weight, bias, a, x0, vec, rows)
    if x.dtype != torch.float32 or not x.is_contiguous() or x.dim() != 2:
        raise RuntimeError("residual_tanh_norm: the residual stream is contiguous fp32 [T, dim]")
    d = x.shape[1]
    if a is not None and (not a.is_contiguous() or a.shape != x.shape or (weight is not None and a.dtype != weight.dtype)):
        raise RuntimeError("residual_tanh_norm: a matches x, is contiguous and shares the weight's dtype")
    for t, shape in ((x0, tuple(x.shape)), (vec, (d,))):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != shape):
            raise RuntimeError("residual_tanh_norm: x0 [T, dim] and vec [dim] are contiguous fp32")
    if (weight is None) != (bias is None) or (weight is not None and (weight.dtype != bias.dtype or weight.numel() != d
                                                                       or bias.numel() != d)):
        raise RuntimeError("residual_tanh_norm: weight and bias are [dim] in one dtype")
    ref = weight if weight is not None else a
    if ref is None:  # nothing but fp32 terms to add
        ref = x
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, d), device=x.device, dtype=weight.dtype) if weight is not None else None
    check(lib.spd_residual_tanh_norm(_ptr(out), x.data_ptr(), _ptr(a), _ptr(x0), _ptr(vec), _ptr(weight), _ptr(bias),
                                     _ptr(rows), n, d, float(alpha), _dta(ref), _stream()), "spd_residual_tanh_norm")
    return out


def rotary_segment(src: torch.Tensor, dst: torch.Tensor, heads: int, head_dim: int, rot: int = 0,
                   bias: Optional[torch.Tensor] = None, src_head: Optional[int] = None, dst_head: Optional[int] = None,
                   to_pool: bool = False) -> _lib.RotarySegment:
    """One piece of rotary_segments: src / dst are 2-D views whose first element is the first head's first channel
    (row stride = stride(0); src_head / dst_head default to head_dim)."""
    _cuda(src, dst, bias)
    if src.stride(-1) != 1 or dst.stride(-1) != 1 or src.dtype != dst.dtype:
        raise RuntimeError("rotary_segment: src and dst have contiguous rows and one dtype")
    if bias is not None and (bias.dtype != torch.float32 or not bias.is_contiguous() or bias.numel() != heads * head_dim):
        raise RuntimeError("rotary_segment: bias is contiguous fp32 [heads * head_dim]")
    seg = _lib.RotarySegment(src.data_ptr(), _ptr(bias), dst.data_ptr(), src.stride(0), dst.stride(0), heads, head_dim, rot,
                             head_dim if src_head is None else src_head, head_dim if dst_head is None else dst_head,
                             1 if to_pool else 0)
    seg.keep = (src, dst, bias)  # the descriptor holds raw pointers: the tensors live as long as it does
    return seg


def rotary_segments(segments, positions: torch.Tensor, cos_sin: Optional[torch.Tensor], dtype: torch.dtype,
                    loc: Optional[torch.Tensor] = None, paired: bool = False) -> None:
    """Bias + partial rotation + scatter of up to four strided segments in one launch (see rotary_segment).
    cos_sin fp32 [positions, rot_max] = cos ‖ sin; paired: channel 2 i turns with 2 i + 1, else i with i + rot / 2."""
    _cuda(positions, cos_sin, loc)
    if positions.dtype != torch.int64 or (loc is not None and loc.dtype != torch.int64):
        raise RuntimeError("rotary_segments: positions and loc are int64")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous()):
        raise RuntimeError("rotary_segments: the cos / sin table is contiguous fp32")
    arr = (_lib.RotarySegment * len(segments))(*segments)
    check(lib.spd_rotary_segments(arr, len(segments), positions.data_ptr(), _ptr(loc), _ptr(cos_sin),
                                  cos_sin.shape[1] if cos_sin is not None else 0,
                                  cos_sin.shape[0] if cos_sin is not None else 0, 1 if paired else 0,
                                  positions.numel(), _DTYPE_ANY[dtype], _stream()), "spd_rotary_segments")


def heads_gate(a: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int, a2: Optional[torch.Tensor] = None,
               lam: float = 0.0, eps: float = 0.0, post: float = 1.0) -> torch.Tensor:
    """[T, heads·vdim] = y · sigmoid(gate) with y = a, or (a2 given, a view with a's strides) the unit-RMS per head of
    a − lam · a2 times post.  a / a2 / gate may be row-strided views."""
    _cuda(a, a2, gate)
    if a.stride(1) != 1 or gate.stride(1) != 1 or a.dtype != gate.dtype:
        raise RuntimeError("heads_gate: a and gate need contiguous rows and one dtype")
    if a2 is not None and (a2.stride(0) != a.stride(0) or a2.stride(1) != 1 or a2.dtype != a.dtype):
        raise RuntimeError("heads_gate: a2 shares a's strides and dtype")
    T = a.shape[0]
    out = torch.empty((T, heads * vdim), device=a.device, dtype=a.dtype)
    check(lib.spd_heads_gate(out.data_ptr(), a.data_ptr(), _ptr(a2), gate.data_ptr(), T, heads, vdim, a.stride(0),
                             gate.stride(0), out.stride(0), float(lam), float(eps), float(post), _dta(a), _stream()),
          "spd_heads_gate")
    return out


# ------------------------------------------------------------------------------------------------
# SM partitions (green contexts)
# ------------------------------------------------------------------------------------------------
import ctypes as _C


class SmPartition:
    """Two disjoint SM sets of one GPU with a stream each — the in-process replacement for the
    per-process MPS caps (S/entrypoints/engine.py:591-593,632-634)."""

    def __init__(self, device: int, prefill_sms: int, decode_sms: int):
        h = _C.c_void_p()
        check(lib.spd_partition_create(device, prefill_sms, decode_sms, _C.byref(h)),
              "spd_partition_create")
        self._h = h
        a, b = _C.c_int(), _C.c_int()
        check(lib.spd_partition_sm_counts(h, _C.byref(a), _C.byref(b)), "spd_partition_sm_counts")
        self.prefill_sms, self.decode_sms = a.value, b.value
        s0, s1 = _C.c_void_p(), _C.c_void_p()
        check(lib.spd_partition_stream(h, 0, _C.byref(s0)), "spd_partition_stream")
        check(lib.spd_partition_stream(h, 1, _C.byref(s1)), "spd_partition_stream")
        self.prefill_stream = torch.cuda.ExternalStream(s0.value, device=device)
        self.decode_stream = torch.cuda.ExternalStream(s1.value, device=device)

    def close(self):
        if self._h is not None:
            lib.spd_partition_destroy(self._h)
            self._h = None


_partitions = {}


def get_partition(device: int, prefill_sms: int, decode_sms: int) -> SmPartition:
    """Process-lifetime pool of SM partitions.  Green contexts and their streams are created once
    per (device, split) and REUSED by every engine built afterwards: torch's caching allocator
    and CUDA graphs keep referring to a stream long after the engine that used it is gone, so a
    partition is never destroyed under them (doing so was measured to abort the process);
    `SmPartition.close()` / spd_partition_destroy remain for embedders that own the streams'
    whole lifetime."""
    key = (int(device), int(prefill_sms), int(decode_sms))
    part = _partitions.get(key)
    if part is None:
        part = _partitions[key] = SmPartition(device, prefill_sms, decode_sms)
    return part


def device_sm_count(device: int = 0) -> int:
    n = _C.c_int()
    check(lib.spd_device_sm_count(device, _C.byref(n)), "spd_device_sm_count")
    return n.value
