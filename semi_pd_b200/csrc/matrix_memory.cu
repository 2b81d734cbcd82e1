// Exponentially gated matrix memory (the mLSTM cell): per (request, head) a matrix state S [head_dim x v_dim],
// a normaliser n [head_dim] and a running maximum m of the log gates, all fp32:
//     i = cap tanh((zi + bi) / cap)            f = logsigmoid(cap tanh((zf + bf) / cap))      (cap <= 0: no cap)
//     m' = max(f + m, i)        a = exp(f + m - m')        b = exp(i - m')
//     S' = a S + b k v^T        n' = a n + b k
//     o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)        with q scaled by q_scale as it is read
// m starts at 0 with S = n = 0 for a request that starts at position 0.  The gates are computed inside the
// kernel from the raw projection outputs zi, zf (one value per token and head), so everything that enters the
// recurrence is fp32 whatever the projections' dtype.  Layout as retention.cu: a CTA owns (request, head,
// 32 value columns) and keeps its [head_dim x 32] slice of S in registers (warp w the ROWS rows w * ROWS ..,
// lane l column l), and beside it the rows of n that belong to its warp's rows (every lane of the warp keeps the
// same copy: a butterfly over lanes that hold one row each measured slower than the repeated FMAs); the request's new tokens are
// walked in blocks of 16 (decode: its one token) staged through shared memory; one more warp turns a block's gate
// values into (a, b, exp(-m')) with the m chain run in registers, one block ahead of the accumulating warps;
// partial outputs and partial n . q of the warps meet in shared memory once per block.  Every output element is summed in one fixed order, so o does
// not depend on how a prompt was cut or batched.  Every column block keeps a copy of n and m of its own in
// the vector state ([heads, column blocks, head_dim + 1] per slot): no CTA reads what another one writes.
// ASYNC (ragged extend with 16-byte aligned rows): the raw q / k / v rows of the NEXT block are fetched with
// 16-byte cp.async into a raw staging area while the current block is accumulated.
// Launched in plain stream order, like the other recurrent mixers.  The reference has none.
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

constexpr int kMemTok = 16;   // tokens staged per block (extend); decode stages its one token
constexpr int kMemCols = 32;  // value columns per CTA

__device__ __forceinline__ float soft_cap(float z, float cap) { return cap > 0.f ? cap * tanhf(z / cap) : z; }
__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int W, int ROWS, bool ASYNC, int TOK>
__global__ void __launch_bounds__(W * 32 + 32)
matrix_memory_kernel(float* __restrict__ o, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const T* __restrict__ zi, const T* __restrict__ zf, float* __restrict__ state,
                     float* __restrict__ vec, int64_t vec_stride, const int64_t* __restrict__ req_pool_indices,
                     const int64_t* __restrict__ seq_lens, const int64_t* __restrict__ out_cache_loc,
                     const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                     const int32_t* __restrict__ extend_start_loc, int H, int dk, int dv, int64_t q_stride,
                     int64_t k_stride, int64_t v_stride, int64_t zi_stride, int64_t zf_stride,
                     const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale) {
  static_assert(ROWS % 4 == 0, "rows per thread are read as float4");
  static_assert(TOK <= 32, "warp 0 holds a block's gates one per lane");
  constexpr int DKP = W * ROWS;  // padded head_dim
  constexpr int NT = W * 32;  // accumulating threads; one more warp computes the gates
  constexpr int N = 16 / (int)sizeof(T);
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                        // [TOK][DKP] scaled
  float* ks = qs + TOK * DKP;              // [TOK][DKP]
  float* vs = ks + TOK * DKP;              // [TOK][kMemCols]
  float* part = vs + TOK * kMemCols;       // [W][TOK][kMemCols]
  float* partn = part + W * TOK * kMemCols;  // [W][TOK]
  float* gates = partn + W * TOK;          // [2][3][TOK]: a, b, exp(-m') of a block, two blocks in flight
  T* rq = reinterpret_cast<T*>(gates + 6 * TOK);  // ASYNC: [TOK][dk] raw
  T* rk = rq + TOK * dk;                   // ASYNC: [TOK][dk] raw
  T* rv = rk + TOK * dk;                   // ASYNC: [TOK][kMemCols] raw
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.z * kMemCols;
  const int c = col0 + lane;
  const bool col_ok = c < dv;

  int64_t pos0, row0;
  int n;
  bool keep_state = true;
  if (!ASYNC && seq_lens != nullptr) {
    pos0 = seq_lens[r] - 1;
    row0 = r;
    n = 1;
    if (out_cache_loc != nullptr && out_cache_loc[r] == 0) keep_state = false;  // padded row of a captured batch
  } else {
    pos0 = prefix_lens[r];
    row0 = extend_start_loc[r];
    n = extend_lens[r];
  }
  if (n <= 0 || pos0 < 0) return;
  const int64_t slot = req_pool_indices[r];
  float* st = state + (slot * H + h) * (int64_t)dk * dv;
  float* vc = vec + slot * vec_stride + ((int64_t)h * gridDim.z + blockIdx.z) * (dk + 1);  // n [dk], then m
  const bool cont = pos0 > 0;

  float S[ROWS], Nn[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = warp * ROWS + i;
    S[i] = (cont && row < dk && col_ok) ? st[(int64_t)row * dv + c] : 0.f;
    Nn[i] = (cont && row < dk) ? vc[row] : 0.f;
  }
  float m_run = cont ? vc[dk] : 0.f;  // the gate warp's
  const float bi = i_bias != nullptr ? i_bias[h] : 0.f, bf = f_bias != nullptr ? f_bias[h] : 0.f;
  const int qc = dk / N, vcn = kMemCols / N;  // ASYNC: 16-byte chunks per row
  auto fetch = [&](int t0) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    for (int idx = threadIdx.x; idx < nt * qc; idx += NT) {
      const int tt = idx / qc, ch = idx - tt * qc;
      const int64_t row = row0 + t0 + tt;
      cp_async16(smem_u32(rq + tt * dk + ch * N), q + row * q_stride + (int64_t)h * dk + ch * N, true);
      cp_async16(smem_u32(rk + tt * dk + ch * N), k + row * k_stride + (int64_t)h * dk + ch * N, true);
    }
    for (int idx = threadIdx.x; idx < nt * vcn; idx += NT) {
      const int tt = idx / vcn, ch = idx - tt * vcn;
      const bool ok = col0 + ch * N < dv;  // dv is a multiple of N: a chunk is inside or outside
      cp_async16(smem_u32(rv + tt * kMemCols + ch * N),
                 v + (row0 + t0 + tt) * v_stride + (int64_t)h * dv + (ok ? col0 + ch * N : 0), ok);
    }
    cp_async_commit();
  };
  // A warp of its own (warp W) turns the raw gate values of a block into (a, b, exp(-m')): lane tt computes i and f
  // of token tt, the m chain (one add and one max per token) runs in every lane, the exponentials follow, one token
  // per lane.  It works one block ahead of the W accumulating warps, into the other of two buffers.
  const bool gate_warp = warp == W;
  auto gate_block = [&](int t0) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    float* ga = gates + ((t0 / TOK) & 1) * 3 * TOK;
    float gi = 0.f, gf = 0.f;
    if (lane < nt) {
      const int64_t row = row0 + t0 + lane;
      gi = soft_cap(to_f32<T>(zi[row * zi_stride + h]) + bi, cap);
      gf = log_sigmoid(soft_cap(to_f32<T>(zf[row * zf_stride + h]) + bf, cap));
    }
    float m_before = 0.f, m_me = 0.f;
#pragma unroll
    for (int tt = 0; tt < TOK; ++tt) {
      const float it = __shfl_sync(0xffffffffu, gi, tt), ft = __shfl_sync(0xffffffffu, gf, tt);
      if (tt < nt) {
        const float mn = fmaxf(ft + m_run, it);
        if (lane == tt) {
          m_before = m_run;
          m_me = mn;
        }
        m_run = mn;
      }
    }
    if (lane < nt) {
      ga[lane] = expf(gf + m_before - m_me);
      ga[TOK + lane] = expf(gi - m_me);
      ga[2 * TOK + lane] = expf(-m_me);
    }
  };
  if (gate_warp) gate_block(0);
  if (ASYNC && !gate_warp) fetch(0);
  for (int t0 = 0; t0 < n; t0 += TOK) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    const float* ga = gates + ((t0 / TOK) & 1) * 3 * TOK;
    const float* gb = ga + TOK;
    const float* ge = gb + TOK;
    if (ASYNC) {
      cp_async_wait<0>();
      __syncthreads();  // raw rows of this block visible; the previous block's reduce has finished
    }
    for (int idx = gate_warp ? nt * DKP : threadIdx.x; idx < nt * DKP; idx += NT) {
      const int tt = idx / DKP, d = idx - tt * DKP;
      float qv = 0.f, kv = 0.f;
      if (d < dk) {
        if (ASYNC) {
          qv = to_f32<T>(rq[tt * dk + d]);
          kv = to_f32<T>(rk[tt * dk + d]);
        } else {
          const int64_t row = row0 + t0 + tt;
          qv = to_f32<T>(q[row * q_stride + (int64_t)h * dk + d]);
          kv = to_f32<T>(k[row * k_stride + (int64_t)h * dk + d]);
        }
      }
      qs[idx] = qv * q_scale;
      ks[idx] = kv;
    }
    for (int idx = gate_warp ? nt * kMemCols : threadIdx.x; idx < nt * kMemCols; idx += NT) {
      if (ASYNC) {
        vs[idx] = to_f32<T>(rv[idx]);
      } else {
        const int tt = idx / kMemCols, cl = idx - tt * kMemCols;
        vs[idx] = col0 + cl < dv ? to_f32<T>(v[(row0 + t0 + tt) * v_stride + (int64_t)h * dv + col0 + cl]) : 0.f;
      }
    }
    __syncthreads();  // staging and this block's gates complete (ASYNC: the raw area is free again)
    if (gate_warp) {
      // the next block's gates, while the other warps accumulate this one; their buffer was last read by the
      // reduce of the previous block, which every warp left before the barrier above
      if (t0 + TOK < n) gate_block(t0 + TOK);
    } else if (ASYNC && t0 + TOK < n) {
      fetch(t0 + TOK);
    }
    for (int tt = 0; tt < (gate_warp ? 0 : nt); ++tt) {
      const float a = ga[tt], b = gb[tt];
      const float bv = b * vs[tt * kMemCols + lane];
      const float4* kt = reinterpret_cast<const float4*>(ks + tt * DKP + warp * ROWS);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * DKP + warp * ROWS);
      float acc0 = 0.f, acc1 = 0.f, an0 = 0.f, an1 = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS / 4; ++i) {
        const float4 k4 = kt[i], q4 = qt[i];
        S[4 * i] = fmaf(a, S[4 * i], k4.x * bv);
        Nn[4 * i] = fmaf(a, Nn[4 * i], k4.x * b);
        acc0 = fmaf(S[4 * i], q4.x, acc0);
        an0 = fmaf(Nn[4 * i], q4.x, an0);
        S[4 * i + 1] = fmaf(a, S[4 * i + 1], k4.y * bv);
        Nn[4 * i + 1] = fmaf(a, Nn[4 * i + 1], k4.y * b);
        acc1 = fmaf(S[4 * i + 1], q4.y, acc1);
        an1 = fmaf(Nn[4 * i + 1], q4.y, an1);
        S[4 * i + 2] = fmaf(a, S[4 * i + 2], k4.z * bv);
        Nn[4 * i + 2] = fmaf(a, Nn[4 * i + 2], k4.z * b);
        acc0 = fmaf(S[4 * i + 2], q4.z, acc0);
        an0 = fmaf(Nn[4 * i + 2], q4.z, an0);
        S[4 * i + 3] = fmaf(a, S[4 * i + 3], k4.w * bv);
        Nn[4 * i + 3] = fmaf(a, Nn[4 * i + 3], k4.w * b);
        acc1 = fmaf(S[4 * i + 3], q4.w, acc1);
        an1 = fmaf(Nn[4 * i + 3], q4.w, an1);
      }
      part[(warp * TOK + tt) * kMemCols + lane] = acc0 + acc1;
      if (lane == 0) partn[warp * TOK + tt] = an0 + an1;
    }
    __syncthreads();
    for (int tt = gate_warp ? nt : warp; tt < nt; tt += W) {
      float sum = 0.f, nq = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        sum += part[(w * TOK + tt) * kMemCols + lane];
        nq += partn[w * TOK + tt];
      }
      const float den = fmaxf(fabsf(nq), ge[tt]) + 1e-6f;
      if (col_ok) o[((row0 + t0 + tt) * H + h) * (int64_t)dv + c] = sum / den;
    }
    // the next block's staging writes qs / ks / vs (last read before the barrier above) and its accumulation writes
    // part only after the barrier that follows the staging
  }
  if (keep_state) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = warp * ROWS + i;
      if (row < dk && col_ok) st[(int64_t)row * dv + c] = S[i];
      if (row < dk && lane == 0) vc[row] = Nn[i];
    }
    if (gate_warp && lane == 0) vc[dk] = m_run;
  }
}

template <typename T, int W, int ROWS, bool ASYNC, int TOK>
int matrix_memory_launch(dim3 grid, size_t smem, cudaStream_t stream, float* o, const void* q, const void* k,
                         const void* v, const void* zi, const void* zf, float* state, float* vec, int64_t vec_stride,
                         const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                         const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc, int H,
                         int dk, int dv, int64_t q_stride, int64_t k_stride, int64_t v_stride, int64_t zi_stride,
                         int64_t zf_stride, const float* i_bias, const float* f_bias, float cap, float q_scale) {
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    SPD_CUDA(cudaFuncSetAttribute(matrix_memory_kernel<T, W, ROWS, ASYNC, TOK>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  SPD_CUDA(launch(matrix_memory_kernel<T, W, ROWS, ASYNC, TOK>, grid, dim3(W * 32 + 32), smem, stream, /*pdl=*/false, o,
                  (const T*)q, (const T*)k, (const T*)v, (const T*)zi, (const T*)zf, state, vec, vec_stride,
                  req_pool_indices, seq_lens, out_cache_loc, prefix_lens, extend_lens, extend_start_loc, H, dk, dv,
                  q_stride, k_stride, v_stride, zi_stride, zf_stride, i_bias, f_bias, cap, q_scale));
  return 0;
}

}  // namespace spd

using namespace spd;

extern "C" {

int64_t spd_matrix_memory_vector_dim(int num_heads, int head_dim, int v_dim) {
  return (int64_t)num_heads * ((v_dim + kMemCols - 1) / kMemCols) * (head_dim + 1);
}

int spd_matrix_memory(float* o, const void* q, const void* k, const void* v, const void* zi, const void* zf,
                      float* state, float* vec, int64_t vec_stride, const int64_t* req_pool_indices,
                      const int64_t* seq_lens, const int64_t* out_cache_loc, const int32_t* prefix_lens,
                      const int32_t* extend_lens, const int32_t* extend_start_loc, int64_t batch, int num_heads,
                      int head_dim, int v_dim, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                      int64_t zi_stride, int64_t zf_stride, const float* i_bias, const float* f_bias, float cap,
                      float q_scale, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(o && q && k && v && zi && zf && state && vec && req_pool_indices, SPD_E_BADARG,
              "spd_matrix_memory: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_matrix_memory: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(num_heads > 0 && head_dim > 0 && head_dim <= 256 && v_dim > 0, SPD_E_SHAPE,
              "spd_matrix_memory: head_dim %d above 256", head_dim);
  SPD_REQUIRE(vec_stride >= spd_matrix_memory_vector_dim(num_heads, head_dim, v_dim), SPD_E_SHAPE,
              "spd_matrix_memory: vector state rows of %lld, need %lld", (long long)vec_stride,
              (long long)spd_matrix_memory_vector_dim(num_heads, head_dim, v_dim));
  if (batch == 0) return 0;
  const dim3 grid((unsigned)batch, (unsigned)num_heads, (unsigned)((v_dim + kMemCols - 1) / kMemCols));
  const int warps = head_dim <= 32 ? 4 : head_dim <= 64 ? 8 : 16;
  const int dkp = head_dim <= 128 ? warps * 8 : 256;
  const bool decode = seq_lens != nullptr;
  const size_t tok = decode ? 1 : kMemTok;
  const size_t smem = sizeof(float) * ((size_t)2 * tok * dkp + tok * kMemCols + (size_t)warps * tok * kMemCols +
                                       (size_t)warps * tok + 6 * tok);
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  const bool async_ok = !decode && head_dim % vecn == 0 && v_dim % vecn == 0 && q_stride % vecn == 0 &&
                        k_stride % vecn == 0 && v_stride % vecn == 0 && aligned16(q) && aligned16(k) && aligned16(v) &&
                        getenv("SPD_MATRIX_MEMORY_SYNC") == nullptr;
  const size_t esz = dtype == SPD_F32 ? 4 : 2;
  // with 16 tokens per block every fp32 area is a multiple of 4 floats, so the raw area is 16-byte aligned
  const size_t smem_async = smem + esz * kMemTok * (2 * (size_t)head_dim + kMemCols);
#define SPD_MEM_ARGS                                                                                              \
  as_stream(stream), o, q, k, v, zi, zf, state, vec, vec_stride, req_pool_indices, seq_lens, out_cache_loc,       \
      prefix_lens, extend_lens, extend_start_loc, num_heads, head_dim, v_dim, q_stride, k_stride, v_stride,      \
      zi_stride, zf_stride, i_bias, f_bias, cap, q_scale
#define SPD_MEM_SHAPE(W, ROWS)                                                                                    \
  return decode     ? matrix_memory_launch<T, W, ROWS, false, 1>(grid, smem, SPD_MEM_ARGS)                        \
         : async_ok ? matrix_memory_launch<T, W, ROWS, true, kMemTok>(grid, smem_async, SPD_MEM_ARGS)             \
                    : matrix_memory_launch<T, W, ROWS, false, kMemTok>(grid, smem, SPD_MEM_ARGS)
  SPD_DISPATCH_ANY(dtype, {
    if (head_dim <= 32) SPD_MEM_SHAPE(4, 8);
    else if (head_dim <= 64) SPD_MEM_SHAPE(8, 8);
    else if (head_dim <= 128) SPD_MEM_SHAPE(16, 8);
    else SPD_MEM_SHAPE(16, 16);
  });
#undef SPD_MEM_SHAPE
#undef SPD_MEM_ARGS
  return 0;
}

}  // extern "C"
