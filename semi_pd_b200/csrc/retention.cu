// Retention mixer: linear attention with a fixed decay per head and a matrix-valued recurrent
// state per (request, head), S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, no softmax and no
// denominator.  q and k are rotated (rotate-half pairing over the first rot_dims dimensions, fp32
// cos/sin table) and k is scaled inside the kernel, so everything that enters the recurrence is
// fp32 whatever the projections' dtype.  Decode and ragged extend (chunked prefill, mixed batches)
// are one kernel: a CTA owns (request, head, 32 value columns) and keeps its [head_dim x 32] slice
// of the state in registers: warp w holds the ROWS consecutive state rows w * ROWS .. and lane l
// the column l, so a token costs a thread two 16-byte shared-memory loads per four rows and
// 3 * ROWS FMAs, and W = head_dim / ROWS warps (4 to 16) share a token.  The request's new tokens
// are walked in blocks of 16 (decode: its one token) staged through shared memory (rows zero-padded
// to W * ROWS); the
// warps' partial outputs of a block meet in shared memory once per block; the state goes back to
// the request's slot at the end.  Every output element is summed in one fixed order (rows of a
// thread ascending over two interleaved accumulators, then warps ascending), so o does not depend
// on how a prompt was cut or batched.
// ASYNC (ragged extend with 16-byte aligned rows): the raw q / k / v rows and the cos / sin rows of
// the NEXT block are fetched with 16-byte cp.async into a raw staging area while the current block
// is accumulated, so a block costs its arithmetic instead of a chain of dependent global loads.
// Beside attn_general.cu in role (a mixer over per-request memory); the reference has none.
// These kernels are launched WITHOUT programmatic dependent launch (plain stream order): with it,
// the prefetching form between two tcgen05 GEMMs stopped making progress on B200 — the cause was
// not found — and a mixer of this length gains nothing from starting a few microseconds early.
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

// activation applied to q, k and v as they are read (before rotation): 0 none, 1 SiLU
__device__ __forceinline__ float ret_in_act(float x, int act) { return act == 1 ? x / (1.0f + expf(-x)) : x; }

constexpr int kRetTok = 16;   // tokens staged per block (extend); decode stages its one token
constexpr int kRetCols = 32;  // value columns per CTA

template <typename T, int W, int ROWS, bool ASYNC, int TOK>  // W warps x ROWS state rows per thread >= head_dim; TOK tokens per block
__global__ void __launch_bounds__(W * 32)
retention_kernel(float* __restrict__ o, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                 float* __restrict__ state, const int64_t* __restrict__ req_pool_indices,
                 const int64_t* __restrict__ seq_lens, const int64_t* __restrict__ out_cache_loc,
                 const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                 const int32_t* __restrict__ extend_start_loc, int H, int dk, int dv, int64_t q_stride,
                 int64_t k_stride, int64_t v_stride, const float* __restrict__ decay,
                 const float* __restrict__ cos_sin, int rot, int64_t max_positions, float k_scale, int in_act) {
  static_assert(ROWS % 4 == 0, "rows per thread are read as float4");
  constexpr int DKP = W * ROWS;  // padded head_dim
  constexpr int NT = W * 32;
  constexpr int N = 16 / (int)sizeof(T);
  extern __shared__ __align__(16) float smem[];
  float* qs = smem;                       // [TOK][DKP] rotated
  float* ks = qs + TOK * DKP;         // [TOK][DKP] rotated, scaled
  float* vs = ks + TOK * DKP;         // [TOK][kRetCols]
  float* part = vs + TOK * kRetCols;  // [W][TOK][kRetCols]
  float* cs = part + W * TOK * kRetCols;               // ASYNC: [TOK][rot] raw cos || sin rows
  T* rq = reinterpret_cast<T*>(cs + TOK * rot);        // ASYNC: [TOK][dk] raw
  T* rk = rq + TOK * dk;                               // ASYNC: [TOK][dk] raw
  T* rv = rk + TOK * dk;                               // ASYNC: [TOK][kRetCols] raw
  const int r = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.z * kRetCols;
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
  const float dec = decay[h];
  float* st = state + ((int64_t)req_pool_indices[r] * H + h) * (int64_t)dk * dv;

  float S[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = warp * ROWS + i;
    S[i] = (pos0 > 0 && row < dk && col_ok) ? st[(int64_t)row * dv + c] : 0.f;
  }
  const int half = rot >> 1;
  const int qc = dk / N, vc = kRetCols / N, cc = rot / 4;  // ASYNC: 16-byte chunks per row
  auto fetch = [&](int t0) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    for (int idx = threadIdx.x; idx < nt * qc; idx += NT) {
      const int tt = idx / qc, ch = idx - tt * qc;
      const int64_t row = row0 + t0 + tt;
      cp_async16(smem_u32(rq + tt * dk + ch * N), q + row * q_stride + (int64_t)h * dk + ch * N, true);
      cp_async16(smem_u32(rk + tt * dk + ch * N), k + row * k_stride + (int64_t)h * dk + ch * N, true);
    }
    for (int idx = threadIdx.x; idx < nt * vc; idx += NT) {
      const int tt = idx / vc, ch = idx - tt * vc;
      const bool ok = col0 + ch * N < dv;  // dv is a multiple of N: a chunk is inside or outside
      cp_async16(smem_u32(rv + tt * kRetCols + ch * N),
                 v + (row0 + t0 + tt) * v_stride + (int64_t)h * dv + (ok ? col0 + ch * N : 0), ok);
    }
    for (int idx = threadIdx.x; idx < nt * cc; idx += NT) {
      const int tt = idx / cc, ch = idx - tt * cc;
      int64_t p = pos0 + t0 + tt;
      p = p < max_positions ? p : max_positions - 1;
      cp_async16(smem_u32(cs + tt * rot + ch * 4), cos_sin + p * rot + ch * 4, true);
    }
    cp_async_commit();
  };
  if (ASYNC) fetch(0);
  for (int t0 = 0; t0 < n; t0 += TOK) {
    const int nt = n - t0 < TOK ? n - t0 : TOK;
    if (ASYNC) {
      cp_async_wait<0>();
      __syncthreads();  // raw rows of this block visible; the previous block's reduce has finished
    }
    // stage rotated q, rotated + scaled k (rows zero-padded to DKP), and v of nt tokens
    for (int idx = threadIdx.x; idx < nt * DKP; idx += NT) {
      const int tt = idx / DKP, d = idx - tt * DKP;
      float qv = 0.f, kv = 0.f;
      if (d < dk) {
        if (ASYNC) {
          const T* qr = rq + tt * dk;
          const T* kr = rk + tt * dk;
          qv = ret_in_act(to_f32<T>(qr[d]), in_act);
          kv = ret_in_act(to_f32<T>(kr[d]), in_act);
          if (d < rot) {
            const int i = d < half ? d : d - half;
            const float cv = cs[tt * rot + i], sn = cs[tt * rot + half + i];
            if (d < half) {
              qv = qv * cv - ret_in_act(to_f32<T>(qr[d + half]), in_act) * sn;
              kv = kv * cv - ret_in_act(to_f32<T>(kr[d + half]), in_act) * sn;
            } else {
              qv = qv * cv + ret_in_act(to_f32<T>(qr[d - half]), in_act) * sn;
              kv = kv * cv + ret_in_act(to_f32<T>(kr[d - half]), in_act) * sn;
            }
          }
        } else {
          const int64_t row = row0 + t0 + tt;
          const T* qr = q + row * q_stride + (int64_t)h * dk;
          const T* kr = k + row * k_stride + (int64_t)h * dk;
          qv = ret_in_act(to_f32<T>(qr[d]), in_act);
          kv = ret_in_act(to_f32<T>(kr[d]), in_act);
          if (d < rot) {
            int64_t p = pos0 + t0 + tt;
            p = p < max_positions ? p : max_positions - 1;
            const int i = d < half ? d : d - half;
            const float cv = cos_sin[p * rot + i], sn = cos_sin[p * rot + half + i];
            if (d < half) {
              qv = qv * cv - ret_in_act(to_f32<T>(qr[d + half]), in_act) * sn;
              kv = kv * cv - ret_in_act(to_f32<T>(kr[d + half]), in_act) * sn;
            } else {
              qv = qv * cv + ret_in_act(to_f32<T>(qr[d - half]), in_act) * sn;
              kv = kv * cv + ret_in_act(to_f32<T>(kr[d - half]), in_act) * sn;
            }
          }
        }
      }
      qs[idx] = qv;
      ks[idx] = kv * k_scale;
    }
    for (int idx = threadIdx.x; idx < nt * kRetCols; idx += NT) {
      if (ASYNC) {
        vs[idx] = ret_in_act(to_f32<T>(rv[idx]), in_act);
      } else {
        const int tt = idx / kRetCols, cl = idx - tt * kRetCols;
        vs[idx] = col0 + cl < dv ? ret_in_act(to_f32<T>(v[(row0 + t0 + tt) * v_stride + (int64_t)h * dv + col0 + cl]), in_act) : 0.f;
      }
    }
    __syncthreads();  // staging complete (ASYNC: the raw area is free again)
    if (ASYNC && t0 + TOK < n) fetch(t0 + TOK);
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = vs[tt * kRetCols + lane];
      const float4* kt = reinterpret_cast<const float4*>(ks + tt * DKP + warp * ROWS);
      const float4* qt = reinterpret_cast<const float4*>(qs + tt * DKP + warp * ROWS);
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS / 4; ++i) {
        const float4 k4 = kt[i], q4 = qt[i];
        S[4 * i] = fmaf(dec, S[4 * i], k4.x * vv);
        acc0 = fmaf(S[4 * i], q4.x, acc0);
        S[4 * i + 1] = fmaf(dec, S[4 * i + 1], k4.y * vv);
        acc1 = fmaf(S[4 * i + 1], q4.y, acc1);
        S[4 * i + 2] = fmaf(dec, S[4 * i + 2], k4.z * vv);
        acc0 = fmaf(S[4 * i + 2], q4.z, acc0);
        S[4 * i + 3] = fmaf(dec, S[4 * i + 3], k4.w * vv);
        acc1 = fmaf(S[4 * i + 3], q4.w, acc1);
      }
      part[(warp * TOK + tt) * kRetCols + lane] = acc0 + acc1;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += W) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w) sum += part[(w * TOK + tt) * kRetCols + lane];
      if (col_ok) o[((row0 + t0 + tt) * H + h) * (int64_t)dv + c] = sum;
    }
    // the next block's staging writes qs / ks / vs (last read before the barrier above) and its
    // accumulation writes part only after the barrier that follows the staging
  }
  if (keep_state && col_ok) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
      const int row = warp * ROWS + i;
      if (row < dk) st[(int64_t)row * dv + c] = S[i];
    }
  }
}

template <typename T, int W, int ROWS, bool ASYNC, int TOK>
int retention_launch(dim3 grid, size_t smem, cudaStream_t stream, float* o, const void* q, const void* k, const void* v,
                     float* state, const int64_t* req_pool_indices, const int64_t* seq_lens,
                     const int64_t* out_cache_loc, const int32_t* prefix_lens, const int32_t* extend_lens,
                     const int32_t* extend_start_loc, int H, int dk, int dv, int64_t q_stride, int64_t k_stride,
                     int64_t v_stride, const float* decay, const float* cos_sin, int rot, int64_t max_positions,
                     float k_scale, int in_act) {
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    SPD_CUDA(cudaFuncSetAttribute(retention_kernel<T, W, ROWS, ASYNC, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem));
    configured = smem;
  }
  SPD_CUDA(launch(retention_kernel<T, W, ROWS, ASYNC, TOK>, grid, dim3(W * 32), smem, stream, /*pdl=*/false, o, (const T*)q,
                  (const T*)k, (const T*)v, state, req_pool_indices, seq_lens, out_cache_loc, prefix_lens, extend_lens,
                  extend_start_loc, H, dk, dv, q_stride, k_stride, v_stride, decay, cos_sin, rot, max_positions,
                  k_scale, in_act));
  return 0;
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_retention(float* o, const void* q, const void* k, const void* v, float* state,
                  const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                  const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                  int64_t batch, int num_heads, int head_dim, int v_dim, int64_t q_stride, int64_t k_stride,
                  int64_t v_stride, const float* decay, const float* cos_sin, int rot_dims,
                  int64_t max_positions, float k_scale, int in_act, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(o && q && k && v && state && req_pool_indices && decay, SPD_E_BADARG, "spd_retention: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_retention: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(num_heads > 0 && head_dim > 0 && head_dim <= 256 && v_dim > 0, SPD_E_SHAPE,
              "spd_retention: head_dim %d above 256", head_dim);
  SPD_REQUIRE(rot_dims >= 0 && rot_dims <= head_dim && rot_dims % 2 == 0 && (rot_dims == 0 || (cos_sin && max_positions > 0)),
              SPD_E_BADARG, "spd_retention: bad rotation (rot_dims %d)", rot_dims);
  SPD_REQUIRE(in_act == 0 || in_act == 1, SPD_E_BADARG, "spd_retention: in_act is 0 (none) or 1 (SiLU)");
  if (batch == 0) return 0;
  const dim3 grid((unsigned)batch, (unsigned)num_heads, (unsigned)((v_dim + kRetCols - 1) / kRetCols));
  // warps x rows per thread covering head_dim: 8 rows per thread up to 128, 16 above
  const int warps = head_dim <= 32 ? 4 : head_dim <= 64 ? 8 : 16;
  const int dkp = head_dim <= 128 ? warps * 8 : 256;
  const bool decode = seq_lens != nullptr;
  const size_t tok = decode ? 1 : kRetTok;
  const size_t smem = sizeof(float) * ((size_t)2 * tok * dkp + tok * kRetCols + (size_t)warps * tok * kRetCols);
  // ragged extend with 16-byte aligned rows: the prefetching form
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  const bool async_ok = !decode && head_dim % vecn == 0 && v_dim % vecn == 0 && q_stride % vecn == 0 &&
                        k_stride % vecn == 0 && v_stride % vecn == 0 && rot_dims % 4 == 0 && aligned16(q) &&
                        aligned16(k) && aligned16(v) && (rot_dims == 0 || aligned16(cos_sin)) &&
                        getenv("SPD_RETENTION_SYNC") == nullptr;
  const size_t esz = dtype == SPD_F32 ? 4 : 2;
  const size_t smem_async = smem + sizeof(float) * kRetTok * (size_t)rot_dims + esz * kRetTok * (2 * (size_t)head_dim + kRetCols);
#define SPD_RET_ARGS                                                                                              \
  as_stream(stream), o, q, k, v, state, req_pool_indices, seq_lens, out_cache_loc, prefix_lens, extend_lens,      \
      extend_start_loc, num_heads, head_dim, v_dim, q_stride, k_stride, v_stride, decay, cos_sin, rot_dims,       \
      max_positions, k_scale, in_act
#define SPD_RET_SHAPE(W, ROWS)                                                                                    \
  return decode     ? retention_launch<T, W, ROWS, false, 1>(grid, smem, SPD_RET_ARGS)                            \
         : async_ok ? retention_launch<T, W, ROWS, true, kRetTok>(grid, smem_async, SPD_RET_ARGS)                 \
                    : retention_launch<T, W, ROWS, false, kRetTok>(grid, smem, SPD_RET_ARGS)
  SPD_DISPATCH_ANY(dtype, {
    if (head_dim <= 32) SPD_RET_SHAPE(4, 8);
    else if (head_dim <= 64) SPD_RET_SHAPE(8, 8);
    else if (head_dim <= 128) SPD_RET_SHAPE(16, 8);
    else SPD_RET_SHAPE(16, 16);
  });
#undef SPD_RET_SHAPE
#undef SPD_RET_ARGS
  return 0;
}

}  // extern "C"
