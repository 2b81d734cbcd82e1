// Softmax attention over the paged KV pool with the options the tcgen05 kernels do not have:
// a sliding window, a learned per-head sink in the denominator, a linear distance bias, a
// position-dependent query temperature, key size != value size, and 32-bit storage.  Decode and
// ragged extend (chunked prefill, mixed batches) are the same kernel: one warp owns one (query
// token, query head), walks its visible keys in tiles of 32 (one key per lane for the scores, one
// slice of the value row per lane for the output) and keeps the online-softmax state in fp32.
// The four warps of a CTA are four consecutive tokens of one head, so their K/V rows meet in L1.
// Beside attn_simt.cu (plain causal SIMT attention) in role; the reference has no such kernel.
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

constexpr int kGenMaxVPerLane = 16;  // v_dim <= 512: value columns a lane holds (instantiated for 8 and 16)
constexpr int kGenMaxHeadDim = 1024;  // key rows may be wider than value rows (a latent with a rotated slice)

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ krow, int dk);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ qs, const float* __restrict__ krow, int dk) {
  float s = 0.f;
  if ((dk & 3) == 0 && (reinterpret_cast<uintptr_t>(krow) & 15u) == 0) {
    for (int d = 0; d < dk; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(krow + d);
      s = fmaf(qs[d], kv.x, s);
      s = fmaf(qs[d + 1], kv.y, s);
      s = fmaf(qs[d + 2], kv.z, s);
      s = fmaf(qs[d + 3], kv.w, s);
    }
  } else {
    for (int d = 0; d < dk; ++d) s = fmaf(qs[d], krow[d], s);
  }
  return s;
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ krow, int dk) {
  float s = 0.f;
  if ((dk & 7) == 0 && (reinterpret_cast<uintptr_t>(krow) & 15u) == 0) {
    for (int d = 0; d < dk; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(qs[d + i], to_f32<T>(e[i]), s);
    }
  } else {
    for (int d = 0; d < dk; ++d) s = fmaf(qs[d], to_f32<T>(krow[d]), s);
  }
  return s;
}

template <typename T, int VMAX>
__global__ void __launch_bounds__(128)
attn_general_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool,
                    const T* __restrict__ v_pool, const int32_t* __restrict__ req_to_token,
                    const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens,
                    const int32_t* __restrict__ prefix_lens, const int32_t* __restrict__ extend_lens,
                    const int32_t* __restrict__ extend_start_loc, int batch, int64_t total_tokens, int H, int G,
                    int dk, int dv, int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale,
                    int window, const float* __restrict__ sinks, const float* __restrict__ slopes, float qtemp_coef,
                    int qtemp_every, float softcap, int Gv, int64_t v_slot) {
  extern __shared__ float q_smem[];  // [4][dk]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // item = h * tokens_padded + t with tokens_padded a multiple of 4: the warps of a CTA share a head
  const int64_t tokens4 = (total_tokens + 3) / 4 * 4;
  const int64_t item = blockIdx.x * 4ll + warp;
  const int h = (int)(item / tokens4);
  const int64_t t = item - (int64_t)h * tokens4;
  if (h >= H || t >= total_tokens) return;  // warp-uniform; no block-level barrier below

  int r;
  int64_t pos;
  if (seq_lens != nullptr) {
    r = (int)t;
    pos = seq_lens[r] - 1;
  } else {
    int lo = 0, hi = batch - 1;  // last request whose first row is <= t and that is not empty
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((int64_t)extend_start_loc[mid] <= t) lo = mid; else hi = mid - 1;
    }
    r = lo;
    while (r > 0 && extend_lens[r] == 0) --r;  // (empty entries share their successor's start)
    pos = (int64_t)prefix_lens[r] + (t - extend_start_loc[r]);
  }
  if (pos < 0) return;
  const int32_t* page = req_to_token + req_pool_indices[r] * r2t_stride;
  const int g = h / (H / G);

  float* qs = q_smem + warp * dk;
  float temp = 1.f;
  if (qtemp_every > 0) temp = 1.f + qtemp_coef * logf((float)((pos + 1) / qtemp_every + 1));
  const float qmul = sm_scale * temp;
  for (int d = lane; d < dk; d += 32) qs[d] = to_f32<T>(q[t * q_stride + (int64_t)h * dk + d]) * qmul;
  __syncwarp();

  const float slope = slopes != nullptr ? slopes[h] : 0.f;
  float m = -INFINITY, l = 0.f;
  if (sinks != nullptr) { m = sinks[h]; l = 1.f; }
  float acc[VMAX];
#pragma unroll
  for (int i = 0; i < VMAX; ++i) acc[i] = 0.f;

  const int64_t j_lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  for (int64_t j0 = j_lo; j0 <= pos; j0 += 32) {
    const int64_t j = j0 + lane;
    const bool valid = j <= pos;
    int slot = 0;
    float s = -INFINITY;
    if (valid) {
      slot = page[j];
      s = dot_row<T>(qs, k_pool + ((int64_t)slot * G + g) * dk, dk);
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      s -= slope * (float)(pos - j);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf (first tile, no sink): 0
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < VMAX; ++i) acc[i] *= corr;
    const int n = (int)(pos - j0 + 1 < 32 ? pos - j0 + 1 : 32);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vrow = v_pool + (int64_t)sj * v_slot + (int64_t)(g % Gv) * dv;
#pragma unroll
      for (int i = 0; i < VMAX; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] = fmaf(pj, to_f32<T>(vrow[c]), acc[i]);
      }
    }
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) out[t * out_stride + (int64_t)h * dv + c] = from_f32<T>(acc[i] * inv);
  }
}

// Decode: one CTA per (request, query head); its four warps take the key tiles of the window in turn
// (tile i goes to warp i mod 4) and their partial (max, sum, output) triples are merged through shared
// memory by warp 0 — four times the loads in flight per (request, head) of the one-warp form.
template <typename T, int VMAX>
__global__ void __launch_bounds__(128)
attn_general_decode_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool,
                           const T* __restrict__ v_pool, const int32_t* __restrict__ req_to_token,
                           const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens, int H,
                           int G, int dk, int dv, int64_t q_stride, int64_t out_stride, int64_t r2t_stride,
                           float sm_scale, int window, const float* __restrict__ sinks,
                           const float* __restrict__ slopes, float qtemp_coef, int qtemp_every, float softcap, int Gv,
                           int64_t v_slot) {
  extern __shared__ float dec_smem[];  // q [dk] | m [4] | l [4] | acc [4][dv]
  float* qs = dec_smem;
  float* sm_m = qs + dk;
  float* sm_l = sm_m + 4;
  float* sm_acc = sm_l + 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x, h = blockIdx.y;
  const int64_t pos = seq_lens[r] - 1;
  if (pos < 0) return;
  const int32_t* page = req_to_token + req_pool_indices[r] * r2t_stride;
  const int g = h / (H / G);
  float temp = 1.f;
  if (qtemp_every > 0) temp = 1.f + qtemp_coef * logf((float)((pos + 1) / qtemp_every + 1));
  const float qmul = sm_scale * temp;
  for (int d = threadIdx.x; d < dk; d += 128) qs[d] = to_f32<T>(q[(int64_t)r * q_stride + (int64_t)h * dk + d]) * qmul;
  __syncthreads();
  const float slope = slopes != nullptr ? slopes[h] : 0.f;
  float m = -INFINITY, l = 0.f;
  float acc[VMAX];
#pragma unroll
  for (int i = 0; i < VMAX; ++i) acc[i] = 0.f;
  const int64_t j_lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  for (int64_t j0 = j_lo + 32 * warp; j0 <= pos; j0 += 128) {
    const int64_t j = j0 + lane;
    const bool valid = j <= pos;
    int slot = 0;
    float s = -INFINITY;
    if (valid) {
      slot = page[j];
      s = dot_row<T>(qs, k_pool + ((int64_t)slot * G + g) * dk, dk);
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      s -= slope * (float)(pos - j);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < VMAX; ++i) acc[i] *= corr;
    const int n = (int)(pos - j0 + 1 < 32 ? pos - j0 + 1 : 32);
    for (int jj = 0; jj < n; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int sj = __shfl_sync(0xffffffffu, slot, jj);
      const T* vrow = v_pool + (int64_t)sj * v_slot + (int64_t)(g % Gv) * dv;
#pragma unroll
      for (int i = 0; i < VMAX; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] = fmaf(pj, to_f32<T>(vrow[c]), acc[i]);
      }
    }
  }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) sm_acc[warp * dv + c] = acc[i];
  }
  __syncthreads();
  if (warp != 0) return;
  float mt = sinks != nullptr ? sinks[h] : -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm_m[w]);
  float lt = sinks != nullptr ? expf(sinks[h] - mt) : 0.f;
  float f[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    f[w] = sm_m[w] == -INFINITY ? 0.f : expf(sm_m[w] - mt);  // a warp without keys contributes nothing
    lt += sm_l[w] * f[w];
  }
  const float inv = 1.0f / lt;
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) v += sm_acc[w * dv + c] * f[w];
      out[(int64_t)r * out_stride + (int64_t)h * dv + c] = from_f32<T>(v * inv);
    }
  }
}

// Decode over a whole key/value group: one CTA per (request, key/value head) serves the R = H / G query
// heads that share it, so a K / V row leaves the pool once per group instead of once per query head.
// The NW (8, or 4 where shared memory is short) warps take the key tiles of the window in turn (tile i
// goes to warp i mod NW).  A warp
// stages its tile of 32 keys in shared memory with 16-byte cp.async (rows padded by 16 bytes, so the
// per-lane row reads are bank-conflict free), scores one key per lane against all R queries (q in
// shared memory, fp32, pre-scaled), then walks the tile's V rows with VPL = v_dim / 32 contiguous
// columns per lane; online-softmax state per (warp, head) stays in registers and the warps' partial
// (max, sum, output) triples per head are merged through shared memory at the end, where the sink
// enters the denominator once.  Needs 16-byte rows (head_dim a multiple of 16 / sizeof(T)), v_dim in
// {32, 64, 128, 256} and R <= 8; other shapes take attn_general_decode_kernel.
template <typename T, int VPL>
__device__ __forceinline__ void load_cols(const unsigned char* p, float* f) {
  constexpr int BYTES = VPL * (int)sizeof(T);
  if constexpr (BYTES >= 16) {
#pragma unroll
    for (int b = 0; b < BYTES / 16; ++b) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + 16 * b);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 16 / (int)sizeof(T); ++i) f[b * (16 / (int)sizeof(T)) + i] = to_f32<T>(e[i]);
    }
  } else if constexpr (BYTES == 8) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VPL; ++i) f[i] = to_f32<T>(e[i]);
  } else if constexpr (BYTES == 4) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VPL; ++i) f[i] = to_f32<T>(e[i]);
  } else {
    f[0] = to_f32<T>(*reinterpret_cast<const T*>(p));
  }
}

constexpr int kGrpWarpHdr = 128;  // bytes in front of a warp's tiles: its 32 slot numbers

template <typename T, int VPL, int RMAX, int NW>
__global__ void __launch_bounds__(NW * 32)
attn_general_decode_group_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool,
                                 const T* __restrict__ v_pool, const int32_t* __restrict__ req_to_token,
                                 const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens,
                                 int H, int G, int dk, int64_t q_stride, int64_t out_stride, int64_t r2t_stride,
                                 float sm_scale, int window, const float* __restrict__ sinks,
                                 const float* __restrict__ slopes, float qtemp_coef, int qtemp_every, int q_bytes,
                                 float softcap, int Gv, int64_t v_slot) {
  constexpr int N = 16 / (int)sizeof(T);
  constexpr int DV = 32 * VPL;
  constexpr int vstride = DV * (int)sizeof(T) + 16;
  extern __shared__ __align__(16) unsigned char gsm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x, g = blockIdx.y;
  const int R = H / G;
  const int64_t pos = seq_lens[r] - 1;
  if (pos < 0) return;
  const int kstride = dk * (int)sizeof(T) + 16;
  float* qs = reinterpret_cast<float*>(gsm);  // [R][dk]
  unsigned char* wbase = gsm + q_bytes + (size_t)warp * (kGrpWarpHdr + 32 * (kstride + vstride));
  int* slots = reinterpret_cast<int*>(wbase);
  unsigned char* kt = wbase + kGrpWarpHdr;
  unsigned char* vt = kt + 32 * kstride;
  const int32_t* page = req_to_token + req_pool_indices[r] * r2t_stride;
  float temp = 1.f;
  if (qtemp_every > 0) temp = 1.f + qtemp_coef * logf((float)((pos + 1) / qtemp_every + 1));
  const float qmul = sm_scale * temp;
  for (int idx = threadIdx.x; idx < R * dk; idx += NW * 32)
    qs[idx] = to_f32<T>(q[(int64_t)r * q_stride + (int64_t)g * R * dk + idx]) * qmul;
  __syncthreads();
  float slope[RMAX], m[RMAX], l[RMAX], acc[RMAX][VPL];
#pragma unroll
  for (int rr = 0; rr < RMAX; ++rr) {
    slope[rr] = (slopes != nullptr && rr < R) ? slopes[g * R + rr] : 0.f;
    m[rr] = -INFINITY;
    l[rr] = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[rr][i] = 0.f;
  }
  const int kc = dk / N;
  constexpr int vc = DV / N;
  // a row's 16-byte chunks go to consecutive lanes; rows short enough share an instruction
  const int k_rows = kc >= 32 ? 1 : 32 / kc, k_lrow = kc >= 32 ? 0 : lane / kc, k_lch = kc >= 32 ? lane : lane - k_lrow * kc;
  constexpr int v_rows = vc >= 32 ? 1 : 32 / vc;
  const int v_lrow = vc >= 32 ? 0 : lane / vc, v_lch = vc >= 32 ? lane : lane - v_lrow * vc;
  const int64_t j_lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  for (int64_t j0 = j_lo + 32 * warp; j0 <= pos; j0 += 32 * NW) {
    const int n = (int)(pos - j0 + 1 < 32 ? pos - j0 + 1 : 32);
    const bool valid = lane < n;
    __syncwarp();  // the previous tile has been read
    if (valid) slots[lane] = page[j0 + lane];
    __syncwarp();
    if (lane < k_rows * kc)
      for (int kk = k_lrow; kk < n; kk += k_rows) {
        const T* src = k_pool + ((int64_t)slots[kk] * G + g) * dk;
        for (int ch = k_lch; ch < kc; ch += 32) cp_async16(smem_u32(kt + kk * kstride + ch * 16), src + ch * N, true);
      }
    if (lane < v_rows * vc)
      for (int kk = v_lrow; kk < n; kk += v_rows) {
        const T* src = v_pool + (int64_t)slots[kk] * v_slot + (int64_t)(g % Gv) * DV;
#pragma unroll
        for (int ch = v_lch; ch < vc; ch += 32) cp_async16(smem_u32(vt + kk * vstride + ch * 16), src + ch * N, true);
      }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    float s[RMAX];
#pragma unroll
    for (int rr = 0; rr < RMAX; ++rr) s[rr] = 0.f;
    if (valid) {
      const unsigned char* krow = kt + lane * kstride;
#pragma unroll 2
      for (int d = 0; d < dk; d += N) {
        float kf[N];
        load_cols<T, N>(krow + d * (int)sizeof(T), kf);
#pragma unroll
        for (int rr = 0; rr < RMAX; ++rr) {
          if (rr < R) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + rr * dk + d);
#pragma unroll
            for (int i = 0; i < N / 4; ++i) {
              const float4 qq = q4[i];
              s[rr] = fmaf(qq.x, kf[4 * i], s[rr]);
              s[rr] = fmaf(qq.y, kf[4 * i + 1], s[rr]);
              s[rr] = fmaf(qq.z, kf[4 * i + 2], s[rr]);
              s[rr] = fmaf(qq.w, kf[4 * i + 3], s[rr]);
            }
          }
        }
      }
    }
    const float dist = (float)(pos - (j0 + lane));
    float p[RMAX];
#pragma unroll
    for (int rr = 0; rr < RMAX; ++rr) {
      p[rr] = 0.f;
      if (rr < R) {
        const float sc = softcap > 0.f ? softcap * tanhf(s[rr] / softcap) : s[rr];
        const float sv = valid ? sc - slope[rr] * dist : -INFINITY;
        const float m_new = fmaxf(m[rr], warp_max(sv));  // finite: the tile has at least one key
        const float corr = expf(m[rr] - m_new);          // first tile (m = -inf): 0
        p[rr] = valid ? expf(sv - m_new) : 0.f;
        l[rr] = l[rr] * corr + warp_sum(p[rr]);
        m[rr] = m_new;
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[rr][i] *= corr;
      }
    }
#pragma unroll 4
    for (int jj = 0; jj < n; ++jj) {
      float vf[VPL];
      load_cols<T, VPL>(vt + jj * vstride + lane * VPL * (int)sizeof(T), vf);
#pragma unroll
      for (int rr = 0; rr < RMAX; ++rr) {
        if (rr < R) {
          const float pj = __shfl_sync(0xffffffffu, p[rr], jj);
#pragma unroll
          for (int i = 0; i < VPL; ++i) acc[rr][i] = fmaf(pj, vf[i], acc[rr][i]);
        }
      }
    }
  }
  __syncthreads();  // the tiles are dead: their shared memory carries the partials
  float* sm_acc = reinterpret_cast<float*>(gsm + q_bytes);  // [NW][R][DV]
  float* sm_m = sm_acc + NW * R * DV;                       // [NW][R]
  float* sm_l = sm_m + NW * R;                              // [NW][R]
#pragma unroll
  for (int rr = 0; rr < RMAX; ++rr) {
    if (rr < R) {
      if (lane == 0) { sm_m[warp * R + rr] = m[rr]; sm_l[warp * R + rr] = l[rr]; }
#pragma unroll
      for (int i = 0; i < VPL; ++i) sm_acc[(warp * R + rr) * DV + lane * VPL + i] = acc[rr][i];
    }
  }
  __syncthreads();
  for (int rr = warp; rr < R; rr += NW) {
    const int h = g * R + rr;
    float mt = sinks != nullptr ? sinks[h] : -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mt = fmaxf(mt, sm_m[w * R + rr]);
    float lt = sinks != nullptr ? expf(sinks[h] - mt) : 0.f;
    float f[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      f[w] = sm_m[w * R + rr] == -INFINITY ? 0.f : expf(sm_m[w * R + rr] - mt);  // a warp without keys adds nothing
      lt += sm_l[w * R + rr] * f[w];
    }
    const float inv = 1.0f / lt;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane * VPL + i;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) v += sm_acc[(w * R + rr) * DV + c] * f[w];
      out[(int64_t)r * out_stride + (int64_t)h * DV + c] = from_f32<T>(v * inv);
    }
  }
}

template <typename T, int VPL, int RMAX, int NW>
int attn_general_decode_group_launch(size_t smem, int q_bytes, int64_t batch, cudaStream_t stream, void* out, const void* q,
                                     const void* k_pool, const void* v_pool, const int32_t* req_to_token,
                                     const int64_t* req_pool_indices, const int64_t* seq_lens, int H, int G, int dk,
                                     int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                                     const float* sinks, const float* slopes, float qtemp_coef, int qtemp_every,
                                     float softcap, int Gv, int64_t v_slot) {
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    SPD_CUDA(cudaFuncSetAttribute(attn_general_decode_group_kernel<T, VPL, RMAX, NW>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  SPD_CUDA(launch(attn_general_decode_group_kernel<T, VPL, RMAX, NW>, dim3((unsigned)batch, (unsigned)G), dim3(NW * 32), smem,
                  stream, /*pdl=*/false, (T*)out, (const T*)q, (const T*)k_pool, (const T*)v_pool, req_to_token,
                  req_pool_indices, seq_lens, H, G, dk, q_stride, out_stride, r2t_stride, sm_scale, window, sinks, slopes,
                  qtemp_coef, qtemp_every, q_bytes, softcap, Gv, v_slot));
  return 0;
}

template <typename T>
__global__ void __launch_bounds__(256)
kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ k_pool, T* __restrict__ v_pool,
                const int64_t* __restrict__ loc, int64_t k_row, int64_t v_row, int64_t k_stride, int64_t v_stride) {
  const int64_t t = blockIdx.x;
  const int64_t slot = loc[t];
  for (int64_t i = threadIdx.x; i < k_row; i += 256) k_pool[slot * k_row + i] = k[t * k_stride + i];
  if (v != nullptr)
    for (int64_t i = threadIdx.x; i < v_row; i += 256) v_pool[slot * v_row + i] = v[t * v_stride + i];
}

int attn_general_mma_try(void* out, const void* q, const void* k_pool, const void* v_pool, const int32_t* req_to_token,
                         const int64_t* req_pool_indices, const int32_t* prefix_lens, const int32_t* extend_lens,
                         const int32_t* extend_start_loc, int64_t batch, int64_t max_extend_len, int H, int G, int dk,
                         int dv, int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                         const float* sinks, const float* slopes, float qtemp_coef, int qtemp_every, float softcap,
                         int Gv, int64_t v_slot, int dtype, cudaStream_t stream);

int attn_general_mma_decode_try(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                                int64_t batch, int H, int G, int dk, int dv, int64_t q_stride, int64_t out_stride,
                                int64_t r2t_stride, float sm_scale, int window, const float* sinks, const float* slopes,
                                float qtemp_coef, int qtemp_every, float softcap, int Gv, int64_t v_slot, int dtype,
                                cudaStream_t stream);

}  // namespace spd

using namespace spd;

extern "C" {

int spd_kv_store(const void* k, const void* v, void* k_pool, void* v_pool, const int64_t* loc,
                 int64_t tokens, int64_t k_row_elems, int64_t v_row_elems, int64_t k_stride,
                 int64_t v_stride, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(k && k_pool && loc && (v == nullptr || v_pool), SPD_E_BADARG, "spd_kv_store: null pointer");
  SPD_REQUIRE(tokens >= 0 && k_row_elems > 0 && v_row_elems >= 0, SPD_E_BADARG, "spd_kv_store: bad sizes");
  if (tokens == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(kv_store_kernel<T>, dim3((unsigned)tokens), dim3(256), 0, as_stream(stream), /*pdl=*/false,
                    (const T*)k, (const T*)v, (T*)k_pool, (T*)v_pool, loc, k_row_elems, v_row_elems, k_stride,
                    v_stride));
  });
  return 0;
}

int spd_attn_general_ex(void* out, const void* q, const void* k_pool, const void* v_pool,
                        const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                        const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                        int64_t batch, int64_t total_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                        int v_dim, int64_t q_stride, int64_t out_stride, int64_t req_to_token_stride,
                        float sm_scale, int window, const float* sinks, const float* slopes, float qtemp_coef,
                        int qtemp_every, int64_t max_extend_len, float softcap, int num_v_heads,
                        int64_t v_slot_stride, int dtype, spd_stream_t stream) {
  if (num_v_heads <= 0) num_v_heads = num_kv_heads;
  if (v_slot_stride <= 0) v_slot_stride = (int64_t)num_v_heads * v_dim;
  const int Gv = num_v_heads;
  const int64_t v_slot = v_slot_stride;
  SPD_REQUIRE(num_kv_heads % num_v_heads == 0 && softcap >= 0.f, SPD_E_SHAPE,
              "spd_attn_general: kv heads %d not a multiple of value heads %d", num_kv_heads, num_v_heads);
  SPD_REQUIRE(out && q && k_pool && v_pool && req_to_token && req_pool_indices, SPD_E_BADARG,
              "spd_attn_general: null pointer");
  SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
              "spd_attn_general: extend needs prefix_lens, extend_lens and extend_start_loc");
  SPD_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, SPD_E_SHAPE,
              "spd_attn_general: heads %d not a multiple of kv heads %d", num_q_heads, num_kv_heads);
  SPD_REQUIRE(head_dim > 0 && head_dim <= kGenMaxHeadDim && v_dim > 0 && v_dim <= 32 * kGenMaxVPerLane, SPD_E_SHAPE,
              "spd_attn_general: head_dim %d / v_dim %d above %d", head_dim, v_dim, kGenMaxHeadDim);
  SPD_REQUIRE(seq_lens == nullptr || batch == total_tokens, SPD_E_BADARG, "spd_attn_general: decode has one row per request");
  if (total_tokens == 0 || batch == 0) return 0;
  if (seq_lens != nullptr) {
    SPD_REQUIRE(batch < (1ll << 31) && num_q_heads <= 65535, SPD_E_SHAPE, "spd_attn_general: batch too large");
    // 16-bit models, instantiated head sizes: the tensor-core form (SPD_ATTN_DECODE_SIMT=1 keeps the CUDA cores)
    if (getenv("SPD_ATTN_DECODE_SIMT") == nullptr) {
      const int rc = attn_general_mma_decode_try(out, q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens, batch,
                                                 num_q_heads, num_kv_heads, head_dim, v_dim, q_stride, out_stride,
                                                 req_to_token_stride, sm_scale, window, sinks, slopes, qtemp_coef,
                                                 qtemp_every, softcap, Gv, v_slot, dtype, as_stream(stream));
      if (rc != 1) return rc;
    }
    // grouped form: 16-byte rows, v_dim 32 x {1, 2, 4, 8}, up to 8 query heads per key/value head
    const int R = num_q_heads / num_kv_heads;
    const size_t esz = dtype == SPD_F32 ? 4 : 2;
    const int q_bytes = (int)((sizeof(float) * (size_t)R * head_dim + 15) / 16 * 16);
    const size_t warp_tiles = (size_t)kGrpWarpHdr + 32 * (esz * head_dim + 16 + esz * v_dim + 16);
    const size_t warp_merge = sizeof(float) * (size_t)R * ((size_t)v_dim + 2);
    const size_t per_warp = warp_tiles > warp_merge ? warp_tiles : warp_merge;
    const int nw = (size_t)q_bytes + 8 * per_warp <= 160 * 1024 ? 8 : 4;  // eight warps where their tiles fit
    const size_t gsmem = (size_t)q_bytes + nw * per_warp;
    const bool grouped = (dtype == SPD_F32 || dtype == SPD_BF16) && R <= 8 && head_dim % (16 / (int)esz) == 0 &&
                         (v_dim == 32 || v_dim == 64 || v_dim == 128 || v_dim == 256) && aligned16(k_pool) &&
                         aligned16(v_pool) && v_slot % (16 / (int64_t)esz) == 0 && gsmem <= 200 * 1024 && num_kv_heads <= 65535 &&
                         getenv("SPD_ATTN_DECODE_PER_HEAD") == nullptr;
    if (grouped) {
#define SPD_GRP_ARGS                                                                                                  \
  gsmem, q_bytes, batch, as_stream(stream), out, q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens,         \
      num_q_heads, num_kv_heads, head_dim, q_stride, out_stride, req_to_token_stride, sm_scale, window, sinks, slopes, \
      qtemp_coef, qtemp_every, softcap, Gv, v_slot
#define SPD_GRP_R(TT, VPL)                                                                     \
  do {                                                                                         \
    if (R <= 1) return nw == 8 ? attn_general_decode_group_launch<TT, VPL, 1, 8>(SPD_GRP_ARGS)  \
                               : attn_general_decode_group_launch<TT, VPL, 1, 4>(SPD_GRP_ARGS); \
    if (R <= 2) return nw == 8 ? attn_general_decode_group_launch<TT, VPL, 2, 8>(SPD_GRP_ARGS)  \
                               : attn_general_decode_group_launch<TT, VPL, 2, 4>(SPD_GRP_ARGS); \
    if (R <= 4) return nw == 8 ? attn_general_decode_group_launch<TT, VPL, 4, 8>(SPD_GRP_ARGS)  \
                               : attn_general_decode_group_launch<TT, VPL, 4, 4>(SPD_GRP_ARGS); \
    return nw == 8 ? attn_general_decode_group_launch<TT, VPL, 8, 8>(SPD_GRP_ARGS)              \
                   : attn_general_decode_group_launch<TT, VPL, 8, 4>(SPD_GRP_ARGS);             \
  } while (0)
#define SPD_GRP_V(TT)                                                                          \
  do {                                                                                         \
    if (v_dim == 32) SPD_GRP_R(TT, 1);                                                         \
    else if (v_dim == 64) SPD_GRP_R(TT, 2);                                                    \
    else if (v_dim == 128) SPD_GRP_R(TT, 4);                                                   \
    else SPD_GRP_R(TT, 8);                                                                     \
  } while (0)
      if (dtype == SPD_F32) SPD_GRP_V(float);
      else SPD_GRP_V(__nv_bfloat16);
#undef SPD_GRP_V
#undef SPD_GRP_R
#undef SPD_GRP_ARGS
    }
    const size_t dsmem = sizeof(float) * ((size_t)head_dim + 8 + 4 * (size_t)v_dim);
    SPD_DISPATCH_ANY(dtype, {
      auto kern = v_dim <= 256 ? attn_general_decode_kernel<T, 8> : attn_general_decode_kernel<T, 16>;
      SPD_CUDA(launch(kern, dim3((unsigned)batch, (unsigned)num_q_heads), dim3(128), dsmem,
                      as_stream(stream), /*pdl=*/false, (T*)out, (const T*)q, (const T*)k_pool, (const T*)v_pool,
                      req_to_token, req_pool_indices, seq_lens, num_q_heads, num_kv_heads, head_dim, v_dim, q_stride,
                      out_stride, req_to_token_stride, sm_scale, window, sinks, slopes, qtemp_coef, qtemp_every, softcap,
                      Gv, v_slot));
    });
    return 0;
  }
  if (max_extend_len > 0) {  // 16-bit prefill on the tensor cores where the head sizes are instantiated
    const int rc = attn_general_mma_try(out, q, k_pool, v_pool, req_to_token, req_pool_indices, prefix_lens, extend_lens,
                                        extend_start_loc, batch, max_extend_len, num_q_heads, num_kv_heads, head_dim,
                                        v_dim, q_stride, out_stride, req_to_token_stride, sm_scale, window, sinks, slopes,
                                        qtemp_coef, qtemp_every, softcap, Gv, v_slot, dtype, as_stream(stream));
    if (rc != 1) return rc;
  }
  const int64_t tokens4 = (total_tokens + 3) / 4 * 4;
  const int64_t ctas = tokens4 / 4 * num_q_heads;
  SPD_REQUIRE(ctas < (1ll << 31), SPD_E_SHAPE, "spd_attn_general: batch too large");
  const size_t smem = 4 * (size_t)head_dim * sizeof(float);
  SPD_DISPATCH_ANY(dtype, {
    auto kern = v_dim <= 256 ? attn_general_kernel<T, 8> : attn_general_kernel<T, 16>;
    SPD_CUDA(launch(kern, dim3((unsigned)ctas), dim3(128), smem, as_stream(stream), /*pdl=*/false,
                    (T*)out, (const T*)q, (const T*)k_pool, (const T*)v_pool, req_to_token, req_pool_indices, seq_lens,
                    prefix_lens, extend_lens, extend_start_loc, (int)batch, total_tokens, num_q_heads, num_kv_heads,
                    head_dim, v_dim, q_stride, out_stride, req_to_token_stride, sm_scale, window, sinks, slopes,
                    qtemp_coef, qtemp_every, softcap, Gv, v_slot));
  });
  return 0;
}

int spd_attn_general(void* out, const void* q, const void* k_pool, const void* v_pool,
                     const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                     const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                     int64_t batch, int64_t total_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                     int v_dim, int64_t q_stride, int64_t out_stride, int64_t req_to_token_stride,
                     float sm_scale, int window, const float* sinks, const float* slopes, float qtemp_coef,
                     int qtemp_every, int64_t max_extend_len, int dtype, spd_stream_t stream) {
  return spd_attn_general_ex(out, q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens, prefix_lens, extend_lens,
                             extend_start_loc, batch, total_tokens, num_q_heads, num_kv_heads, head_dim, v_dim, q_stride,
                             out_stride, req_to_token_stride, sm_scale, window, sinks, slopes, qtemp_coef, qtemp_every,
                             max_extend_len, 0.f, 0, 0, dtype, stream);
}

}  // extern "C"
