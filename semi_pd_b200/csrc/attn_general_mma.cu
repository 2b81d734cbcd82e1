// Tensor-core prefill path of the general attention (window, sink, distance bias, query temperature,
// key size != value size) for 16-bit models: a CTA owns 64 consecutive query rows of one request and
// one query head, its four warps 16 rows each; K / V tiles of 64 keys are gathered through the page
// table with 16-byte cp.async into a double-buffered shared-memory ring, S = Q K^T and O += P V run
// on warp-level mma.sync.m16n8k16 (fp32 accumulators), and the online softmax — scale, temperature,
// bias, window mask, sink — is fp32 in the exp2 domain.  Only the keys a tile can see are visited:
// [first row - window + 1, last row].  The CUDA-core kernel of attn_general.cu keeps decode, float32
// models and head sizes outside the instantiated set.  (mma.sync, not tcgen05: the first tensor-core
// kernel of this mechanism.)
#include "common.cuh"
#include "ptx.cuh"
#include <stdlib.h>

namespace spd {

constexpr int kGmBQ = 64, kGmBK = 64, kGmThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ void gm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void gm_mma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void gm_mma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gm_ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void gm_ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}

// tanh for the score cap of the 16-bit kernels: 1 - 2 / (e^(2x) + 1) on the fast exponential and division (absolute
// error of a few 1e-7; the argument is clamped where tanh is 1 to fp32 precision).  The 32-bit kernels call tanhf.
__device__ __forceinline__ float gm_tanh(float x) {
  x = fminf(fmaxf(x, -15.f), 15.f);
  return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);
}

template <typename T, int DK, int DV>
__global__ void __launch_bounds__(kGmThreads)
attn_general_mma_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool,
                        const T* __restrict__ v_pool, const int32_t* __restrict__ req_to_token,
                        const int64_t* __restrict__ req_pool_indices, const int32_t* __restrict__ prefix_lens,
                        const int32_t* __restrict__ extend_lens, const int32_t* __restrict__ extend_start_loc, int H,
                        int G, int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                        const float* __restrict__ sinks, const float* __restrict__ slopes, float qtemp_coef,
                        int qtemp_every, float softcap, int Gv, int64_t v_slot) {
  constexpr int LDK = DK + 8, LDV = DV + 8;  // +16 B per row: ldmatrix rows fall into distinct banks
  extern __shared__ __align__(16) unsigned char gm_smem[];
  T* sQ = reinterpret_cast<T*>(gm_smem);   // [BQ][LDK]
  T* sK = sQ + kGmBQ * LDK;                // [2][BK][LDK]
  T* sV = sK + 2 * kGmBK * LDK;            // [2][BK][LDV]
  const int r = blockIdx.y, h = blockIdx.z;
  const int ext = extend_lens[r];
  const int q0 = blockIdx.x * kGmBQ;
  if (q0 >= ext) return;
  const int nq = ext - q0 < kGmBQ ? ext - q0 : kGmBQ;
  const int64_t i0 = (int64_t)prefix_lens[r] + q0;        // position of the tile's first query
  const int64_t row0 = (int64_t)extend_start_loc[r] + q0;  // its row in q / out
  const int32_t* page = req_to_token + req_pool_indices[r] * r2t_stride;
  const int g = h / (H / G);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int idx = tid; idx < kGmBQ * (DK / 8); idx += kGmThreads) {
    const int row = idx / (DK / 8), c = idx % (DK / 8);
    const bool ok = row < nq;
    cp_async16(smem_u32(sQ + row * LDK + c * 8), q + (row0 + (ok ? row : 0)) * q_stride + (int64_t)h * DK + c * 8, ok);
  }
  const int64_t j_hi = i0 + nq - 1;
  const int64_t j_lo = window > 0 ? (i0 - window + 1 > 0 ? i0 - window + 1 : 0) : 0;
  const int ntiles = (int)((j_hi - j_lo) / kGmBK) + 1;
  auto load_kv = [&](int t, int buf) {
    const int64_t jb = j_lo + (int64_t)t * kGmBK;
    for (int idx = tid; idx < kGmBK * (DK / 8); idx += kGmThreads) {
      const int row = idx / (DK / 8), c = idx % (DK / 8);
      const bool ok = jb + row <= j_hi;
      const int64_t slot = ok ? page[jb + row] : 0;
      cp_async16(smem_u32(sK + (buf * kGmBK + row) * LDK + c * 8), k_pool + (slot * G + g) * DK + c * 8, ok);
    }
    for (int idx = tid; idx < kGmBK * (DV / 8); idx += kGmThreads) {
      const int row = idx / (DV / 8), c = idx % (DV / 8);
      const bool ok = jb + row <= j_hi;
      const int64_t slot = ok ? page[jb + row] : 0;
      cp_async16(smem_u32(sV + (buf * kGmBK + row) * LDV + c * 8), v_pool + slot * v_slot + (int64_t)(g % Gv) * DV + c * 8, ok);
    }
  };
  load_kv(0, 0);
  cp_async_commit();

  const int rl[2] = {warp * 16 + (lane >> 2), warp * 16 + (lane >> 2) + 8};
  const int64_t pi[2] = {i0 + rl[0], i0 + rl[1]};
  float sc[2], scc[2];  // score multipliers into the exp2 domain, and (with a cap) into units of the cap
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    float temp = 1.f;
    if (qtemp_every > 0) temp = 1.f + qtemp_coef * logf((float)((pi[x] + 1) / qtemp_every + 1));
    scc[x] = softcap > 0.f ? sm_scale * temp / softcap : 0.f;
    sc[x] = sm_scale * temp * kLog2e;
  }
  const float capl = softcap * kLog2e;
  const float sl = (slopes != nullptr ? slopes[h] : 0.f) * kLog2e;
  const float sink2 = sinks != nullptr ? sinks[h] * kLog2e : -INFINITY;
  float m[2] = {sink2, sink2}, l[2] = {0.f, 0.f};  // l: this thread's share of the row sum
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;

  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) {
      load_kv(t + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    float s[kGmBK / 8][4];
#pragma unroll
    for (int i = 0; i < kGmBK / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk) {
      uint32_t a[4];
      gm_ldsm_x4(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nb2 = 0; nb2 < kGmBK / 16; ++nb2) {
        uint32_t b[4];
        gm_ldsm_x4(b, sK + (buf * kGmBK + nb2 * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
        gm_mma<T>(s[2 * nb2], a, b[0], b[1]);
        gm_mma<T>(s[2 * nb2 + 1], a, b[2], b[3]);
      }
    }
    const int64_t jb = j_lo + (int64_t)t * kGmBK;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < kGmBK / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int x = e >> 1;
        const int64_t j = jb + nb * 8 + (lane & 3) * 2 + (e & 1);
        const int64_t dist = pi[x] - j;
        const bool ok = dist >= 0 && (window <= 0 || dist < window) && pi[x] <= j_hi;
        const float z = softcap > 0.f ? capl * gm_tanh(s[nb][e] * scc[x]) : s[nb][e] * sc[x];
        const float v = ok ? z - sl * (float)dist : -INFINITY;
        s[nb][e] = v;
        mx[x] = fmaxf(mx[x], v);
      }
    float ms[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
      const float m_new = fmaxf(m[x], mx[x]);
      ms[x] = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m[x] - ms[x]);  // m = -inf: 0 (nothing accumulated yet)
      m[x] = m_new;
      l[x] *= corr;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        o[i][2 * x] *= corr;
        o[i][2 * x + 1] *= corr;
      }
    }
#pragma unroll
    for (int nb = 0; nb < kGmBK / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nb][e] - ms[e >> 1]);
        s[nb][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int kk = 0; kk < kGmBK / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nb2 = 0; nb2 < DV / 16; ++nb2) {
        uint32_t b[4];
        gm_ldsm_x4_trans(b, sV + (buf * kGmBK + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + nb2 * 16 + (lane >> 4) * 8);
        gm_mma<T>(o[2 * nb2], a, b[0], b[1]);
        gm_mma<T>(o[2 * nb2 + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // the next iteration's prefetch overwrites the buffer just read
  }
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    float sum = l[x];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (sinks != nullptr) sum += exp2f(sink2 - m[x]);
    if (rl[x] < nq) {
      const float inv = 1.0f / sum;
      T* dst = out + (row0 + rl[x]) * out_stride + (int64_t)h * DV + (lane & 3) * 2;
#pragma unroll
      for (int nb = 0; nb < DV / 8; ++nb)
        *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack2<T>(o[nb][2 * x] * inv, o[nb][2 * x + 1] * inv);
    }
  }
}

template <typename T, int DK, int DV>
static int gm_launch(void* out, const void* q, const void* k_pool, const void* v_pool, const int32_t* req_to_token,
                     const int64_t* req_pool_indices, const int32_t* prefix_lens, const int32_t* extend_lens,
                     const int32_t* extend_start_loc, int64_t batch, int64_t max_extend_len, int H, int G,
                     int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                     const float* sinks, const float* slopes, float qtemp_coef, int qtemp_every, float softcap, int Gv,
                     int64_t v_slot, cudaStream_t stream) {
  constexpr size_t smem = sizeof(T) * ((size_t)kGmBQ * (DK + 8) + 2 * kGmBK * (DK + 8) + 2 * kGmBK * (DV + 8));
  static bool configured = false;  // per instantiation
  if (!configured) {
    SPD_CUDA(cudaFuncSetAttribute(attn_general_mma_kernel<T, DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const dim3 grid((unsigned)((max_extend_len + kGmBQ - 1) / kGmBQ), (unsigned)batch, (unsigned)H);
  SPD_CUDA(launch(attn_general_mma_kernel<T, DK, DV>, grid, dim3(kGmThreads), smem, stream, /*pdl=*/false, (T*)out,
                  (const T*)q, (const T*)k_pool, (const T*)v_pool, req_to_token, req_pool_indices, prefix_lens,
                  extend_lens, extend_start_loc, H, G, q_stride, out_stride, r2t_stride, sm_scale, window, sinks, slopes,
                  qtemp_coef, qtemp_every, softcap, Gv, v_slot));
  return 0;
}

// → 0 launched, 1 not applicable (the caller falls back to the CUDA-core kernel), else an error
int attn_general_mma_try(void* out, const void* q, const void* k_pool, const void* v_pool, const int32_t* req_to_token,
                         const int64_t* req_pool_indices, const int32_t* prefix_lens, const int32_t* extend_lens,
                         const int32_t* extend_start_loc, int64_t batch, int64_t max_extend_len, int H, int G, int dk,
                         int dv, int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                         const float* sinks, const float* slopes, float qtemp_coef, int qtemp_every, float softcap,
                         int Gv, int64_t v_slot, int dtype, cudaStream_t stream) {
  if (dtype != SPD_BF16 && dtype != SPD_F16) return 1;
  if (v_slot % 8 != 0) return 1;
  if (max_extend_len < 16 || batch > 65535 || H > 65535) return 1;  // short portions: the CUDA-core kernel
  if (q_stride % 8 != 0 || out_stride % 2 != 0 || !aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool) ||
      (reinterpret_cast<uintptr_t>(out) & 3u) != 0)
    return 1;
#define SPD_GM_CASE(DKV, DVV)                                                                                       \
  if (dk == DKV && dv == DVV) {                                                                                     \
    if (dtype == SPD_BF16)                                                                                          \
      return gm_launch<__nv_bfloat16, DKV, DVV>(out, q, k_pool, v_pool, req_to_token, req_pool_indices, prefix_lens, \
                                                extend_lens, extend_start_loc, batch, max_extend_len, H, G, q_stride, \
                                                out_stride, r2t_stride, sm_scale, window, sinks, slopes, qtemp_coef, \
                                                qtemp_every, softcap, Gv, v_slot, stream);                          \
    return gm_launch<__half, DKV, DVV>(out, q, k_pool, v_pool, req_to_token, req_pool_indices, prefix_lens,        \
                                       extend_lens, extend_start_loc, batch, max_extend_len, H, G, q_stride,        \
                                       out_stride, r2t_stride, sm_scale, window, sinks, slopes, qtemp_coef,         \
                                       qtemp_every, softcap, Gv, v_slot, stream);                                   \
  }
  SPD_GM_CASE(32, 32)
  SPD_GM_CASE(64, 64)
  SPD_GM_CASE(64, 128)
  SPD_GM_CASE(128, 64)
  SPD_GM_CASE(128, 128)
  SPD_GM_CASE(192, 128)
#undef SPD_GM_CASE
  return 1;
}

// ------------------------------------------------------------------------------------------------
// Decode on the tensor cores: one CTA per (request, key/value head) — per 16 of its query heads where more
// than 16 share it; the R <= 16 query heads are the 16 rows of the MMA's A operand (rows >= R are zero), so a K / V row leaves
// the pool once per group and a tile of 32 keys costs 2 * DK / 16 + DV / 4 MMAs instead of 64 R FMAs
// per lane.  The NW warps take the window's key tiles in turn (tile i goes to warp i mod NW); a warp
// stages its own tile with 16-byte cp.async (rows past the end are zero-filled) and keeps the
// online-softmax state of the 16 rows in the accumulator layout; at the end the warps' partial
// (max, sum, output) triples meet in shared memory, where the sink enters the denominator once.
// Everything but the two products' operands (q, k, v, and P rounded to 16 bits) is fp32.
// Few (request, head) pairs (small batches, one shared key/value head): the keys are split over the
// gridDim.z CTAs of a thread-block cluster (tile i goes to warp i mod (NW gridDim.z) of the cluster);
// each CTA merges its warps, the CTA of rank 0 then merges the CTAs' triples out of their shared
// memory (distributed shared memory) between two cluster barriers — no workspace in global memory.
// ------------------------------------------------------------------------------------------------
constexpr int kGdTK = 32;        // keys per warp tile
constexpr int kGdWarpHdr = 128;  // bytes in front of a warp's tiles: its slot numbers

template <typename T, int DK, int DV, int NW>
__global__ void __launch_bounds__(NW * 32)
attn_general_mma_decode_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool,
                               const T* __restrict__ v_pool, const int32_t* __restrict__ req_to_token,
                               const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens,
                               int H, int G, int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale,
                               int window, const float* __restrict__ sinks, const float* __restrict__ slopes,
                               float qtemp_coef, int qtemp_every, float softcap, int Gv, int64_t v_slot) {
  constexpr int LDK = DK + 8, LDV = DV + 8;
  constexpr size_t kQBytes = sizeof(T) * 16 * LDK;
  constexpr size_t kWarpBytes = kGdWarpHdr + sizeof(T) * kGdTK * (LDK + LDV);
  extern __shared__ __align__(16) unsigned char gd_smem[];
  T* sQ = reinterpret_cast<T*>(gd_smem);  // [16][LDK], rows >= R zero
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // a group of more than 16 query heads takes several CTAs of 16 rows each (blockIdx.y = head * chunks + chunk)
  const int chunks = (H / G + 15) / 16;
  const int r = blockIdx.x, g = blockIdx.y / chunks;
  const int h0 = g * (H / G) + (blockIdx.y % chunks) * 16;  // this CTA's first query head
  const int R = H / G - (blockIdx.y % chunks) * 16 < 16 ? H / G - (blockIdx.y % chunks) * 16 : 16;
  const int64_t pos = seq_lens[r] - 1;
  if (pos < 0) return;
  unsigned char* wbase = gd_smem + kQBytes + (size_t)warp * kWarpBytes;
  int* slots = reinterpret_cast<int*>(wbase);
  T* sK = reinterpret_cast<T*>(wbase + kGdWarpHdr);  // [32][LDK]
  T* sV = sK + kGdTK * LDK;                          // [32][LDV]
  const int32_t* page = req_to_token + req_pool_indices[r] * r2t_stride;
  for (int idx = tid; idx < 16 * (DK / 8); idx += NW * 32) {
    const int row = idx / (DK / 8), c = idx % (DK / 8);
    const bool ok = row < R;
    cp_async16(smem_u32(sQ + row * LDK + c * 8), q + (int64_t)r * q_stride + ((int64_t)h0 + (ok ? row : 0)) * DK + c * 8, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  const int rr[2] = {lane >> 2, (lane >> 2) + 8};  // this thread's two rows (query heads of the group)
  float temp = 1.f;
  if (qtemp_every > 0) temp = 1.f + qtemp_coef * logf((float)((pos + 1) / qtemp_every + 1));
  const float sc = sm_scale * temp * kLog2e, scc = softcap > 0.f ? sm_scale * temp / softcap : 0.f, capl = softcap * kLog2e;
  float sl[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) sl[x] = (slopes != nullptr && rr[x] < R) ? slopes[h0 + rr[x]] * kLog2e : 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};  // l: this thread's share of the row sum
  float o[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;

  constexpr int kc = DK / 8, vc = DV / 8;  // 16-byte chunks per row; vc divides 32, kc is at most 32
  const int64_t j_lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  const int n_split = gridDim.z;  // CTAs of the cluster that share this (request, head)
  for (int64_t j0 = j_lo + kGdTK * ((int64_t)blockIdx.z * NW + warp); j0 <= pos; j0 += (int64_t)kGdTK * NW * n_split) {
    const int n = (int)(pos - j0 + 1 < kGdTK ? pos - j0 + 1 : kGdTK);
    __syncwarp();  // the previous tile has been read
    if (lane < n) slots[lane] = page[j0 + lane];
    __syncwarp();
    for (int row = lane / kc; row < kGdTK && lane < (32 / kc) * kc; row += 32 / kc) {  // (lanes past the last whole row idle)
      const bool ok = row < n;
      const int64_t slot = ok ? slots[row] : 0;
      cp_async16(smem_u32(sK + row * LDK + (lane % kc) * 8), k_pool + (slot * G + g) * DK + (lane % kc) * 8, ok);
    }
    for (int row = lane / vc; row < kGdTK; row += 32 / vc) {
      const bool ok = row < n;
      const int64_t slot = ok ? slots[row] : 0;
      cp_async16(smem_u32(sV + row * LDV + (lane % vc) * 8), v_pool + slot * v_slot + (int64_t)(g % Gv) * DV + (lane % vc) * 8, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();

    float s[kGdTK / 8][4];
#pragma unroll
    for (int i = 0; i < kGdTK / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk) {
      uint32_t a[4];
      gm_ldsm_x4(a, sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nb2 = 0; nb2 < kGdTK / 16; ++nb2) {
        uint32_t b[4];
        gm_ldsm_x4(b, sK + (nb2 * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + kk * 16 + ((lane >> 3) & 1) * 8);
        gm_mma<T>(s[2 * nb2], a, b[0], b[1]);
        gm_mma<T>(s[2 * nb2 + 1], a, b[2], b[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < kGdTK / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int x = e >> 1;
        const int col = nb * 8 + (lane & 3) * 2 + (e & 1);
        const float z = softcap > 0.f ? capl * gm_tanh(s[nb][e] * scc) : s[nb][e] * sc;
        const float v = col < n ? z - sl[x] * (float)(pos - (j0 + col)) : -INFINITY;
        s[nb][e] = v;
        mx[x] = fmaxf(mx[x], v);
      }
    float ms[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 1));
      mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], 2));
      const float m_new = fmaxf(m[x], mx[x]);
      ms[x] = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m[x] - ms[x]);  // m = -inf: 0 (nothing accumulated yet)
      m[x] = m_new;
      l[x] *= corr;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        o[i][2 * x] *= corr;
        o[i][2 * x + 1] *= corr;
      }
    }
#pragma unroll
    for (int nb = 0; nb < kGdTK / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(s[nb][e] - ms[e >> 1]);
        s[nb][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int kk = 0; kk < kGdTK / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nb2 = 0; nb2 < DV / 16; ++nb2) {
        uint32_t b[4];
        gm_ldsm_x4_trans(b, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + nb2 * 16 + (lane >> 4) * 8);
        gm_mma<T>(o[2 * nb2], a, b[0], b[1]);
        gm_mma<T>(o[2 * nb2 + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 1);
    l[x] += __shfl_xor_sync(0xffffffffu, l[x], 2);
  }
  __syncthreads();  // the tiles are dead: their shared memory carries the partials
  float* pm = reinterpret_cast<float*>(gd_smem + kQBytes);  // [NW][16]
  float* pl = pm + NW * 16;                                 // [NW][16]
  float* po = pl + NW * 16;                                 // [NW][16][DV]
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    if ((lane & 3) == 0) {
      pm[warp * 16 + rr[x]] = m[x];
      pl[warp * 16 + rr[x]] = l[x];
    }
#pragma unroll
    for (int nb = 0; nb < DV / 8; ++nb) {
      float* dst = po + (size_t)(warp * 16 + rr[x]) * DV + nb * 8 + (lane & 3) * 2;
      dst[0] = o[nb][2 * x];
      dst[1] = o[nb][2 * x + 1];
    }
  }
  __syncthreads();
  if (n_split > 1) {
    // this CTA's triple per row (no sink yet), then the cluster's merge by rank 0
    float* cm = po + (size_t)NW * 16 * DV;  // [16]
    float* cl = cm + 16;                    // [16]
    float* co = cl + 16;                    // [16][DV]
    for (int idx = tid; idx < R * DV; idx += NW * 32) {
      const int row = idx / DV, c = idx - row * DV;
      float mt = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) mt = fmaxf(mt, pm[w * 16 + row]);
      float lt = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float mw = pm[w * 16 + row];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - mt);
        lt += pl[w * 16 + row] * f;
        acc += po[(size_t)(w * 16 + row) * DV + c] * f;
      }
      co[row * DV + c] = acc;
      if (c == 0) {
        cm[row] = mt;
        cl[row] = lt;
      }
    }
    cluster_sync_all();  // every CTA's triple is in its shared memory
    if (blockIdx.z == 0) {
      for (int idx = tid; idx < R * DV; idx += NW * 32) {
        const int row = idx / DV, c = idx - row * DV;
        const int h = h0 + row;
        const float sink2 = sinks != nullptr ? sinks[h] * kLog2e : -INFINITY;
        float mt = sink2;
        for (int z = 0; z < n_split; ++z) mt = fmaxf(mt, ld_cluster_f32(map_to_rank(smem_u32(cm + row), z)));
        float lt = sinks != nullptr ? exp2f(sink2 - mt) : 0.f;
        float acc = 0.f;
        for (int z = 0; z < n_split; ++z) {
          const float mz = ld_cluster_f32(map_to_rank(smem_u32(cm + row), z));
          const float f = mz == -INFINITY ? 0.f : exp2f(mz - mt);  // a CTA without keys adds nothing
          lt += ld_cluster_f32(map_to_rank(smem_u32(cl + row), z)) * f;
          acc += ld_cluster_f32(map_to_rank(smem_u32(co + row * DV + c), z)) * f;
        }
        out[(int64_t)r * out_stride + (int64_t)h * DV + c] = from_f32<T>(acc / lt);
      }
    }
    cluster_sync_all();  // the other CTAs' shared memory stays alive until rank 0 has read it
    return;
  }
  for (int idx = tid; idx < R * DV; idx += NW * 32) {
    const int row = idx / DV, c = idx - row * DV;
    const int h = h0 + row;
    const float sink2 = sinks != nullptr ? sinks[h] * kLog2e : -INFINITY;
    float mt = sink2;
#pragma unroll
    for (int w = 0; w < NW; ++w) mt = fmaxf(mt, pm[w * 16 + row]);
    float lt = sinks != nullptr ? exp2f(sink2 - mt) : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = pm[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mt);  // a warp without keys adds nothing
      lt += pl[w * 16 + row] * f;
      acc += po[(size_t)(w * 16 + row) * DV + c] * f;
    }
    out[(int64_t)r * out_stride + (int64_t)h * DV + c] = from_f32<T>(acc / lt);
  }
}

template <typename T, int DK, int DV, int NW>
static int gd_launch_nw(void* out, const void* q, const void* k_pool, const void* v_pool, const int32_t* req_to_token,
                        const int64_t* req_pool_indices, const int64_t* seq_lens, int64_t batch, int H, int G,
                        int64_t q_stride, int64_t out_stride, int64_t r2t_stride, float sm_scale, int window,
                        const float* sinks, const float* slopes, float qtemp_coef, int qtemp_every, float softcap, int Gv,
                        int64_t v_slot, cudaStream_t stream) {
  constexpr size_t tiles = (size_t)NW * (kGdWarpHdr + sizeof(T) * kGdTK * (DK + 8 + DV + 8));
  constexpr size_t merge = sizeof(float) * (NW + 1) * 16 * (DV + 2);  // the warps' triples + the CTA's own
  constexpr size_t smem = sizeof(T) * 16 * (DK + 8) + (tiles > merge ? tiles : merge);
  static bool configured = false;  // per instantiation
  if (!configured) {
    SPD_CUDA(cudaFuncSetAttribute(attn_general_mma_decode_kernel<T, DK, DV, NW>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  // split the keys over a cluster while (request, head) pairs alone leave SMs idle; a window bounds the
  // tiles there are to share (one per warp at least)
  int split = 1;
  const int64_t pairs = batch * G * ((H / G + 15) / 16);
  const int sms = device_sm_count_cached();
  const int64_t max_split = window > 0 ? (window + kGdTK * NW - 1) / (kGdTK * NW) : 8;
  while (split * 2 <= 8 && split * 2 <= max_split && pairs * split * 2 <= sms) split *= 2;
  static const bool no_split = getenv("SPD_ATTN_DECODE_NO_SPLIT") != nullptr;
  if (no_split) split = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)batch, (unsigned)(G * ((H / G + 15) / 16)), (unsigned)split);
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)split;
  cfg.attrs = attr;
  cfg.numAttrs = split > 1 ? 1 : 0;
  SPD_CUDA(cudaLaunchKernelEx(&cfg, attn_general_mma_decode_kernel<T, DK, DV, NW>, (T*)out, (const T*)q,
                              (const T*)k_pool, (const T*)v_pool, req_to_token, req_pool_indices, seq_lens, H, G,
                              q_stride, out_stride, r2t_stride, sm_scale, window, sinks, slopes, qtemp_coef,
                              qtemp_every, softcap, Gv, v_slot));
  return 0;
}

// → 0 launched, 1 not applicable (the caller falls back to the CUDA-core decode kernels), else an error
int attn_general_mma_decode_try(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                                int64_t batch, int H, int G, int dk, int dv, int64_t q_stride, int64_t out_stride,
                                int64_t r2t_stride, float sm_scale, int window, const float* sinks, const float* slopes,
                                float qtemp_coef, int qtemp_every, float softcap, int Gv, int64_t v_slot, int dtype,
                                cudaStream_t stream) {
  if (dtype != SPD_BF16 && dtype != SPD_F16) return 1;
  if (v_slot % 8 != 0) return 1;
  if ((int64_t)G * ((H / G + 15) / 16) > 65535 || batch >= (1ll << 31)) return 1;
  if (q_stride % 8 != 0 || !aligned16(q) || !aligned16(k_pool) || !aligned16(v_pool)) return 1;
  // short windows do not fill eight warps: four warps then leave room for more CTAs per SM
  const bool wide = window <= 0 || window > 4 * kGdTK;
#define SPD_GD_CASE(DKV, DVV)                                                                                         \
  if (dk == DKV && dv == DVV) {                                                                                       \
    if (dtype == SPD_BF16)                                                                                            \
      return wide ? gd_launch_nw<__nv_bfloat16, DKV, DVV, 8>(out, q, k_pool, v_pool, req_to_token, req_pool_indices,  \
                                                             seq_lens, batch, H, G, q_stride, out_stride, r2t_stride, \
                                                             sm_scale, window, sinks, slopes, qtemp_coef, qtemp_every, \
                                                             softcap, Gv, v_slot, stream)                                                  \
                  : gd_launch_nw<__nv_bfloat16, DKV, DVV, 4>(out, q, k_pool, v_pool, req_to_token, req_pool_indices,  \
                                                             seq_lens, batch, H, G, q_stride, out_stride, r2t_stride, \
                                                             sm_scale, window, sinks, slopes, qtemp_coef, qtemp_every, \
                                                             softcap, Gv, v_slot, stream);                                                 \
    return wide ? gd_launch_nw<__half, DKV, DVV, 8>(out, q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens, \
                                                    batch, H, G, q_stride, out_stride, r2t_stride, sm_scale, window,  \
                                                    sinks, slopes, qtemp_coef, qtemp_every, softcap, Gv, v_slot, stream)                   \
                : gd_launch_nw<__half, DKV, DVV, 4>(out, q, k_pool, v_pool, req_to_token, req_pool_indices, seq_lens, \
                                                    batch, H, G, q_stride, out_stride, r2t_stride, sm_scale, window,  \
                                                    sinks, slopes, qtemp_coef, qtemp_every, softcap, Gv, v_slot, stream);                  \
  }
  SPD_GD_CASE(32, 32)
  SPD_GD_CASE(64, 64)
  SPD_GD_CASE(64, 128)
  SPD_GD_CASE(128, 64)
  SPD_GD_CASE(128, 128)
  SPD_GD_CASE(192, 128)
#undef SPD_GD_CASE
  return 1;
}

}  // namespace spd
