// Operators of the hybrid model family (windowed attention + retention mixers, dense / MoE
// feed-forward, fp32 residual stream) that exist in 32-bit as well as in 16-bit: residual-add +
// RMS norm over an fp32 stream, embedding into it, gated activations, the per-head norm + gate of
// a retention mixer, a CUDA-core GEMM (any shape, any dtype, expert-grouped rows), and sigmoid /
// softmax routing with experts that weight their input.  The reference has no such model; these
// sit beside elementwise.cu / moe.cu and follow their conventions (C ABI, no allocation, no sync).
#include "common.cuh"
#include "ptx.cuh"

namespace spd {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kRowThreads / 32; ++i) t += red[i];  // same order in every thread
  __syncthreads();
  return t;
}

__device__ __forceinline__ float silu_precise(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float gelu_tanh_precise(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_precise(float z) { return 1.0f / (1.0f + expf(-z)); }
// act(g) * u of a gated feed-forward.  act 0 SiLU, 1 tanh-form GELU, 2 clamped sigmoid-linear unit:
// g' = min(g, p0), u' = clamp(u, -p0, p0), g' sigmoid(p1 g') (u' + 1)
__device__ __forceinline__ float gated_act(float g, float u, int act, float p0, float p1) {
  if (act == 0) return silu_precise(g) * u;
  if (act == 1) return gelu_tanh_precise(g) * u;
  g = fminf(g, p0);
  u = fminf(fmaxf(u, -p0), p0);
  return g * sigmoid_precise(p1 * g) * (u + 1.0f);
}

// one CTA per row: x += a (+ b); out = x * rsqrt(mean(x^2) + eps) * (off + w); a second weight w2
// gives a second normed copy out2 of the same row (layers whose two sublayers have a norm each)
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
residual_rmsnorm_kernel(T* __restrict__ out, float* __restrict__ x, const T* __restrict__ a,
                        const T* __restrict__ b, const T* __restrict__ w, int64_t dim, float eps, float off,
                        T* __restrict__ out2, const T* __restrict__ w2) {
  griddep_wait();
  griddep_launch_dependents();
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  float* xr = x + row * dim;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < dim; i += kRowThreads) {
    float v = xr[i];
    if (a != nullptr) {
      float d = to_f32<T>(a[row * dim + i]);
      if (b != nullptr) d += to_f32<T>(b[row * dim + i]);
      v += d;
      xr[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum_256(ss, red);
  if (out == nullptr) return;
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  for (int64_t i = threadIdx.x; i < dim; i += kRowThreads) {
    const float y = xr[i] * inv;
    out[row * dim + i] = from_f32<T>(y * (off + to_f32<T>(w[i])));
    if (out2 != nullptr) out2[row * dim + i] = from_f32<T>(y * (off + to_f32<T>(w2[i])));
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
embed_f32_kernel(float* __restrict__ x, const T* __restrict__ table, const int64_t* __restrict__ idx,
                 int64_t dim, int64_t table_rows) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t row = blockIdx.x;
  int64_t id = idx[row];
  id = id < 0 ? 0 : (id >= table_rows ? table_rows - 1 : id);
  for (int64_t i = threadIdx.x; i < dim; i += kRowThreads) x[row * dim + i] = to_f32<T>(table[id * dim + i]);
}

// vector form: inter a multiple of the vector width, 16-byte aligned pointers
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
act_and_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int64_t inter, int act, float p0,
                       float p1) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int N = Vec16<T>::kN;
  const int64_t per_row = inter / N, n = rows * per_row;
  for (int64_t i = blockIdx.x * (int64_t)kRowThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kRowThreads) {
    const int64_t r = i / per_row, c = (i - r * per_row) * N;
    const Vec16<T> g = ldv(x + r * 2 * inter + c), u = ldv(x + r * 2 * inter + inter + c);
    Vec16<T> o;
#pragma unroll
    for (int k = 0; k < N; ++k) {
      o.e()[k] = from_f32<T>(gated_act(to_f32<T>(g.e()[k]), to_f32<T>(u.e()[k]), act, p0, p1));
    }
    stv(out + r * inter + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
act_and_mul_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int64_t inter, int act, float p0,
                   float p1) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t n = rows * inter;
  for (int64_t i = blockIdx.x * (int64_t)kRowThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kRowThreads) {
    const int64_t r = i / inter, c = i - r * inter;
    const float g = to_f32<T>(x[r * 2 * inter + c]);
    const float u = to_f32<T>(x[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(gated_act(g, u, act, p0, p1));
  }
}

// one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
headnorm_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const T* __restrict__ g, int64_t tokens,
                     int heads, int vdim, int64_t g_stride, float eps, const T* __restrict__ w, int w_head_stride,
                     int gate_act) {
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t item = blockIdx.x * 4ll + (threadIdx.x >> 5);
  if (item >= tokens * heads) return;
  const int64_t t = item / heads;
  const int h = (int)(item - t * heads);
  const float* orow = o + (t * heads + h) * (int64_t)vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss += orow[c] * orow[c];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    const float gz = to_f32<T>(g[t * g_stride + (int64_t)h * vdim + c]);
    const float gate = gate_act == 0 ? silu_precise(gz) : sigmoid_precise(gz);
    const float wt = w != nullptr ? to_f32<T>(w[h * w_head_stride + c]) : 1.f;
    out[(t * heads + h) * (int64_t)vdim + c] = from_f32<T>(orow[c] * inv * wt * gate);
  }
}

// ------------------------------------------------------------------------------------------------
// CUDA-core GEMM: 64 x 64 output tile, k-steps of 16, 4 x 4 outputs per thread, fp32 accumulation
// in ascending k — the sum of an output element does not depend on M, on the tile it falls in or
// on what else is in the batch.
// ------------------------------------------------------------------------------------------------
constexpr int kSBM = 64, kSBN = 64, kSBK = 16, kSPad = 68;

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
linear_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TA* __restrict__ W, int64_t M, int64_t N,
                   int64_t K, int64_t lda, int64_t ldw, int64_t ldc, const int32_t* __restrict__ tile_group,
                   int64_t w_group_rows, int64_t a_group_cols, int64_t c_group_cols) {
  griddep_wait();
  griddep_launch_dependents();
  __shared__ __align__(16) float As[kSBK][kSPad];
  __shared__ __align__(16) float Ws[kSBK][kSPad];
  const int64_t m0 = (int64_t)blockIdx.y * kSBM, n0 = (int64_t)blockIdx.x * kSBN;
  // block-diagonal form: block z multiplies columns [z * a_group_cols, + K) of A by rows
  // [z * w_group_rows, + N) of W into columns [z * c_group_cols, + N) of C
  A += (int64_t)blockIdx.z * a_group_cols;
  C += (int64_t)blockIdx.z * c_group_cols;
  if (tile_group == nullptr) W += (int64_t)blockIdx.z * w_group_rows * ldw;
  if (tile_group != nullptr) {
    const int g = tile_group[m0 / 128];
    if (g < 0) return;
    W += (int64_t)g * w_group_rows * ldw;
  }
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row lr, k lk .. lk + 3
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += kSBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t k = k0 + lk + i;
      const int64_t am = m0 + lr, wn = n0 + lr;
      As[lk + i][lr] = (am < M && k < K) ? to_f32<TA>(A[am * lda + k]) : 0.f;
      Ws[lk + i][lr] = (wn < N && k < K) ? to_f32<TA>(W[wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kSBK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w};
      const float w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < N) C[m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// routing from fp32 logits: one warp per token
// ------------------------------------------------------------------------------------------------
constexpr int kRouteMaxExperts = 256;
constexpr int kRouteMaxTopK = 16;
constexpr int kRouteMaxGroups = 32;

// scores s = sigmoid(z) or softmax(z); selection runs on the biased score c = s + correction.  With groups the
// experts are cut into equal runs of neighbours, every run is ranked by its top-2 biased scores added together,
// and experts outside the keep_groups highest-ranked runs are ineligible (c = -inf there).  The weight of a
// selected expert is its unbiased s (optionally renormalised).
__global__ void __launch_bounds__(128)
moe_route_scores_kernel(int32_t* __restrict__ topk_ids, float* __restrict__ topk_w, const float* __restrict__ logits,
                        int64_t ld, int64_t tokens, int E, int k, int score_func, int renorm, float scale,
                        const float* __restrict__ correction, int num_groups, int keep_groups) {
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * 4ll + (threadIdx.x >> 5);
  if (t >= tokens) return;
  constexpr int PER = kRouteMaxExperts / 32;
  float v[PER];  // scores (0 outside the experts)
  if (score_func == 1) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < E ? sigmoid_precise(logits[t * ld + e]) : 0.f;
    }
  } else {
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < E ? logits[t * ld + e] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] = (i * 32 + lane) < E ? expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = v[i] / sum;
  }
  float c[PER];  // choice scores; -inf: not an expert, outside the kept groups, or taken
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    c[i] = e < E ? v[i] + (correction != nullptr ? correction[e] : 0.f) : -INFINITY;
  }
  if (num_groups > 1 && keep_groups < num_groups) {
    const int per = E / num_groups;
    float gscore = -INFINITY;  // lane g keeps the score of group g
    for (int g = 0; g < num_groups; ++g) {
      float a1 = -INFINITY, a2 = -INFINITY;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        if (e < E && e / per == g) {
          if (c[i] > a1) { a2 = a1; a1 = c[i]; }
          else if (c[i] > a2) a2 = c[i];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float b1 = __shfl_xor_sync(0xffffffffu, a1, o), b2 = __shfl_xor_sync(0xffffffffu, a2, o);
        const float hi = fmaxf(a1, b1), lo = fmaxf(fminf(a1, b1), fmaxf(a2, b2));
        a1 = hi;
        a2 = lo;
      }
      if (lane == g) gscore = a1 + (per >= 2 ? a2 : 0.f);
    }
    unsigned kept = 0u;
    for (int j = 0; j < keep_groups; ++j) {
      float best = gscore;
      int bg = lane < num_groups ? lane : 0x7fffffff;
      if (lane >= num_groups) best = -INFINITY;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, bg, o);
        if (ob > best || (ob == best && og < bg)) { best = ob; bg = og; }
      }
      if (bg < num_groups) {
        kept |= 1u << bg;
        if (lane == bg) gscore = -INFINITY;
      } else {
        // every remaining group scores -inf (or NaN): keep the lowest one not yet kept
        for (int g = 0; g < num_groups; ++g)
          if (!((kept >> g) & 1u)) { kept |= 1u << g; if (lane == g) gscore = -INFINITY; break; }
      }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (e < E && !((kept >> (e / per)) & 1u)) c[i] = -INFINITY;
    }
  }
  float pw[kRouteMaxTopK];
  int pe[kRouteMaxTopK];
  float wsum = 0.f;
#pragma unroll
  for (int j = 0; j < kRouteMaxTopK; ++j) {
    if (j < k) {
      float best = -INFINITY;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        if (c[i] > best) { best = c[i]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
      }
      float w = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i * 32 + lane == be) { w = v[i]; c[i] = -INFINITY; }
      w = warp_sum(w);
      pe[j] = be < E ? be : 0;
      pw[j] = w;
      wsum += w;
    }
  }
  if (lane == 0) {
    const float f = renorm ? scale / (wsum + 1e-20f) : scale;
#pragma unroll
    for (int j = 0; j < kRouteMaxTopK; ++j)
      if (j < k) {
        topk_ids[t * k + j] = pe[j];
        topk_w[t * k + j] = pw[j] * f;
      }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
moe_gather_scaled_kernel(T* __restrict__ xs, const T* __restrict__ x, const int32_t* __restrict__ row_token,
                         const int32_t* __restrict__ inv_pos, const float* __restrict__ topk_w, int top_k,
                         int64_t dim, int64_t x_stride) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t r = blockIdx.x;
  const int t = row_token[r];
  float w = 1.f;
  if (t >= 0 && topk_w != nullptr) {
    for (int j = 0; j < top_k; ++j)
      if (inv_pos[(int64_t)t * top_k + j] == (int32_t)r) w = topk_w[(int64_t)t * top_k + j];
  }
  constexpr int N = Vec16<T>::kN;
  if (dim % N == 0 && x_stride % N == 0 && ((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(x)) & 15u) == 0) {
    for (int64_t i = threadIdx.x * N; i < dim; i += kRowThreads * N) {
      Vec16<T> o;
      if (t < 0) {
        o.raw = make_uint4(0u, 0u, 0u, 0u);
      } else {
        const Vec16<T> v = ldv(x + (int64_t)t * x_stride + i);
#pragma unroll
        for (int k = 0; k < N; ++k) o.e()[k] = from_f32<T>(w * to_f32<T>(v.e()[k]));
      }
      stv(xs + r * dim + i, o);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < dim; i += kRowThreads)
    xs[r * dim + i] = t < 0 ? from_f32<T>(0.f) : from_f32<T>(w * to_f32<T>(x[(int64_t)t * x_stride + i]));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
moe_combine_gated_kernel(T* __restrict__ out, const T* __restrict__ y, const int32_t* __restrict__ inv_pos,
                         const float* __restrict__ topk_w, const T* __restrict__ shared,
                         const float* __restrict__ shared_gate, int64_t gate_stride, int top_k, int64_t dim) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  const float sg = shared_gate != nullptr ? sigmoid_precise(shared_gate[t * gate_stride]) : 1.f;
  constexpr int N = Vec16<T>::kN;
  if (dim % N == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(y) |
                        reinterpret_cast<uintptr_t>(shared)) & 15u) == 0) {
    for (int64_t i = threadIdx.x * N; i < dim; i += kRowThreads * N) {
      float acc[N];
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const float w = topk_w != nullptr ? topk_w[t * top_k + j] : 1.f;
        const Vec16<T> v = ldv(y + (int64_t)inv_pos[t * top_k + j] * dim + i);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += w * to_f32<T>(v.e()[k]);
      }
      if (shared != nullptr) {
        const Vec16<T> v = ldv(shared + t * dim + i);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] += sg * to_f32<T>(v.e()[k]);
      }
      Vec16<T> o;
#pragma unroll
      for (int k = 0; k < N; ++k) o.e()[k] = from_f32<T>(acc[k]);
      stv(out + t * dim + i, o);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < dim; i += kRowThreads) {
    float acc = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const float w = topk_w != nullptr ? topk_w[t * top_k + j] : 1.f;
      acc += w * to_f32<T>(y[(int64_t)inv_pos[t * top_k + j] * dim + i]);
    }
    if (shared != nullptr) acc += sg * to_f32<T>(shared[t * dim + i]);
    out[t * dim + i] = from_f32<T>(acc);
  }
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_residual_rmsnorm(void* out, float* x, const void* a, const void* b, const void* w, int64_t rows,
                         int64_t dim, float eps, float weight_offset, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(x && (out == nullptr || w), SPD_E_BADARG, "spd_residual_rmsnorm: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0, SPD_E_BADARG, "spd_residual_rmsnorm: bad sizes");
  SPD_REQUIRE(a != nullptr || b == nullptr, SPD_E_BADARG, "spd_residual_rmsnorm: b without a");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(residual_rmsnorm_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, x, (const T*)a, (const T*)b, (const T*)w, dim, eps, weight_offset,
                    (T*)nullptr, (const T*)nullptr));
  });
  return 0;
}

int spd_residual_rmsnorm2(void* out, void* out2, float* x, const void* a, const void* b, const void* w,
                          const void* w2, int64_t rows, int64_t dim, float eps, float weight_offset, int dtype,
                          spd_stream_t stream) {
  SPD_REQUIRE(x && out && w && (out2 == nullptr) == (w2 == nullptr), SPD_E_BADARG, "spd_residual_rmsnorm2: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0, SPD_E_BADARG, "spd_residual_rmsnorm2: bad sizes");
  SPD_REQUIRE(a != nullptr || b == nullptr, SPD_E_BADARG, "spd_residual_rmsnorm2: b without a");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(residual_rmsnorm_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, x, (const T*)a, (const T*)b, (const T*)w, dim, eps, weight_offset,
                    (T*)out2, (const T*)w2));
  });
  return 0;
}

int spd_embed_f32(float* x, const void* table, const int64_t* idx, int64_t rows, int64_t dim,
                  int64_t table_rows, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(x && table && idx, SPD_E_BADARG, "spd_embed_f32: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0 && table_rows > 0, SPD_E_BADARG, "spd_embed_f32: bad sizes");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(embed_f32_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, as_stream(stream),
                    pdl_enabled(), x, (const T*)table, idx, dim, table_rows));
  });
  return 0;
}

int spd_act_and_mul(void* out, const void* x, int64_t rows, int64_t inter, int act, float p0, float p1, int dtype,
                    spd_stream_t stream) {
  SPD_REQUIRE(out && x, SPD_E_BADARG, "spd_act_and_mul: null pointer");
  SPD_REQUIRE(rows >= 0 && inter > 0 && act >= 0 && act <= 2, SPD_E_BADARG, "spd_act_and_mul: bad arguments");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    constexpr int N = 16 / (int)sizeof(T);
    const bool vec = inter % N == 0 && aligned16(out) && aligned16(x);
    const int64_t n = vec ? rows * inter / N : rows * inter;
    const int64_t blocks = (n + kRowThreads - 1) / kRowThreads;
    const unsigned grid = (unsigned)(blocks < 8192 ? blocks : 8192);
    if (vec) {
      SPD_CUDA(launch(act_and_mul_vec_kernel<T>, dim3(grid), dim3(kRowThreads), 0, as_stream(stream), pdl_enabled(),
                      (T*)out, (const T*)x, rows, inter, act, p0, p1));
    } else {
      SPD_CUDA(launch(act_and_mul_kernel<T>, dim3(grid), dim3(kRowThreads), 0, as_stream(stream), pdl_enabled(),
                      (T*)out, (const T*)x, rows, inter, act, p0, p1));
    }
  });
  return 0;
}

int spd_headnorm_gate(void* out, const float* o, const void* g, int64_t tokens, int heads, int vdim,
                      int64_t g_stride, float eps, const void* w, int w_head_stride, int gate_act, int dtype,
                      spd_stream_t stream) {
  SPD_REQUIRE(out && o && g, SPD_E_BADARG, "spd_headnorm_gate: null pointer");
  SPD_REQUIRE(gate_act == 0 || gate_act == 1, SPD_E_BADARG, "spd_headnorm_gate: gate_act is 0 (SiLU) or 1 (sigmoid)");
  SPD_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0, SPD_E_BADARG, "spd_headnorm_gate: bad sizes");
  if (tokens == 0) return 0;
  const int64_t items = tokens * heads;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(headnorm_gate_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, o, (const T*)g, tokens, heads, vdim, g_stride, eps, (const T*)w,
                    w_head_stride, gate_act));
  });
  return 0;
}

int spd_linear_simt(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldw, int64_t ldc, const int32_t* tile_group, int64_t w_group_rows, int dtype,
                    int out_f32, spd_stream_t stream) {
  SPD_REQUIRE(C && A && W, SPD_E_BADARG, "spd_linear_simt: null pointer");
  SPD_REQUIRE(M >= 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, SPD_E_BADARG,
              "spd_linear_simt: bad sizes M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  SPD_REQUIRE(tile_group == nullptr || M % 128 == 0, SPD_E_SHAPE, "spd_linear_simt: grouped rows come in 128-row tiles");
  if (M == 0) return 0;
  const dim3 grid((unsigned)((N + kSBN - 1) / kSBN), (unsigned)((M + kSBM - 1) / kSBM));
  SPD_DISPATCH_ANY(dtype, {
    if (out_f32) {
      SPD_CUDA(launch(linear_simt_kernel<T, float>, grid, dim3(256), 0, as_stream(stream), pdl_enabled(), (float*)C,
                      (const T*)A, (const T*)W, M, N, K, lda, ldw, ldc, tile_group, w_group_rows, (int64_t)0,
                      (int64_t)0));
    } else {
      SPD_CUDA(launch(linear_simt_kernel<T, T>, grid, dim3(256), 0, as_stream(stream), pdl_enabled(), (T*)C,
                      (const T*)A, (const T*)W, M, N, K, lda, ldw, ldc, tile_group, w_group_rows, (int64_t)0,
                      (int64_t)0));
    }
  });
  return 0;
}

int spd_linear_simt_block_diag(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldw, int64_t ldc, int num_groups, int64_t a_group_cols,
                               int64_t c_group_cols, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(C && A && W, SPD_E_BADARG, "spd_linear_simt_block_diag: null pointer");
  SPD_REQUIRE(M >= 0 && N > 0 && K > 0 && num_groups > 0 && num_groups <= 65535 && ldw >= K &&
                  lda >= (num_groups - 1) * a_group_cols + K && ldc >= (num_groups - 1) * c_group_cols + N,
              SPD_E_BADARG, "spd_linear_simt_block_diag: bad sizes M=%lld N=%lld K=%lld groups=%d", (long long)M,
              (long long)N, (long long)K, num_groups);
  if (M == 0) return 0;
  const dim3 grid((unsigned)((N + kSBN - 1) / kSBN), (unsigned)((M + kSBM - 1) / kSBM), (unsigned)num_groups);
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(linear_simt_kernel<T, T>, grid, dim3(256), 0, as_stream(stream), pdl_enabled(), (T*)C, (const T*)A,
                    (const T*)W, M, N, K, lda, ldw, ldc, (const int32_t*)nullptr, N, a_group_cols, c_group_cols));
  });
  return 0;
}

int spd_moe_route_scores(int32_t* topk_ids, float* topk_w, const float* logits, int64_t ld, int64_t tokens,
                         int num_experts, int top_k, int score_func, int renormalize, float scale,
                         const float* correction, int num_groups, int keep_groups, spd_stream_t stream) {
  SPD_REQUIRE(topk_ids && topk_w && logits, SPD_E_BADARG, "spd_moe_route_scores: null pointer");
  SPD_REQUIRE(num_experts > 0 && num_experts <= kRouteMaxExperts && top_k > 0 && top_k <= kRouteMaxTopK &&
                  top_k <= num_experts && ld >= num_experts && (score_func == 0 || score_func == 1),
              SPD_E_SHAPE, "spd_moe_route_scores: experts %d (max %d), top_k %d (max %d)", num_experts,
              kRouteMaxExperts, top_k, kRouteMaxTopK);
  SPD_REQUIRE(num_groups <= 1 || (num_groups <= kRouteMaxGroups && num_experts % num_groups == 0 && keep_groups >= 1 &&
                                  keep_groups <= num_groups && (int64_t)keep_groups * (num_experts / num_groups) >= top_k),
              SPD_E_SHAPE, "spd_moe_route_scores: %d groups (max %d, dividing the experts), keep %d", num_groups,
              kRouteMaxGroups, keep_groups);
  if (tokens == 0) return 0;
  SPD_CUDA(launch(moe_route_scores_kernel, dim3((unsigned)((tokens + 3) / 4)), dim3(128), 0, as_stream(stream),
                  pdl_enabled(), topk_ids, topk_w, logits, ld, tokens, num_experts, top_k, score_func, renormalize,
                  scale, correction, num_groups, keep_groups));
  return 0;
}

int spd_moe_gather_scaled(void* xs, const void* x, const int32_t* row_token, const int32_t* inv_pos,
                          const float* topk_w, int64_t rows, int top_k, int64_t dim, int64_t x_stride,
                          int dtype, spd_stream_t stream) {
  SPD_REQUIRE(xs && x && row_token && inv_pos, SPD_E_BADARG, "spd_moe_gather_scaled: null pointer");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(moe_gather_scaled_kernel<T>, dim3((unsigned)rows), dim3(kRowThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)xs, (const T*)x, row_token, inv_pos, topk_w, top_k, dim, x_stride));
  });
  return 0;
}

int spd_moe_combine_gated(void* out, const void* y, const int32_t* inv_pos, const float* topk_w,
                          const void* shared, const float* shared_gate, int64_t gate_stride, int64_t tokens,
                          int top_k, int64_t dim, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(out && y && inv_pos, SPD_E_BADARG, "spd_moe_combine_gated: null pointer");
  if (tokens == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(moe_combine_gated_kernel<T>, dim3((unsigned)tokens), dim3(kRowThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, (const T*)y, inv_pos, topk_w, (const T*)shared, shared_gate, gate_stride,
                    top_k, dim));
  });
  return 0;
}

}  // extern "C"
