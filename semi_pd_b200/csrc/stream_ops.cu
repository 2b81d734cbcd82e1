// A residual that is kept as several parallel streams (hyper-connections), and the rotary step of an
// attention whose projections carry biases.  The residual of a token is X[s, :] for s < S streams, fp32;
// a sublayer reads  u = sum_s in[s] X[s]  through an RMS norm and writes its result y back as
//     X'[t] = sum_s mix[s, t] X[s] + mult * out[t] * y          (every new stream from the old ones).
// One kernel closes sublayer i and opens sublayer i + 1: it applies the write of i (y may be the weighted
// sum of two branch outputs plus a bias, all combined in fp32), forms the read of i + 1 and norms it, in one
// pass over the token's streams — the role residual_rmsnorm has for a single stream; S = 1 with unit
// coefficients is the plain residual x += mult * y.  Beside hybrid_ops.cu in role; the reference has none.
#include "common.cuh"
#include "ptx.cuh"

namespace spd {

constexpr int kStrThreads = 256;
constexpr int kMaxStreams = 8;

__device__ __forceinline__ float block_sum_str(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < kStrThreads / 32; ++i) t += red[i];  // same order in every thread
  __syncthreads();
  return t;
}

// X[r, s, :] = table[idx[r], :] / sqrt(mean(.^2) + eps) * w for every stream s (w == nullptr: the raw row)
template <typename T>
__global__ void __launch_bounds__(kStrThreads)
embed_norm_streams_kernel(float* __restrict__ X, const T* __restrict__ table, const int64_t* __restrict__ idx,
                          const T* __restrict__ w, int64_t dim, int64_t table_rows, int S, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  __shared__ float red[kStrThreads / 32];
  const int64_t row = blockIdx.x;
  int64_t id = idx[row];
  id = id < 0 ? 0 : (id >= table_rows ? table_rows - 1 : id);
  const T* tr = table + id * dim;
  float inv = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < dim; i += kStrThreads) {
      const float v = to_f32<T>(tr[i]);
      ss += v * v;
    }
    ss = block_sum_str(ss, red);
    inv = 1.0f / sqrtf(ss / (float)dim + eps);
  }
  for (int64_t i = threadIdx.x; i < dim; i += kStrThreads) {
    float v = to_f32<T>(tr[i]);
    if (w != nullptr) v = v * inv * to_f32<T>(w[i]);
    for (int s = 0; s < S; ++s) X[(row * S + s) * dim + i] = v;
  }
}

// One CTA per token.  Write part (a != nullptr): y = sa a + sb b + sbias bias, X' = mix^T X + mult out y.
// Read part (out != nullptr): u = sum_s in[s] X'[s] (in == nullptr: every coefficient 1), out = norm(u) w.
// rows != nullptr (read part only): CTA r reads token rows[r] and writes out row r.
template <typename T, bool STASH>
__global__ void __launch_bounds__(kStrThreads)
streams_mix_norm_kernel(T* __restrict__ out, float* __restrict__ X, const T* __restrict__ a, const T* __restrict__ b,
                        const float* __restrict__ bias, float sa, float sb, float sbias,
                        const float* __restrict__ mix, const float* __restrict__ outw, float mult,
                        const float* __restrict__ inw, const T* __restrict__ w, const int64_t* __restrict__ rows,
                        int64_t dim, int S, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  extern __shared__ float ubuf[];  // STASH: the read u of this token, [dim]
  __shared__ float red[kStrThreads / 32];
  __shared__ float cmix[kMaxStreams * kMaxStreams], cout[kMaxStreams], cin[kMaxStreams];
  if (threadIdx.x < S * S) cmix[threadIdx.x] = mix != nullptr ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    cout[threadIdx.x] = outw != nullptr ? mult * outw[threadIdx.x] : 0.f;
    cin[threadIdx.x] = inw != nullptr ? inw[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const int64_t src = rows != nullptr ? rows[blockIdx.x] : (int64_t)blockIdx.x;
  const int64_t dst = blockIdx.x;
  float* xr = X + src * S * dim;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < dim; i += kStrThreads) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) xs[s] = s < S ? xr[s * dim + i] : 0.f;
    if (a != nullptr) {
      float y = sa * to_f32<T>(a[src * dim + i]);
      if (b != nullptr) y = fmaf(sb, to_f32<T>(b[src * dim + i]), y);
      if (bias != nullptr) y = fmaf(sbias, bias[i], y);
      float nx[kMaxStreams];
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        float v = 0.f;
        if (t < S) {
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) v = fmaf(cmix[s * S + t], xs[s], v);
          v = fmaf(cout[t], y, v);
          xr[t * dim + i] = v;
        }
        nx[t] = v;
      }
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) xs[s] = nx[s];
    }
    if (out != nullptr) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) u = fmaf(cin[s], xs[s], u);
      if (STASH) ubuf[i] = u;
      ss += u * u;
    }
  }
  if (out == nullptr) return;
  ss = block_sum_str(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  for (int64_t i = threadIdx.x; i < dim; i += kStrThreads) {
    float u;
    if (STASH) {
      u = ubuf[i];  // written by this thread
    } else {
      u = 0.f;
      for (int s = 0; s < S; ++s) u = fmaf(cin[s], xr[s * dim + i], u);
    }
    out[dst * dim + i] = from_f32<T>(u * inv * to_f32<T>(w[i]));
  }
}

// four consecutive elements of a row as floats
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  v[0] = lo.x, v[1] = lo.y, v[2] = hi.x, v[3] = hi.y;
}
__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  v[0] = lo.x, v[1] = lo.y, v[2] = hi.x, v[3] = hi.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ void store4(__half* p, const float (&v)[4]) {
  uint2 raw;
  *reinterpret_cast<__half2*>(&raw.x) = __floats2half2_rn(v[0], v[1]);
  *reinterpret_cast<__half2*>(&raw.y) = __floats2half2_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same operation for a stream count known at compile time and rows of a multiple of four elements on 16-byte
// boundaries: coefficients in registers, four elements per thread and step, u stashed in shared memory.  Which
// of the two forms runs depends on the model's sizes alone, never on the batch.
template <typename T, int S>
__global__ void __launch_bounds__(kStrThreads)
streams_mix_norm_vec_kernel(T* __restrict__ out, float* __restrict__ X, const T* __restrict__ a, const T* __restrict__ b,
                            const float* __restrict__ bias, float sa, float sb, float sbias,
                            const float* __restrict__ mix, const float* __restrict__ outw, float mult,
                            const float* __restrict__ inw, const T* __restrict__ w, const int64_t* __restrict__ rows,
                            int64_t dim, float eps) {
  griddep_wait();
  griddep_launch_dependents();
  extern __shared__ __align__(16) float ubuf[];  // the read u of this token, [dim]
  __shared__ float red[kStrThreads / 32];
  float cmix[S][S], cout[S], cin[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
#pragma unroll
    for (int t = 0; t < S; ++t) cmix[s][t] = mix != nullptr ? mix[s * S + t] : 0.f;
    cout[s] = outw != nullptr ? mult * outw[s] : 0.f;
    cin[s] = inw != nullptr ? inw[s] : 1.f;
  }
  const int64_t src = rows != nullptr ? rows[blockIdx.x] : (int64_t)blockIdx.x;
  const int64_t dst = blockIdx.x;
  float* xr = X + src * S * dim;
  float ss = 0.f;
  for (int64_t i = threadIdx.x * 4; i < dim; i += kStrThreads * 4) {
    float xs[S][4];
#pragma unroll
    for (int s = 0; s < S; ++s) load4(xr + s * dim + i, xs[s]);
    if (a != nullptr) {
      float y[4], t4[4];
      load4(a + src * dim + i, y);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] *= sa;
      if (b != nullptr) {
        load4(b + src * dim + i, t4);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = fmaf(sb, t4[e], y[e]);
      }
      if (bias != nullptr) {
        load4(bias + i, t4);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = fmaf(sbias, t4[e], y[e]);
      }
      float nx[S][4];
#pragma unroll
      for (int t = 0; t < S; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) v = fmaf(cmix[s][t], xs[s][e], v);
          nx[t][e] = fmaf(cout[t], y[e], v);
        }
        store4(xr + t * dim + i, nx[t]);
      }
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int e = 0; e < 4; ++e) xs[s][e] = nx[s][e];
    }
    if (out != nullptr) {
      float u[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) v = fmaf(cin[s], xs[s][e], v);
        u[e] = v;
        ss += v * v;
      }
      store4(ubuf + i, u);
    }
  }
  if (out == nullptr) return;
  ss = block_sum_str(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  for (int64_t i = threadIdx.x * 4; i < dim; i += kStrThreads * 4) {
    float u[4], wv[4];
    load4(ubuf + i, u);  // written by this thread
    load4(w + i, wv);
#pragma unroll
    for (int e = 0; e < 4; ++e) u[e] = u[e] * inv * wv[e];
    store4(out + dst * dim + i, u);
  }
}

// One CTA per token: q' = rot(q + q_bias), k' = rot(k + k_bias) over the first `rot` dimensions of every head
// (rotate-half pairing; cos_sin [positions, rot] fp32 = cos || sin, any magnitude factor folded in);
// q' -> q_out, k' -> k_pool[loc], and the values -> v_pool[loc]: v (when given) or the biased keys BEFORE
// the rotation (v == nullptr; value size = key size then).
template <typename T>
__global__ void __launch_bounds__(128)
rotary_bias_store_kernel(T* __restrict__ q_out, const T* __restrict__ q, const T* __restrict__ k,
                         const T* __restrict__ v, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                         T* __restrict__ k_pool, T* __restrict__ v_pool, const int64_t* __restrict__ loc,
                         const int64_t* __restrict__ positions, const float* __restrict__ cos_sin, int rot,
                         int64_t max_positions, int Hq, int Hk, int dk, int dv, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t q_out_stride) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  const int half = rot >> 1;
  int64_t p = positions[t];
  p = p < 0 ? 0 : (p < max_positions ? p : max_positions - 1);
  const float* cs = cos_sin + p * rot;
  const int64_t slot = loc[t];
  const int nq = Hq * dk, nk = Hk * dk;
  for (int idx = threadIdx.x; idx < nq + nk; idx += 128) {
    const bool is_q = idx < nq;
    const int e = is_q ? idx : idx - nq;
    const int d = e % dk;
    const T* src = is_q ? q + t * q_stride : k + t * k_stride;
    const float* bs = is_q ? q_bias : k_bias;
    const float x = to_f32<T>(src[e]) + (bs != nullptr ? bs[e] : 0.f);
    float y = x;
    if (d < rot) {
      const int i = d < half ? d : d - half;
      const int pe = d < half ? e + half : e - half;
      const float xp = to_f32<T>(src[pe]) + (bs != nullptr ? bs[pe] : 0.f);
      const float c = cs[i], sn = cs[half + i];
      y = d < half ? x * c - xp * sn : x * c + xp * sn;
    }
    if (is_q) {
      q_out[t * q_out_stride + e] = from_f32<T>(y);
    } else {
      k_pool[slot * nk + e] = from_f32<T>(y);
      if (v == nullptr && v_pool != nullptr) v_pool[slot * nk + e] = from_f32<T>(x);
    }
  }
  if (v != nullptr && v_pool != nullptr) {
    const int nv = Hk * dv;
    for (int e = threadIdx.x; e < nv; e += 128) v_pool[slot * nv + e] = v[t * v_stride + e];
  }
}

// The same step in 16-byte pieces (rot / 2, head_dim and the row strides multiples of the vector width, 16-byte
// aligned rows): a work item is one vector of a head's first rotation half together with its partner vector of the
// second half, or one vector of the channels that pass unrotated.  Same arithmetic, element by element.
template <typename T>
__global__ void __launch_bounds__(128)
rotary_bias_store_vec_kernel(T* __restrict__ q_out, const T* __restrict__ q, const T* __restrict__ k,
                             const T* __restrict__ v, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                             T* __restrict__ k_pool, T* __restrict__ v_pool, const int64_t* __restrict__ loc,
                             const int64_t* __restrict__ positions, const float* __restrict__ cos_sin, int rot,
                             int64_t max_positions, int Hq, int Hk, int dk, int dv, int64_t q_stride, int64_t k_stride,
                             int64_t v_stride, int64_t q_out_stride) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int N = Vec16<T>::kN;
  const int64_t t = blockIdx.x;
  const int half = rot >> 1;
  int64_t p = positions[t];
  p = p < 0 ? 0 : (p < max_positions ? p : max_positions - 1);
  const float* cs = cos_sin + p * rot;
  const int64_t slot = loc[t];
  const int nk = Hk * dk;
  const int rot_items = half / N, pass_items = (dk - rot) / N, per_head = rot_items + pass_items;
  for (int item = threadIdx.x; item < (Hq + Hk) * per_head; item += 128) {
    const int head = item / per_head, j = item - head * per_head;
    const bool is_q = head < Hq;
    const int hb = (is_q ? head : head - Hq) * dk;  // the head's first element in its row
    const T* src = is_q ? q + t * q_stride : k + t * k_stride;
    const float* bs = is_q ? q_bias : k_bias;
    T* dst = is_q ? q_out + t * q_out_stride : k_pool + slot * nk;
    if (j < rot_items) {
      const int d = j * N;
      const Vec16<T> xa = ldv(src + hb + d), xb = ldv(src + hb + half + d);
      Vec16<T> ya, yb, va, vb;
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const float a = to_f32<T>(xa.e()[e]) + (bs != nullptr ? bs[hb + d + e] : 0.f);
        const float b = to_f32<T>(xb.e()[e]) + (bs != nullptr ? bs[hb + half + d + e] : 0.f);
        const float c = cs[d + e], sn = cs[half + d + e];
        ya.e()[e] = from_f32<T>(a * c - b * sn);
        yb.e()[e] = from_f32<T>(b * c + a * sn);
        va.e()[e] = from_f32<T>(a);
        vb.e()[e] = from_f32<T>(b);
      }
      stv(dst + hb + d, ya);
      stv(dst + hb + half + d, yb);
      if (!is_q && v == nullptr && v_pool != nullptr) {
        stv(v_pool + slot * nk + hb + d, va);
        stv(v_pool + slot * nk + hb + half + d, vb);
      }
    } else {
      const int d = rot + (j - rot_items) * N;
      const Vec16<T> x = ldv(src + hb + d);
      Vec16<T> y;
#pragma unroll
      for (int e = 0; e < N; ++e) y.e()[e] = from_f32<T>(to_f32<T>(x.e()[e]) + (bs != nullptr ? bs[hb + d + e] : 0.f));
      stv(dst + hb + d, y);
      if (!is_q && v == nullptr && v_pool != nullptr) stv(v_pool + slot * nk + hb + d, y);
    }
  }
  if (v != nullptr && v_pool != nullptr) {
    const int nv = Hk * dv;
    for (int e = threadIdx.x; e < nv; e += 128) v_pool[slot * nv + e] = v[t * v_stride + e];
  }
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_embed_norm_streams(float* X, const void* table, const int64_t* idx, const void* w, int64_t rows,
                           int64_t dim, int64_t table_rows, int streams, float eps, int dtype,
                           spd_stream_t stream) {
  SPD_REQUIRE(X && table && idx, SPD_E_BADARG, "spd_embed_norm_streams: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0 && table_rows > 0 && streams >= 1, SPD_E_BADARG,
              "spd_embed_norm_streams: bad sizes");
  if (rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(embed_norm_streams_kernel<T>, dim3((unsigned)rows), dim3(kStrThreads), 0, as_stream(stream),
                    pdl_enabled(), X, (const T*)table, idx, (const T*)w, dim, table_rows, streams, eps));
  });
  return 0;
}

int spd_streams_mix_norm(void* out, float* X, const void* a, const void* b, const float* bias, float sa, float sb,
                         float sbias, const float* mix, const float* outw, float mult, const float* inw,
                         const void* w, const int64_t* rows_idx, int64_t rows, int64_t dim, int streams,
                         float eps, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(X && (out == nullptr || w), SPD_E_BADARG, "spd_streams_mix_norm: null pointer");
  SPD_REQUIRE(rows >= 0 && dim > 0 && streams >= 1 && streams <= kMaxStreams, SPD_E_SHAPE,
              "spd_streams_mix_norm: %d streams (1 to %d)", streams, kMaxStreams);
  SPD_REQUIRE(a != nullptr || (b == nullptr && bias == nullptr), SPD_E_BADARG,
              "spd_streams_mix_norm: b / bias without a");
  SPD_REQUIRE(a == nullptr || (mix && outw), SPD_E_BADARG, "spd_streams_mix_norm: a write needs mix and out weights");
  SPD_REQUIRE(rows_idx == nullptr || (a == nullptr && out != nullptr), SPD_E_BADARG,
              "spd_streams_mix_norm: a row selection reads only");
  if (rows == 0) return 0;
  const size_t stash = sizeof(float) * (size_t)dim;
  const bool use_stash = out != nullptr && stash <= 40 * 1024;
  // stream counts 1 to 4, rows of a multiple of 4 elements on 16-byte boundaries: the vector form
  const bool vec = streams <= 4 && dim % 4 == 0 && stash <= 40 * 1024 && aligned16(X) && aligned16(out) && aligned16(a) &&
                   aligned16(b) && aligned16(bias) && aligned16(w) && (dtype == SPD_F32 || dim % 8 == 0);
  SPD_DISPATCH_ANY(dtype, {
    if (vec) {
      auto kern = streams == 1   ? streams_mix_norm_vec_kernel<T, 1>
                  : streams == 2 ? streams_mix_norm_vec_kernel<T, 2>
                  : streams == 3 ? streams_mix_norm_vec_kernel<T, 3>
                                 : streams_mix_norm_vec_kernel<T, 4>;
      SPD_CUDA(launch(kern, dim3((unsigned)rows), dim3(kStrThreads), out != nullptr ? stash : 0, as_stream(stream),
                      pdl_enabled(), (T*)out, X, (const T*)a, (const T*)b, bias, sa, sb, sbias, mix, outw, mult, inw,
                      (const T*)w, rows_idx, dim, eps));
    } else {
      auto kern = use_stash ? streams_mix_norm_kernel<T, true> : streams_mix_norm_kernel<T, false>;
      SPD_CUDA(launch(kern, dim3((unsigned)rows), dim3(kStrThreads), use_stash ? stash : 0, as_stream(stream),
                      pdl_enabled(), (T*)out, X, (const T*)a, (const T*)b, bias, sa, sb, sbias, mix, outw, mult, inw,
                      (const T*)w, rows_idx, dim, streams, eps));
    }
  });
  return 0;
}

int spd_rotary_bias_store(void* q_out, const void* q, const void* k, const void* v, const float* q_bias,
                          const float* k_bias, void* k_pool, void* v_pool, const int64_t* loc,
                          const int64_t* positions, const float* cos_sin, int rot_dims, int64_t max_positions,
                          int64_t tokens, int num_q_heads, int num_kv_heads, int head_dim, int v_dim,
                          int64_t q_stride, int64_t k_stride, int64_t v_stride, int64_t q_out_stride, int dtype,
                          spd_stream_t stream) {
  SPD_REQUIRE(q_out && q && k && k_pool && loc && positions, SPD_E_BADARG, "spd_rotary_bias_store: null pointer");
  SPD_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0 && v_dim > 0, SPD_E_BADARG,
              "spd_rotary_bias_store: bad sizes");
  SPD_REQUIRE(rot_dims >= 0 && rot_dims <= head_dim && rot_dims % 2 == 0 && (rot_dims == 0 || (cos_sin && max_positions > 0)),
              SPD_E_BADARG, "spd_rotary_bias_store: bad rotation (rot_dims %d)", rot_dims);
  SPD_REQUIRE(v != nullptr || v_pool == nullptr || v_dim == head_dim, SPD_E_SHAPE,
              "spd_rotary_bias_store: keys as values need v_dim %d = head_dim %d", v_dim, head_dim);
  if (tokens == 0) return 0;
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  const bool vec = (rot_dims / 2) % vecn == 0 && head_dim % vecn == 0 && q_stride % vecn == 0 && k_stride % vecn == 0 &&
                   q_out_stride % vecn == 0 && aligned16(q) && aligned16(k) && aligned16(q_out) && aligned16(k_pool) &&
                   aligned16(v_pool);
  SPD_DISPATCH_ANY(dtype, {
    auto kern = vec ? rotary_bias_store_vec_kernel<T> : rotary_bias_store_kernel<T>;
    SPD_CUDA(launch(kern, dim3((unsigned)tokens), dim3(128), 0, as_stream(stream), pdl_enabled(),
                    (T*)q_out, (const T*)q, (const T*)k, (const T*)v, q_bias, k_bias, (T*)k_pool, (T*)v_pool, loc,
                    positions, cos_sin, rot_dims, max_positions, num_q_heads, num_kv_heads, head_dim, v_dim, q_stride,
                    k_stride, v_stride, q_out_stride));
  });
  return 0;
}

}  // extern "C"
