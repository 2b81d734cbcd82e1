// Operators of decoder layers whose norm keeps no statistics and whose attention comes in several forms:
//   * the embedding with a hashed token-pair table (the previous token of a request is part of its state),
//   * the fp32 residual update fused with a tanh norm  tanh(alpha x) w + b  (plus what a pass of a looped
//     block adds in front of its first layer),
//   * rotary positions over strided "segments" (q, k, v of a merged projection, or the rotated slice of a
//     latent attention's queries and keys), in the paired or the half-split layout, with the biases of the
//     projections added first and the cache write fused,
//   * the step between an attention and its output projection: an elementwise sigmoid gate, optionally on
//     the unit-RMS difference of two attention maps.
// Everything is computed in fp32; 16-bit only at the loads and stores.
#include "common.cuh"
#include "ptx.cuh"

namespace spd {

constexpr int kMixThreads = 256;

__device__ __forceinline__ float mix_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// the request that owns row t of a ragged extend batch (empty entries share their successor's start)
__device__ __forceinline__ int row_request(const int32_t* __restrict__ extend_start_loc,
                                           const int32_t* __restrict__ extend_lens, int batch, int64_t t) {
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((int64_t)extend_start_loc[mid] <= t) lo = mid; else hi = mid - 1;
  }
  while (lo > 0 && extend_lens[lo] == 0) --lo;
  return lo;
}

// x[t] = table[id] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets]   (pair row `buckets` for a
// request's first token).  prev is the row before in the batch, or — for the first row of a request's portion
// — prev_state[slot]; the CTA of that first row also leaves the portion's last token in prev_state[slot].
template <typename T>
__global__ void __launch_bounds__(kMixThreads)
embed_pair_kernel(float* __restrict__ x, const T* __restrict__ table, const T* __restrict__ pair,
                  const int64_t* __restrict__ idx, int32_t* __restrict__ prev_state,
                  const int64_t* __restrict__ req_pool_indices, const int64_t* __restrict__ seq_lens,
                  const int64_t* __restrict__ out_cache_loc, const int32_t* __restrict__ prefix_lens,
                  const int32_t* __restrict__ extend_lens, const int32_t* __restrict__ extend_start_loc, int batch,
                  int64_t dim, int64_t table_rows, float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  __shared__ int64_t s_prev;
  if (threadIdx.x == 0) {
    int64_t prev = -1;  // -1: the request's first token
    if (pair != nullptr) {
      if (seq_lens != nullptr) {
        const int64_t slot = req_pool_indices[t];
        if (seq_lens[t] > 1) prev = prev_state[slot];
        if (out_cache_loc == nullptr || out_cache_loc[t] != 0) prev_state[slot] = (int32_t)idx[t];  // not a padded row
      } else {
        const int r = row_request(extend_start_loc, extend_lens, batch, t);
        const int64_t first = extend_start_loc[r];
        if (t > first) {
          prev = idx[t - 1];
        } else {
          const int64_t slot = req_pool_indices[r];
          if (prefix_lens[r] > 0) prev = prev_state[slot];
          prev_state[slot] = (int32_t)idx[first + extend_lens[r] - 1];
        }
      }
    }
    s_prev = prev;
  }
  __syncthreads();
  int64_t id = idx[t];
  id = id < 0 ? 0 : (id >= table_rows ? table_rows - 1 : id);
  int64_t prow = buckets;
  if (s_prev >= 0) prow = (s_prev * mul_prev + id * mul_cur) % buckets;
  for (int64_t i = threadIdx.x; i < dim; i += kMixThreads) {
    float v = to_f32<T>(table[id * dim + i]) * scale;
    if (pair != nullptr) v += to_f32<T>(pair[prow * dim + i]);
    x[t * dim + i] = v;
  }
}

// x[row] += a[row] + x0[row] + vec (each optional; written back when any is given), then
// out[r] = tanh(alpha x[row]) w + b with row = rows ? rows[r] : r.
template <typename T>
__global__ void __launch_bounds__(kMixThreads)
residual_tanh_norm_kernel(T* __restrict__ out, float* __restrict__ x, const T* __restrict__ a,
                          const float* __restrict__ x0, const float* __restrict__ vec, const T* __restrict__ w,
                          const T* __restrict__ b, const int64_t* __restrict__ rows, int64_t dim, float alpha) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t r = blockIdx.x;
  const int64_t row = rows != nullptr ? rows[r] : r;
  float* xr = x + row * dim;
  const bool update = a != nullptr || x0 != nullptr || vec != nullptr;
  for (int64_t i = threadIdx.x; i < dim; i += kMixThreads) {
    float v = xr[i];
    if (update) {
      if (a != nullptr) v += to_f32<T>(a[row * dim + i]);
      if (x0 != nullptr) v += x0[row * dim + i];
      if (vec != nullptr) v += vec[i];
      xr[i] = v;
    }
    if (out != nullptr) out[r * dim + i] = from_f32<T>(tanhf(alpha * v) * to_f32<T>(w[i]) + to_f32<T>(b[i]));
  }
}

struct RotarySegment {
  const void* src;    // [tokens, ...]: head h of token t starts at src + t * src_row + h * src_head
  const float* bias;  // [heads * head_dim] or null, added before the rotation
  void* dst;          // head h of token t goes to dst + (to_pool ? loc[t] : t) * dst_row + h * dst_head
  int64_t src_row, dst_row;
  int32_t heads, head_dim, rot, src_head, dst_head, to_pool;
};
struct RotarySegments {
  RotarySegment seg[4];
  int n;
};

// The first `rot` channels of every head turn by position * f_i (cos_sin [positions, rot_max] = cos || sin of
// rot_max / 2 angles each; a segment uses the first rot / 2 of both): paired layout, channel 2 i with 2 i + 1;
// half-split layout, channel i with i + rot / 2.  Channels >= rot are copied (plus bias).
template <typename T>
__global__ void __launch_bounds__(128)
rotary_segments_kernel(RotarySegments segs, const int64_t* __restrict__ positions, const int64_t* __restrict__ loc,
                       const float* __restrict__ cos_sin, int rot_max, int64_t max_positions, int paired) {
  griddep_wait();
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  int64_t p = positions[t];
  p = p < 0 ? 0 : (p < max_positions ? p : max_positions - 1);
  const float* cs = cos_sin != nullptr ? cos_sin + p * rot_max : nullptr;
  const int half_max = rot_max >> 1;
  const int64_t slot = loc != nullptr ? loc[t] : 0;
  for (int sidx = 0; sidx < segs.n; ++sidx) {
    const RotarySegment& sg = segs.seg[sidx];
    const T* src = reinterpret_cast<const T*>(sg.src) + t * sg.src_row;
    T* dst = reinterpret_cast<T*>(sg.dst) + (sg.to_pool ? slot : t) * sg.dst_row;
    const int half = sg.rot >> 1;
    const int n = sg.heads * sg.head_dim;
    for (int idx = threadIdx.x; idx < n; idx += 128) {
      const int h = idx / sg.head_dim, d = idx - h * sg.head_dim;
      const float x = to_f32<T>(src[h * sg.src_head + d]) + (sg.bias != nullptr ? sg.bias[idx] : 0.f);
      float y = x;
      if (d < sg.rot) {
        int pd, i;
        bool first;
        if (paired) { pd = d ^ 1; i = d >> 1; first = (d & 1) == 0; }
        else { first = d < half; pd = first ? d + half : d - half; i = first ? d : d - half; }
        const float xp = to_f32<T>(src[h * sg.src_head + pd]) + (sg.bias != nullptr ? sg.bias[h * sg.head_dim + pd] : 0.f);
        const float c = cs[i], sn = cs[half_max + i];
        y = first ? x * c - xp * sn : x * c + xp * sn;
      }
      dst[h * sg.dst_head + d] = from_f32<T>(y);
    }
  }
}

// The same step in 16-byte pieces (every segment: head_dim, rot / 2 — rot in the paired layout —, the head and row
// strides multiples of the vector width; 16-byte aligned pointers).  A work item is one vector of a head: in the
// paired layout it holds whole pairs; in the half-split layout a vector of the first half is handled together with
// its partner vector of the second half.  Same arithmetic, element by element.
template <typename T>
__global__ void __launch_bounds__(128)
rotary_segments_vec_kernel(RotarySegments segs, const int64_t* __restrict__ positions, const int64_t* __restrict__ loc,
                           const float* __restrict__ cos_sin, int rot_max, int64_t max_positions, int paired) {
  griddep_wait();
  griddep_launch_dependents();
  constexpr int N = Vec16<T>::kN;
  const int64_t t = blockIdx.x;
  int64_t p = positions[t];
  p = p < 0 ? 0 : (p < max_positions ? p : max_positions - 1);
  const float* cs = cos_sin != nullptr ? cos_sin + p * rot_max : nullptr;
  const int half_max = rot_max >> 1;
  const int64_t slot = loc != nullptr ? loc[t] : 0;
  for (int sidx = 0; sidx < segs.n; ++sidx) {
    const RotarySegment& sg = segs.seg[sidx];
    const T* src = reinterpret_cast<const T*>(sg.src) + t * sg.src_row;
    T* dst = reinterpret_cast<T*>(sg.dst) + (sg.to_pool ? slot : t) * sg.dst_row;
    const int half = sg.rot >> 1;
    const int per_head = sg.head_dim / N;
    for (int item = threadIdx.x; item < sg.heads * per_head; item += 128) {
      const int h = item / per_head, d0 = (item - h * per_head) * N;
      const T* sp = src + h * sg.src_head;
      T* dp = dst + h * sg.dst_head;
      const float* bs = sg.bias != nullptr ? sg.bias + h * sg.head_dim : nullptr;
      if (d0 >= sg.rot || paired) {
        const Vec16<T> v = ldv(sp + d0);
        float x[N];
#pragma unroll
        for (int i = 0; i < N; ++i) x[i] = to_f32<T>(v.e()[i]) + (bs != nullptr ? bs[d0 + i] : 0.f);
        Vec16<T> o;
        if (d0 < sg.rot) {
#pragma unroll
          for (int i = 0; i < N; i += 2) {
            const float c = cs[(d0 + i) >> 1], sn = cs[half_max + ((d0 + i) >> 1)];
            o.e()[i] = from_f32<T>(x[i] * c - x[i + 1] * sn);
            o.e()[i + 1] = from_f32<T>(x[i + 1] * c + x[i] * sn);
          }
        } else {
#pragma unroll
          for (int i = 0; i < N; ++i) o.e()[i] = from_f32<T>(x[i]);
        }
        stv(dp + d0, o);
      } else if (d0 < half) {
        const Vec16<T> va = ldv(sp + d0), vb = ldv(sp + d0 + half);
        Vec16<T> oa, ob;
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float a = to_f32<T>(va.e()[i]) + (bs != nullptr ? bs[d0 + i] : 0.f);
          const float b = to_f32<T>(vb.e()[i]) + (bs != nullptr ? bs[d0 + half + i] : 0.f);
          const float c = cs[d0 + i], sn = cs[half_max + d0 + i];
          oa.e()[i] = from_f32<T>(a * c - b * sn);
          ob.e()[i] = from_f32<T>(b * c + a * sn);
        }
        stv(dp + d0, oa);
        stv(dp + d0 + half, ob);
      }  // vectors of the second half were written with their partners
    }
  }
}

// out[t, h, c] = y[c] * sigmoid(gate[t, h * vdim + c]) with y = a[t, h, :] or, a2 given,
// y = unit_rms(a - lambda a2) * post  (unit RMS over the head's vdim values, eps inside the root).
template <typename T>
__global__ void __launch_bounds__(128)
heads_gate_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ a2, const T* __restrict__ gate,
                  int64_t tokens, int heads, int vdim, int64_t a_stride, int64_t gate_stride, int64_t out_stride,
                  float lambda, float eps, float post) {
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t item = blockIdx.x * 4ll + (threadIdx.x >> 5);
  if (item >= tokens * heads) return;
  const int64_t t = item / heads;
  const int h = (int)(item - t * heads);
  const T* ar = a + t * a_stride + (int64_t)h * vdim;
  const T* gr = gate + t * gate_stride + (int64_t)h * vdim;
  T* orow = out + t * out_stride + (int64_t)h * vdim;
  float mul = 1.f;
  const T* br = nullptr;
  if (a2 != nullptr) {
    br = a2 + t * a_stride + (int64_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) {
      const float d = to_f32<T>(ar[c]) - lambda * to_f32<T>(br[c]);
      ss += d * d;
    }
    ss = warp_sum(ss);
    mul = post / sqrtf(ss / (float)vdim + eps);
  }
  for (int c = lane; c < vdim; c += 32) {
    float y = to_f32<T>(ar[c]);
    if (br != nullptr) y = (y - lambda * to_f32<T>(br[c])) * mul;
    orow[c] = from_f32<T>(y * mix_sigmoid(to_f32<T>(gr[c])));
  }
}

}  // namespace spd

using namespace spd;

extern "C" {

int spd_embed_pair(float* x, const void* table, const void* pair, const int64_t* idx, int32_t* prev_state,
                   const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                   const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                   int64_t batch, int64_t tokens, int64_t dim, int64_t table_rows, float scale, int64_t buckets,
                   int64_t mul_prev, int64_t mul_cur, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(x && table && idx, SPD_E_BADARG, "spd_embed_pair: null pointer");
  SPD_REQUIRE(tokens >= 0 && dim > 0 && table_rows > 0, SPD_E_BADARG, "spd_embed_pair: bad sizes");
  if (pair != nullptr) {
    SPD_REQUIRE(prev_state && req_pool_indices && buckets > 0, SPD_E_BADARG,
                "spd_embed_pair: the pair table needs the previous-token state and the request slots");
    SPD_REQUIRE(seq_lens != nullptr || (prefix_lens && extend_lens && extend_start_loc), SPD_E_BADARG,
                "spd_embed_pair: extend needs prefix_lens, extend_lens and extend_start_loc");
    SPD_REQUIRE(seq_lens == nullptr || batch == tokens, SPD_E_BADARG, "spd_embed_pair: decode has one row per request");
    SPD_REQUIRE(batch > 0 && batch < (1ll << 31), SPD_E_BADARG, "spd_embed_pair: bad batch");
  }
  if (tokens == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(embed_pair_kernel<T>, dim3((unsigned)tokens), dim3(kMixThreads), 0, as_stream(stream), pdl_enabled(),
                    x, (const T*)table, (const T*)pair, idx, prev_state, req_pool_indices, seq_lens, out_cache_loc,
                    prefix_lens, extend_lens, extend_start_loc, (int)batch, dim, table_rows, scale, buckets, mul_prev,
                    mul_cur));
  });
  return 0;
}

int spd_residual_tanh_norm(void* out, float* x, const void* a, const float* x0, const float* vec, const void* w,
                           const void* b, const int64_t* rows, int64_t n_rows, int64_t dim, float alpha, int dtype,
                           spd_stream_t stream) {
  SPD_REQUIRE(x && (out == nullptr) == (w == nullptr) && (w == nullptr) == (b == nullptr), SPD_E_BADARG,
              "spd_residual_tanh_norm: null pointer");
  SPD_REQUIRE(rows == nullptr || (a == nullptr && x0 == nullptr && vec == nullptr), SPD_E_BADARG,
              "spd_residual_tanh_norm: selected rows are read only");
  SPD_REQUIRE(n_rows >= 0 && dim > 0, SPD_E_BADARG, "spd_residual_tanh_norm: bad sizes");
  if (n_rows == 0) return 0;
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(residual_tanh_norm_kernel<T>, dim3((unsigned)n_rows), dim3(kMixThreads), 0, as_stream(stream),
                    pdl_enabled(), (T*)out, x, (const T*)a, x0, vec, (const T*)w, (const T*)b, rows, dim, alpha));
  });
  return 0;
}

int spd_rotary_segments(const spd_rotary_segment_t* segments, int num_segments, const int64_t* positions,
                        const int64_t* loc, const float* cos_sin, int rot_max, int64_t max_positions, int paired,
                        int64_t tokens, int dtype, spd_stream_t stream) {
  SPD_REQUIRE(segments && positions && num_segments >= 1 && num_segments <= 4, SPD_E_BADARG,
              "spd_rotary_segments: 1 to 4 segments");
  RotarySegments segs;
  segs.n = num_segments;
  for (int i = 0; i < num_segments; ++i) {
    const spd_rotary_segment_t& s = segments[i];
    SPD_REQUIRE(s.src && s.dst && s.heads > 0 && s.head_dim > 0 && s.rot >= 0 && s.rot <= s.head_dim && s.rot % 2 == 0 &&
                    s.rot <= rot_max, SPD_E_SHAPE, "spd_rotary_segments: segment %d: bad sizes", i);
    SPD_REQUIRE(s.rot == 0 || cos_sin != nullptr, SPD_E_BADARG, "spd_rotary_segments: rotation without a table");
    SPD_REQUIRE(!s.to_pool || loc != nullptr, SPD_E_BADARG, "spd_rotary_segments: a cache segment needs slot ids");
    segs.seg[i] = RotarySegment{s.src, s.bias, s.dst, s.src_row, s.dst_row, s.heads, s.head_dim, s.rot, s.src_head,
                                s.dst_head, s.to_pool};
  }
  if (tokens == 0) return 0;
  const int vecn = dtype == SPD_F32 ? 4 : 8;
  bool vec = true;
  for (int i = 0; i < num_segments; ++i) {
    const RotarySegment& s = segs.seg[i];
    vec = vec && s.head_dim % vecn == 0 && (paired ? s.rot : s.rot / 2) % vecn == 0 && s.src_head % vecn == 0 &&
          s.dst_head % vecn == 0 && s.src_row % vecn == 0 && s.dst_row % vecn == 0 && aligned16(s.src) && aligned16(s.dst);
  }
  SPD_DISPATCH_ANY(dtype, {
    auto kern = vec ? rotary_segments_vec_kernel<T> : rotary_segments_kernel<T>;
    SPD_CUDA(launch(kern, dim3((unsigned)tokens), dim3(128), 0, as_stream(stream), pdl_enabled(), segs, positions, loc,
                    cos_sin, rot_max, max_positions, paired));
  });
  return 0;
}

int spd_heads_gate(void* out, const void* a, const void* a2, const void* gate, int64_t tokens, int heads, int vdim,
                   int64_t a_stride, int64_t gate_stride, int64_t out_stride, float lambda, float eps, float post,
                   int dtype, spd_stream_t stream) {
  SPD_REQUIRE(out && a && gate, SPD_E_BADARG, "spd_heads_gate: null pointer");
  SPD_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0, SPD_E_BADARG, "spd_heads_gate: bad sizes");
  if (tokens == 0) return 0;
  const int64_t ctas = (tokens * heads + 3) / 4;
  SPD_REQUIRE(ctas < (1ll << 31), SPD_E_SHAPE, "spd_heads_gate: batch too large");
  SPD_DISPATCH_ANY(dtype, {
    SPD_CUDA(launch(heads_gate_kernel<T>, dim3((unsigned)ctas), dim3(128), 0, as_stream(stream), pdl_enabled(), (T*)out,
                    (const T*)a, (const T*)a2, (const T*)gate, tokens, heads, vdim, a_stride, gate_stride, out_stride,
                    lambda, eps, post));
  });
  return 0;
}

}  // extern "C"
