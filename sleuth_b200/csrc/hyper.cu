// Several copies of the residual stream (hyper-connections) and the sums that join the results of mixers or experts
// that run side by side. The stream is float32 [tokens, S, d] (S copies of a token's row lie together).
//
//   streams_fill_kernel   every copy <- the embedding's row
//   hyper_read_kernel     u = sum_s in[s] x_s, then h = u / rms(u) * gain in the run dtype (one block a token)
//   hyper_write_kernel    all copies at once from the old ones: x_r <- sum_s mix[s, r] x_s + mult * out[r] * y
//   streams_sum_kernel    x = sum_s x_s
//   pair_combine_kernel   target (=|+=) 0.5 * (a / rms(a) * ga + b / rms(b) * gb), or sa * a + sb * b without gains
//   row_gate_kernel       target (=|+=) sigmoid(h . w) * y, one gate value a token
//   sigmoid_gate_kernel   y <- y * sigmoid(gate), element by element, in place
#include <math.h>

#include "common.cuh"

namespace slb {

constexpr int kMaxStreams = 16;

__global__ void __launch_bounds__(256) streams_fill_kernel(const float* __restrict__ x0, float* __restrict__ xs, long long rows,
                                                           int d, int S) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const long long t = i / d;
  const int c = (int)(i - t * d);
  const float v = x0[i];
  for (int s = 0; s < S; ++s) xs[((size_t)t * S + s) * d + c] = v;
}

template <typename T>
__global__ void __launch_bounds__(256) hyper_read_kernel(const float* __restrict__ xs, const float* __restrict__ coef,
                                                         const float* __restrict__ gain, T* __restrict__ out, int d, int S,
                                                         float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const float* row = xs + (size_t)blockIdx.x * S * d;
  float w[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) w[s] = s < S ? (coef ? coef[s] : 1.0f) : 0.0f;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) u = fmaf(w[s], row[(size_t)s * d + c], u);
    ss = fmaf(u, u, ss);
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  T* o = out + (size_t)blockIdx.x * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) u = fmaf(w[s], row[(size_t)s * d + c], u);
    o[c] = from_f32<T>(u * r * gain[c]);
  }
}

// The same with 16-byte loads for widths that are multiples of 4 up to 1,024 * CH: a thread keeps its CH pieces of the
// weighted sum in registers between the sum of squares and the store, so the copies are read once.
template <typename T, int CH>
__global__ void __launch_bounds__(256) hyper_read_vec_kernel(const float* __restrict__ xs, const float* __restrict__ coef,
                                                             const float* __restrict__ gain, T* __restrict__ out, int d, int S,
                                                             float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const float4* row = reinterpret_cast<const float4*>(xs + (size_t)blockIdx.x * S * d);
  const int d4 = d >> 2;
  float w[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) w[s] = s < S ? (coef ? coef[s] : 1.0f) : 0.0f;
  float4 u[CH];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * 256;
    u[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < d4) {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) {
        if (s < S) {
          const float4 v = row[(size_t)s * d4 + c];
          u[j].x = fmaf(w[s], v.x, u[j].x);
          u[j].y = fmaf(w[s], v.y, u[j].y);
          u[j].z = fmaf(w[s], v.z, u[j].z);
          u[j].w = fmaf(w[s], v.w, u[j].w);
        }
      }
      ss += (u[j].x * u[j].x + u[j].y * u[j].y) + (u[j].z * u[j].z + u[j].w * u[j].w);
    }
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  T* o = out + (size_t)blockIdx.x * d;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < d4) {
      const float4 g = reinterpret_cast<const float4*>(gain)[c];
      o[4 * c + 0] = from_f32<T>(u[j].x * r * g.x);
      o[4 * c + 1] = from_f32<T>(u[j].y * r * g.y);
      o[4 * c + 2] = from_f32<T>(u[j].z * r * g.z);
      o[4 * c + 3] = from_f32<T>(u[j].w * r * g.w);
    }
  }
}

// One thread per (token, four channels): the same arithmetic as hyper_write_kernel with 16-byte loads and stores. MAXS: the
// most copies this instance holds in registers (4, 8 or 16), so that few copies do not pay for the registers of many.
template <int MAXS>
__global__ void __launch_bounds__(256) hyper_write_vec_kernel(float* __restrict__ xs, const float* __restrict__ y,
                                                              const float* __restrict__ mix, const float* __restrict__ out_coef,
                                                              long long rows, int d, int S, float mult) {
  pdl_enter();
  const int d4 = d >> 2;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d4) return;
  const long long t = i / d4;
  const int c = (int)(i - t * d4);
  float4* base = reinterpret_cast<float4*>(xs + (size_t)t * S * d) + c;
  float4 old[MAXS];
#pragma unroll
  for (int s = 0; s < MAXS; ++s) old[s] = s < S ? base[(size_t)s * d4] : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 yv = reinterpret_cast<const float4*>(y)[i];
  yv.x *= mult; yv.y *= mult; yv.z *= mult; yv.w *= mult;
#pragma unroll
  for (int r = 0; r < MAXS; ++r) {
    if (r < S) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (mix) {
#pragma unroll
        for (int s = 0; s < MAXS; ++s) {
          if (s < S) {
            const float m = mix[s * S + r];
            v.x = fmaf(m, old[s].x, v.x);
            v.y = fmaf(m, old[s].y, v.y);
            v.z = fmaf(m, old[s].z, v.z);
            v.w = fmaf(m, old[s].w, v.w);
          }
        }
      } else {
        v = old[r];
      }
      const float oc = out_coef ? out_coef[r] : 1.0f;
      base[(size_t)r * d4] = make_float4(fmaf(oc, yv.x, v.x), fmaf(oc, yv.y, v.y), fmaf(oc, yv.z, v.z), fmaf(oc, yv.w, v.w));
    }
  }
}

// One thread per (token, channel). mix: [S, S] indexed [from, to], or null (the identity); out_coef: [S] or null (ones).
__global__ void __launch_bounds__(256) hyper_write_kernel(float* __restrict__ xs, const float* __restrict__ y,
                                                          const float* __restrict__ mix, const float* __restrict__ out_coef,
                                                          long long rows, int d, int S, float mult) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const long long t = i / d;
  const int c = (int)(i - t * d);
  float* base = xs + (size_t)t * S * d + c;
  float old[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) old[s] = s < S ? base[(size_t)s * d] : 0.0f;
  const float yv = mult * y[i];
#pragma unroll
  for (int r = 0; r < kMaxStreams; ++r) {
    if (r < S) {
      float v = 0.0f;
      if (mix) {
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) v = fmaf(mix[s * S + r], old[s], v);
      } else {
        v = old[r];
      }
      base[(size_t)r * d] = fmaf(out_coef ? out_coef[r] : 1.0f, yv, v);
    }
  }
}

__global__ void __launch_bounds__(256) streams_sum_kernel(const float* __restrict__ xs, float* __restrict__ x, long long rows,
                                                          int d, int S) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const long long t = i / d;
  const int c = (int)(i - t * d);
  float v = 0.0f;
  for (int s = 0; s < S; ++s) v += xs[((size_t)t * S + s) * d + c];
  x[i] = v;
}

// One block per token.
__global__ void __launch_bounds__(256) pair_combine_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                           const float* __restrict__ ga, const float* __restrict__ gb, float sa,
                                                           float sb, float eps, float* __restrict__ target, int d,
                                                           int accumulate) {
  pdl_enter();
  __shared__ float scratch[33];
  const float* ra = a + (size_t)blockIdx.x * d;
  const float* rb = b + (size_t)blockIdx.x * d;
  float fa = sa, fb = sb;
  if (ga != nullptr) {            // each row divided by its own root mean square first
    float s1 = 0.0f, s2 = 0.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      s1 = fmaf(ra[c], ra[c], s1);
      s2 = fmaf(rb[c], rb[c], s2);
    }
    fa *= 1.0f / sqrtf(block_sum(s1, scratch) / (float)d + eps);
    fb *= 1.0f / sqrtf(block_sum(s2, scratch) / (float)d + eps);
  }
  float* o = target + (size_t)blockIdx.x * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = ga != nullptr ? fa * ra[c] * ga[c] + fb * rb[c] * gb[c] : fa * ra[c] + fb * rb[c];
    o[c] = accumulate ? o[c] + v : v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) row_gate_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                                       const float* __restrict__ y, float* __restrict__ target, int k, int d,
                                                       int accumulate) {
  pdl_enter();
  __shared__ float scratch[33];
  const T* row = h + (size_t)blockIdx.x * k;
  float dot = 0.0f;
  for (int c = threadIdx.x; c < k; c += blockDim.x) dot = fmaf(to_f32(row[c]), w[c], dot);
  const float g = 1.0f / (1.0f + expf(-block_sum(dot, scratch)));
  const float* yr = y + (size_t)blockIdx.x * d;
  float* o = target + (size_t)blockIdx.x * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = accumulate ? fmaf(g, yr[c], o[c]) : g * yr[c];
}

template <typename T>
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(T* __restrict__ y, const float* __restrict__ gate, long long gate_stride,
                                                           long long rows, int C) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * C) return;
  const long long t = i / C;
  const int c = (int)(i - t * C);
  y[i] = from_f32<T>(to_f32(y[i]) / (1.0f + expf(-gate[(size_t)t * gate_stride + c])));
}

}  // namespace slb

using namespace slb;

static inline dim3 per_element(long long n) { return dim3((unsigned)((n + 255) / 256)); }

extern "C" int slb_streams_fill(const float* x0, float* xs, long long rows, int d, int S, void* stream) {
  SLB_REQUIRE(rows >= 0 && d > 0 && S >= 1, "streams_fill: rows=%lld d=%d streams=%d", rows, d, S);
  if (rows == 0) return 0;
  launch(streams_fill_kernel, per_element(rows * d), dim3(256), 0, (cudaStream_t)stream, x0, xs, rows, d, S);
  return check_launch("streams_fill");
}

extern "C" int slb_hyper_read(const float* xs, const float* coef, const float* gain, void* out, long long rows, int d, int S,
                              float eps, int dtype, void* stream) {
  SLB_REQUIRE(rows >= 0 && rows < (1ll << 31) && d > 0 && S >= 1 && S <= kMaxStreams, "hyper_read: rows=%lld d=%d streams=%d (at most %d)",
              rows, d, S, kMaxStreams);
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (d % 4 == 0 && d <= 4096 && (uintptr_t)xs % 16 == 0 && (uintptr_t)gain % 16 == 0) {
    const dim3 grid((unsigned)rows), block(256);
    const int ch = d <= 1024 ? 1 : (d <= 2048 ? 2 : 4);
    if (dtype == kF32) {
      if (ch == 1) launch(hyper_read_vec_kernel<float, 1>, grid, block, 0, s, xs, coef, gain, (float*)out, d, S, eps);
      else if (ch == 2) launch(hyper_read_vec_kernel<float, 2>, grid, block, 0, s, xs, coef, gain, (float*)out, d, S, eps);
      else launch(hyper_read_vec_kernel<float, 4>, grid, block, 0, s, xs, coef, gain, (float*)out, d, S, eps);
    } else if (dtype == kBF16) {
      if (ch == 1) launch(hyper_read_vec_kernel<__nv_bfloat16, 1>, grid, block, 0, s, xs, coef, gain, (__nv_bfloat16*)out, d, S, eps);
      else if (ch == 2) launch(hyper_read_vec_kernel<__nv_bfloat16, 2>, grid, block, 0, s, xs, coef, gain, (__nv_bfloat16*)out, d, S, eps);
      else launch(hyper_read_vec_kernel<__nv_bfloat16, 4>, grid, block, 0, s, xs, coef, gain, (__nv_bfloat16*)out, d, S, eps);
    } else {
      return fail(1, "hyper_read: unknown dtype %d", dtype);
    }
    return check_launch("hyper_read");
  }
  if (dtype == kF32) launch(hyper_read_kernel<float>, dim3((unsigned)rows), dim3(256), 0, s, xs, coef, gain, (float*)out, d, S, eps);
  else if (dtype == kBF16) launch(hyper_read_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, s, xs, coef, gain, (__nv_bfloat16*)out, d, S, eps);
  else return fail(1, "hyper_read: unknown dtype %d", dtype);
  return check_launch("hyper_read");
}

extern "C" int slb_hyper_write(float* xs, const float* y, const float* mix, const float* out_coef, long long rows, int d, int S,
                               float mult, void* stream) {
  SLB_REQUIRE(rows >= 0 && d > 0 && S >= 1 && S <= kMaxStreams, "hyper_write: rows=%lld d=%d streams=%d (at most %d)", rows, d, S,
              kMaxStreams);
  if (rows == 0) return 0;
  if (d % 4 == 0 && (uintptr_t)xs % 16 == 0 && (uintptr_t)y % 16 == 0) {
    if (S <= 4) launch(hyper_write_vec_kernel<4>, per_element(rows * (d / 4)), dim3(256), 0, (cudaStream_t)stream, xs, y, mix, out_coef, rows, d, S, mult);
    else if (S <= 8) launch(hyper_write_vec_kernel<8>, per_element(rows * (d / 4)), dim3(256), 0, (cudaStream_t)stream, xs, y, mix, out_coef, rows, d, S, mult);
    else launch(hyper_write_vec_kernel<16>, per_element(rows * (d / 4)), dim3(256), 0, (cudaStream_t)stream, xs, y, mix, out_coef, rows, d, S, mult);
  } else {
    launch(hyper_write_kernel, per_element(rows * d), dim3(256), 0, (cudaStream_t)stream, xs, y, mix, out_coef, rows, d, S, mult);
  }
  return check_launch("hyper_write");
}

extern "C" int slb_streams_sum(const float* xs, float* x, long long rows, int d, int S, void* stream) {
  SLB_REQUIRE(rows >= 0 && d > 0 && S >= 1, "streams_sum: rows=%lld d=%d streams=%d", rows, d, S);
  if (rows == 0) return 0;
  launch(streams_sum_kernel, per_element(rows * d), dim3(256), 0, (cudaStream_t)stream, xs, x, rows, d, S);
  return check_launch("streams_sum");
}

extern "C" int slb_pair_combine(const float* a, const float* b, const float* ga, const float* gb, float sa, float sb, float eps,
                                float* target, long long rows, int d, int accumulate, void* stream) {
  SLB_REQUIRE(rows >= 0 && rows < (1ll << 31) && d > 0 && (ga == nullptr) == (gb == nullptr), "pair_combine: rows=%lld d=%d", rows, d);
  if (rows == 0) return 0;
  launch(pair_combine_kernel, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, a, b, ga, gb, sa, sb, eps, target, d, accumulate);
  return check_launch("pair_combine");
}

extern "C" int slb_row_gate(const void* h, const float* w, const float* y, float* target, long long rows, int k, int d,
                            int accumulate, int dtype, void* stream) {
  SLB_REQUIRE(rows >= 0 && rows < (1ll << 31) && k > 0 && d > 0, "row_gate: rows=%lld k=%d d=%d", rows, k, d);
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch(row_gate_kernel<float>, dim3((unsigned)rows), dim3(256), 0, s, (const float*)h, w, y, target, k, d, accumulate);
  else if (dtype == kBF16) launch(row_gate_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, s, (const __nv_bfloat16*)h, w, y, target, k, d, accumulate);
  else return fail(1, "row_gate: unknown dtype %d", dtype);
  return check_launch("row_gate");
}

extern "C" int slb_sigmoid_gate(void* y, const float* gate, long long gate_stride, long long rows, int C, int dtype, void* stream) {
  SLB_REQUIRE(rows >= 0 && C > 0 && gate_stride >= C, "sigmoid_gate: rows=%lld channels=%d", rows, C);
  if (rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch(sigmoid_gate_kernel<float>, per_element(rows * C), dim3(256), 0, s, (float*)y, gate, gate_stride, rows, C);
  else if (dtype == kBF16) launch(sigmoid_gate_kernel<__nv_bfloat16>, per_element(rows * C), dim3(256), 0, s, (__nv_bfloat16*)y, gate, gate_stride, rows, C);
  else return fail(1, "sigmoid_gate: unknown dtype %d", dtype);
  return check_launch("sigmoid_gate");
}
