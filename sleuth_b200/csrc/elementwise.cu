// Row-wise kernels between the matrix products: embedding lookup, RMSNorm, residual add, gated activation.
#include "common.cuh"

namespace slb {

// x[t, :] = table[ids[t], :] * scale, into the float32 residual stream.
// (Token rows looked up without scaling unless the model sets one: sleuth/forge/model/transformer.py:345-348.)
// With `map`, row t takes token ids[map[t]]: a decode step can then read the tokens the sampler left on the
// device for the previous batch, whose rows need not be this batch's rows.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ map, const TW* __restrict__ table,
                             float* __restrict__ x, int dim, int vocab, float scale) {
  Tracer trace(kTraceEmbed);
  pdl_enter();
  trace.mark(1);
  const int t = blockIdx.x;
  int tok = ids[map ? map[t] : t];
  tok = min(max(tok, 0), vocab - 1);
  const TW* row = table + (size_t)tok * dim;
  float* out = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

// out[r, :] = (x[row(r), :] * (1 / sqrt(mean(x^2) + eps))) * w, float32 arithmetic, one rounding at the store.
// row(r) = rows[r] when `rows` is given (the final norm runs only on the rows whose logits are wanted).
// (sleuth/forge/model/norm.py:50; the reference's own fused form: sleuth/forge/model/fused_ops.py:41-51.)
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>((xr[i] * inv) * w[i]);
}

// The same for widths that are multiples of 4: 16-byte loads, the row kept in registers between the two passes.
template <typename TO, int PER_THREAD>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int dim, float eps) {
  Tracer trace(kTraceNorm);
  pdl_enter();
  trace.mark(1);
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 v[PER_THREAD], gains[PER_THREAD];      // the gains are asked for with the row, not after the sum
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    gains[i] = c < n4 ? w4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c >= n4) continue;
    const float4 g = gains[i];
    const float a = (v[i].x * inv) * g.x, b = (v[i].y * inv) * g.y, cc = (v[i].z * inv) * g.z, d = (v[i].w * inv) * g.w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(o)[c] = make_float4(a, b, cc, d);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(o)[c] = pk;
    }
  }
}

// x += delta (delta in the activation dtype), float32 sum.
template <typename TD>
__global__ void add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) x[i] += to_f32(delta[i]);
}

// act[t, j] = silu(gu[t, j]) * gu[t, inter + j], silu(z) = z / (1 + exp(-z)); float32 arithmetic.
// (sleuth/forge/model/mlp.py:37-40.)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / inter, j = i - t * inter;
    const float g = to_f32(gu[t * 2 * inter + j]);
    const float u = to_f32(gu[t * 2 * inter + inter + j]);
    act[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
  }
}

// bfloat16, inter a multiple of 8: 16 bytes of gate and of up per thread.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int inter,
                                     size_t total8) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  const int per_row = inter >> 3;
  for (; i < total8; i += step) {
    const size_t t = i / per_row, j = (i - t * per_row) << 3;
    const Bf16x8 g = *reinterpret_cast<const Bf16x8*>(gu + t * 2 * inter + j);
    const Bf16x8 u = *reinterpret_cast<const Bf16x8*>(gu + t * 2 * inter + inter + j);
    float gf[8], uf[8];
    unpack8(g, gf);
    unpack8(u, uf);
    Bf16x8 o;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = (gf[2 * e] / (1.0f + expf(-gf[2 * e]))) * uf[2 * e];
      const float b = (gf[2 * e + 1] / (1.0f + expf(-gf[2 * e + 1]))) * uf[2 * e + 1];
      o.v[e] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<Bf16x8*>(act + t * inter + j) = o;
  }
}

// act[t, j] = f(gu[t, j], gu[t, inter + j]) for the gated activations of common.cuh; float32 arithmetic. (The SiLU form
// has kernels of its own above.)
template <typename T>
__global__ void gate_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, size_t total, GateAct f) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / inter, j = i - t * inter;
    const float g = to_f32(gu[t * 2 * inter + j]);
    const float u = to_f32(gu[t * 2 * inter + inter + j]);
    act[i] = from_f32<T>(gated(f, g, u));
  }
}

// Layer norm with a gain and no bias: out[r, :] = (x[row(r), :] - mean) / sqrt(var + eps) * w, var = the mean of the
// squared deviations (formed from the deviations, in a second pass over the row, which sits in shared memory), float32
// arithmetic, one rounding at the store. out may be x itself (float32): a block reads its whole row before it writes.
template <typename TO>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                 const int* __restrict__ rows, int dim, float eps) {
  pdl_enter();
  extern __shared__ float row[];        // [dim]
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = xr[i];
    row[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)dim;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float d = row[i] - mean;
    ss = fmaf(d, d, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>(((row[i] - mean) * inv) * w[i]);
}

// The same for widths that are multiples of 4 (16-byte loads, the row kept in registers between the passes), and for two
// gains at once: two norms of the same rows that differ in their gains only (the two norms of a parallel layer) share the
// mean and the variance, so one pass over the stream serves both; out2 null: one output.
template <typename TO, int PER_THREAD>
__global__ void layernorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                     const float* __restrict__ w2, TO* __restrict__ out2, const int* __restrict__ rows,
                                     int dim, float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  float4 v[PER_THREAD];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = block_sum(sum, scratch) / (float)dim;
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < n4) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      ss = fmaf(v[i].x, v[i].x, ss);
      ss = fmaf(v[i].y, v[i].y, ss);
      ss = fmaf(v[i].z, v[i].z, ss);
      ss = fmaf(v[i].w, v[i].w, ss);
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + eps);
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const float* gw = pass ? w2 : w;
    TO* o = (pass ? out2 : out);
    if (o == nullptr) continue;
    o += (size_t)r * dim;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c >= n4) continue;
      const float4 g = reinterpret_cast<const float4*>(gw)[c];
      const float a = (v[i].x * inv) * g.x, b = (v[i].y * inv) * g.y, cc = (v[i].z * inv) * g.z, d = (v[i].w * inv) * g.w;
      if constexpr (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(o)[c] = make_float4(a, b, cc, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(o)[c] = pk;
      }
    }
  }
}

// v <- cap * tanh(v / cap), in place, float32.
__global__ void softcap_kernel(float* __restrict__ v, long long row_stride, int cols, size_t total, float cap) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  const float inv = 1.0f / cap;
  for (; i < total; i += step) {
    const size_t r = i / cols, c = i - r * cols;
    float* p = v + r * row_stride + c;
    *p = cap * tanhf(*p * inv);
  }
}

// x[t, :] += again[t, :] (if given) + row[:] (if given): what a model adds to the stream between two layer applications.
__global__ void stream_inject_kernel(float* __restrict__ x, const float* __restrict__ again, const float* __restrict__ row,
                                     int dim, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    float v = x[i];
    if (again) v += again[i];
    if (row) v += row[i % dim];
    x[i] = v;
  }
}

// A hashed table of token pairs added to the embedding: x[t, :] += pairs[row(t), :] with
// row = (previous token * mul_prev + token * mul_cur) mod buckets, and row = buckets (the table's last row) for a
// sequence's first token. With `table` the token's own row comes in the same pass: x[t, :] = table[token, :] * scale +
// pairs[row(t), :]. The previous token of a step's first token comes from last[slot], the sequence's state; the
// block of that token then leaves the step's last token there for the next step (it alone reads and writes the entry).
template <typename TW>
__global__ void pair_embed_kernel(const int* __restrict__ ids, const int* __restrict__ map, const TW* __restrict__ pairs,
                                  float* __restrict__ x, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                  const int* __restrict__ seq_start, const int* __restrict__ slots, int* __restrict__ last,
                                  int dim, int vocab, int buckets, long long mul_prev, long long mul_cur,
                                  const TW* __restrict__ table, float scale) {
  pdl_enter();
  const int t = blockIdx.x;
  const int seq = tok_seq[t];
  const bool first = t == seq_start[seq];
  int tok = ids[map ? map[t] : t];
  tok = min(max(tok, 0), vocab - 1);
  long long row = buckets;
  if (tok_pos[t] > 0) {
    int prev = first ? last[slots[seq]] : ids[map ? map[t - 1] : t - 1];
    prev = min(max(prev, 0), vocab - 1);
    row = (prev * mul_prev + tok * mul_cur) % buckets;
    if (row < 0) row += buckets;
  }
  const TW* src = pairs + (size_t)row * dim;
  float* out = x + (size_t)t * dim;
  if (table) {
    const TW* own = table + (size_t)tok * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = fmaf(to_f32(own[i]), scale, to_f32(src[i]));
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] += to_f32(src[i]);
  }
  __syncthreads();      // every warp has read the sequence's previous token before thread 0 replaces it
  if (first && threadIdx.x == 0) {
    const int e = seq_start[seq + 1] - 1;
    last[slots[seq]] = min(max(ids[map ? map[e] : e], 0), vocab - 1);
  }
}

// The end of a sublayer that is gated and normalised before it joins the stream:
//   v = y * sigmoid(g + b) (g absent: v = y);  x += v / sqrt(mean(v^2) + eps) * w
// y [T, dim] float32 (rows too wide for a thread's registers are overwritten with v), g [T, dim] float32 with row stride
// g_stride, b and w [dim] float32.
__global__ void gated_norm_add_kernel(float* __restrict__ x, float* __restrict__ y, const float* __restrict__ g,
                                      long long g_stride, const float* __restrict__ b, const float* __restrict__ w, int dim,
                                      float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  constexpr int kKeep = 8;      // values a thread keeps between the two passes; rows wider than that park the rest in y
  const int r = blockIdx.x;
  float* yr = y + (size_t)r * dim;
  const float* gr = g ? g + (size_t)r * g_stride : nullptr;
  auto gated = [&](int i) {
    float v = yr[i];
    if (gr) {
      const float z = gr[i] + (b ? b[i] : 0.0f);
      v = v * (1.0f / (1.0f + expf(-z)));
    }
    return v;
  };
  float keep[kKeep];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < kKeep; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < dim) {
      keep[k] = gated(i);
      ss = fmaf(keep[k], keep[k], ss);
    }
  }
  for (int i = threadIdx.x + kKeep * blockDim.x; i < dim; i += blockDim.x) {
    const float v = gated(i);
    yr[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  float* xr = x + (size_t)r * dim;
#pragma unroll
  for (int k = 0; k < kKeep; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < dim) xr[i] += (keep[k] * inv) * w[i];
  }
  for (int i = threadIdx.x + kKeep * blockDim.x; i < dim; i += blockDim.x) xr[i] += (yr[i] * inv) * w[i];
}

// The same for rows of whole float4s that fit a block's registers (PER float4s a thread): every load of the row, its gate,
// the stream's row and the gain is asked for before anything is summed, so the kernel waits for memory once.
template <int PER>
__global__ void __launch_bounds__(256) gated_norm_add_vec_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                 const float* __restrict__ g, long long g_stride,
                                                                 const float* __restrict__ b, const float* __restrict__ w, int dim,
                                                                 float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const int r = blockIdx.x, n4 = dim >> 2;
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)r * dim);
  const float4* gr = g ? reinterpret_cast<const float4*>(g + (size_t)r * g_stride) : nullptr;
  const float4* b4 = reinterpret_cast<const float4*>(b);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4* xr = reinterpret_cast<float4*>(x + (size_t)r * dim);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[PER], z[PER], bias[PER], xv[PER], gains[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    const bool in = c < n4;
    v[k] = in ? yr[c] : zero;
    z[k] = in && gr ? gr[c] : zero;
    bias[k] = in && gr && b ? b4[c] : zero;
    xv[k] = in ? xr[c] : zero;
    gains[k] = in ? w4[c] : zero;
  }
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    if (gr) {
      v[k].x = v[k].x * (1.0f / (1.0f + expf(-(z[k].x + bias[k].x))));
      v[k].y = v[k].y * (1.0f / (1.0f + expf(-(z[k].y + bias[k].y))));
      v[k].z = v[k].z * (1.0f / (1.0f + expf(-(z[k].z + bias[k].z))));
      v[k].w = v[k].w * (1.0f / (1.0f + expf(-(z[k].w + bias[k].w))));
    }
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c >= n4) continue;
    xr[c] = make_float4(xv[k].x + (v[k].x * inv) * gains[k].x, xv[k].y + (v[k].y * inv) * gains[k].y,
                        xv[k].z + (v[k].z * inv) * gains[k].z, xv[k].w + (v[k].w * inv) * gains[k].w);
  }
}

// out[t, :] = [a[t, :] | b[t, :]] in the run dtype: two float32 streams side by side as one product's input.
template <typename TO>
__global__ void stream_pair_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out, int dim,
                                   size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / (2 * (size_t)dim), c = i - t * 2 * dim;
    out[i] = from_f32<TO>(c < (size_t)dim ? a[t * dim + c] : b[t * dim + c - dim]);
  }
}

// The same in pieces of four values for widths that are multiples of four.
template <typename TO>
__global__ void stream_pair_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, TO* __restrict__ out, int dim4,
                                       size_t total4) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total4; i += step) {
    const size_t t = i / (2 * (size_t)dim4), c = i - t * 2 * dim4;
    const float4 v = c < (size_t)dim4 ? a[t * dim4 + c] : b[t * dim4 + c - dim4];
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(out)[i] = v;
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(out)[i] = pk;
    }
  }
}

// v *= factor, or with `add` [cols]: v = v * factor + add[col]; v float32 [rows, cols] with a row stride.
__global__ void scale_kernel(float* __restrict__ v, long long row_stride, int cols, size_t total, float factor,
                             const float* __restrict__ add) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t r = i / cols, c = i - r * cols;
    float* p = v + r * row_stride + c;
    *p = add ? fmaf(*p, factor, add[c]) : *p * factor;
  }
}


static int norm_threads(int dim) {
  int t = 32;
  while (t < 512 && t * 4 < dim) t <<= 1;
  return t;
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(elementwise)

extern "C" int slb_embed(const int* ids, const int* map, const void* table, int table_dtype, float* x, int tokens,
                         int dim, int vocab, float scale, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0, "embed: tokens=%d dim=%d vocab=%d", tokens, dim, vocab);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = dim >= 256 ? 256 : 64;
  if (table_dtype == kF32)
    launch(embed_kernel<float>, dim3(tokens), dim3(threads), 0, s, ids, map, (const float*)table, x, dim, vocab, scale);
  else if (table_dtype == kBF16)
    launch(embed_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, s, ids, map, (const __nv_bfloat16*)table, x, dim, vocab, scale);
  else
    return fail(1, "embed: unknown dtype %d", table_dtype);
  return check_launch("embed");
}

extern "C" int slb_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows,
                           int dim, float eps, void* stream) {
  SLB_REQUIRE(n_rows >= 0 && dim > 0 && eps > 0.0f, "rmsnorm: rows=%d dim=%d eps=%g", n_rows, dim, (double)eps);
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  SLB_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "rmsnorm: unknown dtype %d", out_dtype);
  if (dim % 4 == 0 && dim <= 8192 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const int n4 = dim / 4;
    int threads = n4 <= 64 ? 64 : (n4 <= 128 ? 128 : 256);
    // Many rows (prompts), bfloat16 run: half the threads per row, so that twice as many rows are resident and a
    // 2,048-row call runs in one round of blocks instead of two. The float32 run keeps one block shape whatever
    // the row count, so that a row's sum is formed in the same order in every step.
    if (out_dtype == kBF16 && n_rows >= 1024 && threads == 256 && n4 <= 8 * 128) threads = 128;
    const int per = (n4 + threads - 1) / threads;      // at most 8
    #define SLB_NORM(P)                                                                                              \
      if (out_dtype == kF32) launch(rmsnorm_vec_kernel<float, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (float*)out, rows, dim, eps); \
      else launch(rmsnorm_vec_kernel<__nv_bfloat16, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (__nv_bfloat16*)out, rows, dim, eps)
    if (per <= 1) { SLB_NORM(1); } else if (per <= 2) { SLB_NORM(2); } else if (per <= 4) { SLB_NORM(4); } else { SLB_NORM(8); }
    #undef SLB_NORM
    return check_launch("rmsnorm");
  }
  const int threads = norm_threads(dim);
  if (out_dtype == kF32)
    launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, w, (float*)out, rows, dim, eps);
  else
    launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, x, w, (__nv_bfloat16*)out, rows, dim, eps);
  return check_launch("rmsnorm");
}

extern "C" int slb_add(float* x, const void* delta, int delta_dtype, long long n, void* stream) {
  SLB_REQUIRE(n >= 0, "add: n=%lld", n);
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (delta_dtype == kF32)
    launch(add_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, x, (const float*)delta, (size_t)n);
  else if (delta_dtype == kBF16)
    launch(add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, x, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return fail(1, "add: unknown dtype %d", delta_dtype);
  return check_launch("add");
}

extern "C" int slb_swiglu(const void* gu, void* act, int dtype, int tokens, int inter, void* stream) {
  SLB_REQUIRE(tokens >= 0 && inter > 0, "swiglu: tokens=%d inter=%d", tokens, inter);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (dtype == kBF16 && inter % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)act % 16 == 0)) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + threads - 1) / threads;
    if (b8 > sm_count() * 32) b8 = sm_count() * 32;
    launch(swiglu_bf16x8_kernel, dim3((int)b8), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, inter, total8);
    return check_launch("swiglu");
  }
  if (dtype == kF32)
    launch(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, (float*)act, inter, total);
  else if (dtype == kBF16)
    launch(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act,
                                                               inter, total);
  else
    return fail(1, "swiglu: unknown dtype %d", dtype);
  return check_launch("swiglu");
}

// kind: 0 = silu (the kernels of slb_swiglu), 1 = relu, 2 = clamped swish with `limit` and `alpha`, 3 = tanh gelu (common.cuh).
extern "C" int slb_gated_act(const void* gu, void* act, int dtype, int tokens, int inter, int kind, float limit, float alpha,
                             void* stream) {
  if (kind == kGateSilu) return slb_swiglu(gu, act, dtype, tokens, inter, stream);
  SLB_REQUIRE(kind > kGateSilu && kind <= kGateLast, "gated_act: unknown activation %d", kind);
  SLB_REQUIRE(kind != kGateClampedSwish || limit > 0.0f, "gated_act: the clamp limit must be positive, got %g", (double)limit);
  SLB_REQUIRE(tokens >= 0 && inter > 0, "gated_act: tokens=%d inter=%d", tokens, inter);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)tokens * inter;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  const GateAct f{kind, limit, alpha};
  if (dtype == kF32)
    launch(gate_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)gu, (float*)act, inter, total, f);
  else if (dtype == kBF16)
    launch(gate_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, inter, total, f);
  else
    return fail(1, "gated_act: unknown dtype %d", dtype);
  return check_launch("gated_act");
}

// w2 / out2: a second gain and output for the same rows (both null: one norm). out may be x itself when out2 is null.
extern "C" int slb_layernorm(const float* x, const float* w, void* out, const float* w2, void* out2, int out_dtype,
                             const int* rows, int n_rows, int dim, float eps, void* stream) {
  SLB_REQUIRE(n_rows >= 0 && dim > 0 && dim <= 12288 && eps > 0.0f, "layernorm: rows=%d dim=%d (at most 12288) eps=%g", n_rows, dim,
              (double)eps);
  SLB_REQUIRE((w2 == nullptr) == (out2 == nullptr), "layernorm: a second gain and a second output go together");
  SLB_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "layernorm: unknown dtype %d", out_dtype);
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = ((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)w2 | (uintptr_t)out2) % 16 == 0;
  if (dim % 4 == 0 && dim <= 8192 && aligned) {
    const int n4 = dim / 4;
    const int threads = n4 <= 64 ? 64 : (n4 <= 128 ? 128 : 256);      // one shape whatever the row count: the same sums in every step
    const int per = (n4 + threads - 1) / threads;      // at most 8
    #define SLB_LNORM(P)                                                                                              \
      if (out_dtype == kF32) launch(layernorm_vec_kernel<float, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (float*)out, w2, (float*)out2, rows, dim, eps); \
      else launch(layernorm_vec_kernel<__nv_bfloat16, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (__nv_bfloat16*)out, w2, (__nv_bfloat16*)out2, rows, dim, eps)
    if (per <= 1) { SLB_LNORM(1); } else if (per <= 2) { SLB_LNORM(2); } else if (per <= 4) { SLB_LNORM(4); } else { SLB_LNORM(8); }
    #undef SLB_LNORM
    return check_launch("layernorm");
  }
  const int threads = norm_threads(dim);
  const size_t smem = (size_t)dim * sizeof(float);
  for (int pass = 0; pass < (out2 ? 2 : 1); ++pass) {
    const float* gw = pass ? w2 : w;
    void* o = pass ? out2 : out;
    if (out_dtype == kF32)
      launch(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, s, x, gw, (float*)o, rows, dim, eps);
    else
      launch(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, s, x, gw, (__nv_bfloat16*)o, rows, dim, eps);
  }
  return check_launch("layernorm");
}

extern "C" int slb_softcap(float* v, long long row_stride, int rows, int cols, float cap, void* stream) {
  SLB_REQUIRE(rows >= 0 && cols > 0 && row_stride >= cols && cap > 0.0f, "softcap: rows=%d cols=%d stride=%lld cap=%g", rows, cols,
              row_stride, (double)cap);
  if (rows == 0) return 0;
  const size_t total = (size_t)rows * cols;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(softcap_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, v, row_stride, cols, total, cap);
  return check_launch("softcap");
}

extern "C" int slb_stream_inject(float* x, const float* again, const float* row, int tokens, int dim, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0, "stream_inject: tokens=%d dim=%d", tokens, dim);
  if (tokens == 0 || (again == nullptr && row == nullptr)) return 0;
  const size_t total = (size_t)tokens * dim;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(stream_inject_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, x, again, row, dim, total);
  return check_launch("stream_inject");
}

// x [tokens, dim] float32 already holds the tokens' own rows; pairs [buckets + 1, dim]; last: int32 [slots], one
// entry per sequence slot (the sequence's last token so far).
extern "C" int slb_pair_embed(const int* ids, const int* map, const void* pairs, int table_dtype, float* x, const int* tok_seq,
                              const int* tok_pos, const int* seq_start, const int* slots, int* last, int tokens, int dim,
                              int vocab, int buckets, long long mul_prev, long long mul_cur, const void* table, float scale,
                              void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0 && buckets > 0, "pair_embed: tokens=%d dim=%d vocab=%d buckets=%d", tokens, dim,
              vocab, buckets);
  SLB_REQUIRE(mul_prev >= 0 && mul_cur >= 0 && mul_prev < (1LL << 31) && mul_cur < (1LL << 31), "pair_embed: multipliers %lld, %lld",
              mul_prev, mul_cur);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = dim >= 256 ? 256 : 64;
  if (table_dtype == kF32)
    launch(pair_embed_kernel<float>, dim3(tokens), dim3(threads), 0, s, ids, map, (const float*)pairs, x, tok_seq, tok_pos, seq_start,
           slots, last, dim, vocab, buckets, mul_prev, mul_cur, (const float*)table, scale);
  else if (table_dtype == kBF16)
    launch(pair_embed_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, s, ids, map, (const __nv_bfloat16*)pairs, x, tok_seq,
           tok_pos, seq_start, slots, last, dim, vocab, buckets, mul_prev, mul_cur, (const __nv_bfloat16*)table, scale);
  else
    return fail(1, "pair_embed: unknown dtype %d", table_dtype);
  return check_launch("pair_embed");
}

extern "C" int slb_gated_norm_add(float* x, float* y, const float* g, long long g_stride, const float* b, const float* w,
                                  int rows, int dim, float eps, void* stream) {
  SLB_REQUIRE(rows >= 0 && dim > 0 && eps > 0.0f && (g == nullptr || g_stride >= dim), "gated_norm_add: rows=%d dim=%d eps=%g", rows,
              dim, (double)eps);
  if (rows == 0) return 0;
  auto aligned = [](const void* p) { return (uintptr_t)p % 16 == 0; };
  // one block shape for a width whatever the row count, so that a row's sum is formed in the same order in every step
  if (dim % 4 == 0 && dim <= 4096 && g_stride % 4 == 0 && aligned(x) && aligned(y) && aligned(g) && aligned(b) && aligned(w)) {
    const int n4 = dim / 4;
    const int threads = n4 <= 64 ? 64 : (n4 <= 128 ? 128 : 256);
    const int per = (n4 + threads - 1) / threads;      // at most 4
    const float* yc = y;
    if (per <= 1)
      launch(gated_norm_add_vec_kernel<1>, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, x, yc, g, g_stride, b, w, dim, eps);
    else if (per <= 2)
      launch(gated_norm_add_vec_kernel<2>, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, x, yc, g, g_stride, b, w, dim, eps);
    else
      launch(gated_norm_add_vec_kernel<4>, dim3(rows), dim3(threads), 0, (cudaStream_t)stream, x, yc, g, g_stride, b, w, dim, eps);
    return check_launch("gated_norm_add");
  }
  launch(gated_norm_add_kernel, dim3(rows), dim3(norm_threads(dim)), 0, (cudaStream_t)stream, x, y, g, g_stride, b, w, dim, eps);
  return check_launch("gated_norm_add");
}

extern "C" int slb_stream_pair(const float* a, const float* b, void* out, int out_dtype, int tokens, int dim, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0, "stream_pair: tokens=%d dim=%d", tokens, dim);
  SLB_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "stream_pair: unknown dtype %d", out_dtype);
  if (tokens == 0) return 0;
  const size_t total = (size_t)tokens * 2 * dim;
  if (dim % 4 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const size_t total4 = total / 4;
    size_t b4 = (total4 + 255) / 256;
    if (b4 > (size_t)sm_count() * 16) b4 = (size_t)sm_count() * 16;
    if (out_dtype == kF32)
      launch(stream_pair_vec_kernel<float>, dim3((int)b4), dim3(256), 0, (cudaStream_t)stream, (const float4*)a, (const float4*)b,
             (float*)out, dim / 4, total4);
    else
      launch(stream_pair_vec_kernel<__nv_bfloat16>, dim3((int)b4), dim3(256), 0, (cudaStream_t)stream, (const float4*)a,
             (const float4*)b, (__nv_bfloat16*)out, dim / 4, total4);
    return check_launch("stream_pair");
  }
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  if (out_dtype == kF32)
    launch(stream_pair_kernel<float>, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, a, b, (float*)out, dim, total);
  else
    launch(stream_pair_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, a, b, (__nv_bfloat16*)out, dim, total);
  return check_launch("stream_pair");
}

extern "C" int slb_scale(float* v, long long row_stride, int rows, int cols, float factor, const float* add, void* stream) {
  SLB_REQUIRE(rows >= 0 && cols > 0 && row_stride >= cols, "scale: rows=%d cols=%d stride=%lld", rows, cols, row_stride);
  if (rows == 0) return 0;
  const size_t total = (size_t)rows * cols;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(scale_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, v, row_stride, cols, total, factor, add);
  return check_launch("scale");
}
