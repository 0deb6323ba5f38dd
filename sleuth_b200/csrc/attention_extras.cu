// Post-processing of float32 query/key/value rows into the query buffer and the paged cache for attention forms whose
// heads come in units of several score maps, and the combination of two score maps into one head (differential attention).
//
//   unit_post_kernel     a row is [q units | k units | v units]: q has heads * maps units of `dim` channels, k has
//                        kv_heads * maps, v has kv_heads units of `vdim` channels. A q or k unit is optionally divided by
//                        its root mean square (times a gain of `dim` values), then its first `rot` channels turn in
//                        pairs (i, i + rot/2) by the token's position. q goes to [tokens, heads * maps, dim]; k to the
//                        cache row of the token, whose key part is [maps * dim] wide per kv head; v to its value row.
//   diff_combine_kernel  o = a1 - lambda * a2 per head, divided by its root mean square, times `post`, times
//                        sigmoid(gate[t, h])
#include <math.h>

#include "common.cuh"

namespace slb {

struct UnitPostArgs {
  const float* rows;        // [tokens, row_stride]
  long long row_stride;
  const float* q_gain;      // [dim] or null
  const float* k_gain;      // [dim] or null
  const float* cos;         // [positions, rot / 2] or null
  const float* sin;
  void* q_out;              // [tokens, heads * maps, dim]
  void* k_pool;             // [pages, kv_heads, 64, maps * dim] or null (a layer that reads another's cache)
  void* v_pool;             // [pages, kv_heads, 64, vdim]
  const int* tok_seq;
  const int* tok_pos;
  const int* block_table;
  int table_stride;
  int tokens, heads, kv_heads, maps, dim, vdim, rot;
  int writes_kv;            // 0: the rows hold q units only
  float eps;
  int pad;                  // W > 0: a q unit's row in q_out, a key row and a value row of the cache are all W wide; map m's
                            // channels sit at m * dim in a q row too and the rest of that row is zero (the cache's spare channels
                            // are never written and stay zero), so that q . k over W channels is the map's own score
};

// One warp per (token, unit).
template <typename T>
__global__ void __launch_bounds__(256) unit_post_kernel(UnitPostArgs a) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int q_units = a.heads * a.maps, k_units = a.writes_kv ? a.kv_heads * a.maps : 0, v_units = a.writes_kv ? a.kv_heads : 0;
  const int units = q_units + k_units + v_units;
  if (item >= (long long)a.tokens * units) return;
  const int t = (int)(item / units), u = (int)(item - (long long)t * units);
  const float* row = a.rows + (size_t)t * a.row_stride;
  const int pos = a.tok_pos[t];
  T* cache_row = nullptr;
  const size_t key_row = a.pad ? a.pad : (size_t)a.maps * a.dim, value_row = a.pad ? a.pad : a.vdim;
  if (u >= q_units) {
    const int page = a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens];
    const int in_page = pos % kPageTokens;
    if (u < q_units + k_units) {
      const int ku = u - q_units, kh = ku / a.maps, map = ku % a.maps;
      cache_row = (T*)a.k_pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + in_page) * key_row + (size_t)map * a.dim;
    } else {
      const int kh = u - q_units - k_units;
      const float* src = row + (size_t)(q_units + k_units) * a.dim + (size_t)kh * a.vdim;
      T* dst = (T*)a.v_pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + in_page) * value_row;
      for (int c = lane; c < a.vdim; c += 32) dst[c] = from_f32<T>(src[c]);
      return;
    }
  }
  const bool is_q = u < q_units;
  const float* src = row + (size_t)u * a.dim;            // q units, then k units, all `dim` wide
  T* dst = is_q ? (T*)a.q_out + ((size_t)t * q_units + u) * a.dim : cache_row;
  if (is_q && a.pad) {
    T* wide = (T*)a.q_out + ((size_t)t * q_units + u) * a.pad;
    const int lo = (u % a.maps) * a.dim;
    for (int c = lane; c < a.pad; c += 32)
      if (c < lo || c >= lo + a.dim) wide[c] = from_f32<T>(0.0f);
    dst = wide + lo;
  }
  const float* gain = is_q ? a.q_gain : a.k_gain;
  float r = 1.0f;
  if (gain) {
    float ss = 0.0f;
    for (int c = lane; c < a.dim; c += 32) ss = fmaf(src[c], src[c], ss);
    r = 1.0f / sqrtf(warp_sum(ss) / (float)a.dim + a.eps);
  }
  const int half = a.rot / 2;
  for (int i = lane; i < half; i += 32) {
    float x = src[i] * r, y = src[i + half] * r;
    if (gain) { x *= gain[i]; y *= gain[i + half]; }
    const float c = a.cos[(size_t)pos * half + i], s = a.sin[(size_t)pos * half + i];
    dst[i] = from_f32<T>(x * c - y * s);
    dst[i + half] = from_f32<T>(y * c + x * s);
  }
  for (int c = a.rot + lane; c < a.dim; c += 32) {
    float x = src[c] * r;
    if (gain) x *= gain[c];
    dst[c] = from_f32<T>(x);
  }
}

// One warp per (token, head). a: [tokens, heads, 2, a_row] float32 (the first vdim values of a row count); gate:
// [tokens, gate_stride] float32 or null.
template <typename T>
__global__ void __launch_bounds__(256) diff_combine_kernel(const float* __restrict__ a, const float* __restrict__ gate,
                                                           long long gate_stride, T* __restrict__ out, int tokens, int heads,
                                                           int vdim, float lambda, float post, float eps, int a_row) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item - (long long)t * heads);
  const float* a1 = a + (size_t)item * 2 * a_row;
  const float* a2 = a1 + a_row;
  float ss = 0.0f;
  for (int c = lane; c < vdim; c += 32) {
    const float v = a1[c] - lambda * a2[c];
    ss = fmaf(v, v, ss);
  }
  float f = post / sqrtf(warp_sum(ss) / (float)vdim + eps);
  if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
  T* o = out + (size_t)item * vdim;
  for (int c = lane; c < vdim; c += 32) o[c] = from_f32<T>((a1[c] - lambda * a2[c]) * f);
}

}  // namespace slb

using namespace slb;

extern "C" int slb_unit_post(const float* rows, long long row_stride, const float* q_gain, const float* k_gain,
                             const float* cos, const float* sin, void* q_out, void* k_pool, void* v_pool,
                             const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride, int tokens,
                             int heads, int kv_heads, int maps, int dim, int vdim, int rot, int writes_kv, float eps,
                             int pad, int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && maps >= 1 && dim > 0 && vdim > 0,
              "unit_post: heads=%d kv_heads=%d maps=%d dim=%d vdim=%d", heads, kv_heads, maps, dim, vdim);
  SLB_REQUIRE(rot >= 0 && rot <= dim && rot % 2 == 0 && (rot == 0 || (cos != nullptr && sin != nullptr)),
              "unit_post: %d rotated channels of %d", rot, dim);
  SLB_REQUIRE(!writes_kv || (k_pool != nullptr && v_pool != nullptr && block_table != nullptr && table_stride > 0),
              "unit_post: the cache to write is missing");
  SLB_REQUIRE(pad == 0 || (pad >= maps * dim && pad >= vdim), "unit_post: rows of %d channels do not hold %d maps of %d or %d values", pad, maps, dim, vdim);
  const long long need = (long long)heads * maps * dim + (writes_kv ? (long long)kv_heads * maps * dim + (long long)kv_heads * vdim : 0);
  SLB_REQUIRE(row_stride >= need, "unit_post: rows of %lld values do not hold %lld", row_stride, need);
  if (tokens == 0) return 0;
  UnitPostArgs a{rows, row_stride, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table, table_stride,
                 tokens, heads, kv_heads, maps, dim, vdim, rot, writes_kv, eps, pad};
  const long long units = (long long)heads * maps + (writes_kv ? (long long)kv_heads * (maps + 1) : 0);
  const long long warps = (long long)tokens * units;
  const dim3 grid((unsigned)((warps + 7) / 8)), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch(unit_post_kernel<float>, grid, block, 0, s, a);
  else if (dtype == kBF16) launch(unit_post_kernel<__nv_bfloat16>, grid, block, 0, s, a);
  else return fail(1, "unit_post: unknown dtype %d", dtype);
  return check_launch("unit_post");
}

extern "C" int slb_diff_combine(const float* a, const float* gate, long long gate_stride, void* out, int tokens, int heads,
                                int vdim, float lambda, float post, float eps, int a_row, int dtype, void* stream) {
  if (a_row == 0) a_row = vdim;
  SLB_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && a_row >= vdim && (gate == nullptr || gate_stride >= heads),
              "diff_combine: heads=%d vdim=%d", heads, vdim);
  if (tokens == 0) return 0;
  const long long warps = (long long)tokens * heads;
  const dim3 grid((unsigned)((warps + 7) / 8)), block(256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch(diff_combine_kernel<float>, grid, block, 0, s, a, gate, gate_stride, (float*)out, tokens, heads, vdim, lambda, post, eps, a_row);
  else if (dtype == kBF16)
    launch(diff_combine_kernel<__nv_bfloat16>, grid, block, 0, s, a, gate, gate_stride, (__nv_bfloat16*)out, tokens, heads, vdim, lambda, post, eps, a_row);
  else return fail(1, "diff_combine: unknown dtype %d", dtype);
  return check_launch("diff_combine");
}
