// Routed experts: router, grouping of (token, choice) pairs by expert, the experts' two products, the weighted sum.
//
// Nothing here needs the host to know how many tokens an expert got: the router counts, a second kernel lays the
// pairs out expert by expert, and the product kernels are launched over the largest number of row tiles that the
// counts could need; a block finds its expert and tile from the counts and leaves when there is none. A step with
// routed experts can therefore be recorded once and replayed.
//
//   moe_route_kernel     logits = W_r h + b in float32, the `top` largest (lowest index first among equals), weights
//                        = softmax over the chosen logits; or (RouteRule) sigmoid scores, the choice limited to the
//                        best groups of neighbouring experts, weights = the chosen scores over their sum, scaled
//   moe_group_kernel     counts the pairs of each expert; place[pair] = where the pair's row lies in the
//                        expert-ordered list, list[place] = pair
//   moe_gate_up_kernel   act[place, j] = f(gate_e[j] . h, up_e[j] . h), f one of the gated activations of common.cuh
//   moe_down_kernel      y[pair, :] = weight[pair] * (down_e act[place])   (float32)
//   moe_combine_kernel   x[t, :] += sum over the token's choices of y, in the order of the choices
// In bfloat16 with inner sizes that are multiples of 8 the two products run on the tensor cores (moe_mma_kernel);
// the kernels above then serve float32 and odd sizes.
#include "mma_sync.cuh"

namespace slb {

constexpr int kMoeTile = 32;        // rows (pairs) of a product tile
constexpr int kMoeCols = 64;        // output columns of a product tile
constexpr int kMoeK = 32;           // inner-dimension slice staged in shared memory
constexpr int kMoeFewPairs = 64;    // up to this many (token, choice) pairs a step runs a warp per output instead of tiles

// Router logits for many tokens: z[t, e] = w[e] . h[t] + b[e], float32, k ascending. A block takes 32 tokens and 16
// experts; the tokens' rows and the experts' rows go through shared memory 128 values at a time; a lane is a token,
// a warp takes two of the experts.
template <typename T>
__global__ void __launch_bounds__(256) moe_logits_kernel(const T* __restrict__ h, const float* __restrict__ wr,
                                                         const float* __restrict__ bias, float* __restrict__ z, int tokens,
                                                         int dim, int E) {
  pdl_enter();
  constexpr int KC = 128;
  __shared__ float hs[32 * (KC + 1)];
  __shared__ float ws[16 * KC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * 32, e0 = blockIdx.y * 16;
  float acc0 = 0.f, acc1 = 0.f;
  for (int k0 = 0; k0 < dim; k0 += KC) {
    const int nk = min(KC, dim - k0);
    __syncthreads();
    if (sizeof(T) == 2 && dim % 8 == 0 && ((uintptr_t)h & 15) == 0) {      // 16 bytes of a row per load
      for (int i = threadIdx.x; i < 32 * (KC / 8); i += 256) {
        const int r = i / (KC / 8), k = (i % (KC / 8)) * 8;
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (t0 + r < tokens && k < nk) unpack8(*reinterpret_cast<const Bf16x8*>(h + (size_t)(t0 + r) * dim + k0 + k), f);
#pragma unroll
        for (int u = 0; u < 8; ++u) hs[r * (KC + 1) + k + u] = f[u];
      }
    } else {
      for (int i = threadIdx.x; i < 32 * KC; i += 256) {
        const int r = i / KC, k = i % KC;
        hs[r * (KC + 1) + k] = (t0 + r < tokens && k < nk) ? to_f32(h[(size_t)(t0 + r) * dim + k0 + k]) : 0.f;
      }
    }
    for (int i = threadIdx.x; i < 16 * KC; i += 256) {
      const int r = i / KC, k = i % KC;
      ws[i] = (e0 + r < E && k < nk) ? wr[(size_t)(e0 + r) * dim + k0 + k] : 0.f;
    }
    __syncthreads();
    const float* mine = hs + lane * (KC + 1);
    const float* wa = ws + warp * KC;
    const float* wb = ws + (warp + 8) * KC;
#pragma unroll 8
    for (int k = 0; k < KC; ++k) {
      const float x = mine[k];
      acc0 = fmaf(x, wa[k], acc0);
      acc1 = fmaf(x, wb[k], acc1);
    }
  }
  if (t0 + lane < tokens) {
    const int ea = e0 + warp, eb = e0 + warp + 8;
    if (ea < E) z[(size_t)(t0 + lane) * E + ea] = acc0 + (bias ? bias[ea] : 0.f);
    if (eb < E) z[(size_t)(t0 + lane) * E + eb] = acc1 + (bias ? bias[eb] : 0.f);
  }
}

// Router logits for few tokens: a warp per (token, expert), so that a single token's step still has experts * 32 lanes
// fetching the router's rows at once (one block walking them alone waits for memory a hundred times in a row).
template <typename T>
__global__ void __launch_bounds__(256) moe_logits_few_kernel(const T* __restrict__ h, const float* __restrict__ wr,
                                                             const float* __restrict__ bias, float* __restrict__ z, int tokens,
                                                             int dim, int E) {
  pdl_enter();
  const int id = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (id >= tokens * E) return;
  const int t = id / E, e = id - t * E;
  const T* row = h + (size_t)t * dim;
  const float* w = wr + (size_t)e * dim;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int i = lane;
  for (; i + 96 < dim; i += 128) {
    s0 = fmaf(to_f32(row[i]), w[i], s0);
    s1 = fmaf(to_f32(row[i + 32]), w[i + 32], s1);
    s2 = fmaf(to_f32(row[i + 64]), w[i + 64], s2);
    s3 = fmaf(to_f32(row[i + 96]), w[i + 96], s3);
  }
  for (; i < dim; i += 32) s0 = fmaf(to_f32(row[i]), w[i], s0);
  const float sum = warp_sum((s0 + s1) + (s2 + s3));
  if (lane == 0) z[id] = sum + (bias ? bias[e] : 0.f);
}

// How the router turns logits into a choice and weights.
//   scoring 0: the `top` largest logits; weights = softmax over those logits alone.
//   scoring 1: scores = sigmoid(logit). The experts form `groups` equal groups of neighbours; a group's score is the sum
//              of its two largest scores (of its one score, if it has one expert); only experts of the `keep` best
//              groups can be chosen. The `top` largest scores among them; weights = score / (sum of the chosen scores
//              + 1e-20) * scale.
//   scoring 2: scores = softmax(logits) over all experts; the `top` largest of score + pick_bias (a correction per expert
//              that moves the choice and never the weights; absent = 0) are chosen; weights = the chosen experts'
//              scores * scale as they are.
//   scoring 3: the scores and the choice of scoring 2; weights = score / (sum of the chosen scores + 1e-20) * scale.
struct RouteRule {
  int scoring, groups, keep;
  float scale;
};

// One block of eight warps per token. Without given logits a warp forms the logits of every eighth expert (the lanes
// share the row, four partial sums each, joined in a fixed order); warp 0 then picks the `top` largest.
template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr,
                                                        const float* __restrict__ bias, const float* __restrict__ pick_bias,
                                                        const float* __restrict__ given, int* __restrict__ choice,
                                                        float* __restrict__ weight, int tokens, int dim, int E, int top,
                                                        RouteRule rule) {
  pdl_enter();
  extern __shared__ float z[];         // [E], then [groups] group scores and [groups] flags when groups limit the choice,
                                       // then (scoring 2) [E] choice scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* row = h + (size_t)t * dim;
  if (given != nullptr) {              // the logits were formed by moe_logits_kernel
    for (int e = threadIdx.x; e < E; e += blockDim.x) z[e] = given[(size_t)t * E + e];
  } else {
    for (int e = warp; e < E; e += 8) {
      const float* w = wr + (size_t)e * dim;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      int i = lane;
      for (; i + 96 < dim; i += 128) {
        s0 = fmaf(to_f32(row[i]), w[i], s0);
        s1 = fmaf(to_f32(row[i + 32]), w[i + 32], s1);
        s2 = fmaf(to_f32(row[i + 64]), w[i + 64], s2);
        s3 = fmaf(to_f32(row[i + 96]), w[i + 96], s3);
      }
      for (; i < dim; i += 32) s0 = fmaf(to_f32(row[i]), w[i], s0);
      const float sum = warp_sum((s0 + s1) + (s2 + s3));
      if (lane == 0) z[e] = sum + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (rule.scoring == 1) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) z[e] = 1.0f / (1.0f + expf(-z[e]));
    __syncthreads();
  }
  if (warp != 0) return;
  if (rule.scoring == 1 && rule.groups > 1 && rule.keep < rule.groups) {
    float* gscore = z + E;
    int* open = reinterpret_cast<int*>(gscore + rule.groups);
    const int size = E / rule.groups;
    for (int g = lane; g < rule.groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;          // the two largest of the group
      for (int e = g * size; e < (g + 1) * size; ++e) {
        const float v = z[e];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gscore[g] = size > 1 ? a + b : a;
      open[g] = 0;
    }
    __syncwarp();
    for (int k = 0; k < rule.keep; ++k) {
      float best = -INFINITY;
      int best_g = rule.groups;
      for (int g = lane; g < rule.groups; g += 32) {
        const float v = gscore[g];
        if (v > best) { best = v; best_g = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (ov > best || (ov == best && og < best_g)) { best = ov; best_g = og; }
      }
      best_g = min(best_g, rule.groups - 1);
      if (lane == 0) { open[best_g] = 1; gscore[best_g] = -INFINITY; }
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!open[e / size]) z[e] = -INFINITY;
    __syncwarp();
  }
  float* sel = z;                      // what the choice looks at
  if (rule.scoring >= 2) {             // 2 and 3: softmax over all experts (3 divides the chosen scores by their sum)
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(z[e] - mx);
      z[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    sel = z + E + 2 * rule.groups;
    for (int e = lane; e < E; e += 32) {
      const float sc = z[e] / sum;
      z[e] = sc;
      sel[e] = sc + (pick_bias ? pick_bias[e] : 0.f);
    }
    __syncwarp();
  }
  float first = 0.f, mass = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = E;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      if (v > best) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    best_e = min(best_e, E - 1);                 // only logits that are not numbers get here
    if (k == 0) first = best;
    const float p = rule.scoring == 2 ? z[best_e] * rule.scale
                                      : (rule.scoring == 3 ? z[best_e] : (rule.scoring == 1 ? best : expf(best - first)));
    mass += p;
    __syncwarp();
    if (lane == 0) {
      choice[(size_t)t * top + k] = best_e;
      weight[(size_t)t * top + k] = p;
      sel[best_e] = -INFINITY;
    }
    __syncwarp();
  }
  if (rule.scoring == 2) return;
  if (rule.scoring == 1 || rule.scoring == 3) {
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] = weight[(size_t)t * top + k] / (mass + 1e-20f) * rule.scale;
  } else {
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] /= mass;
  }
}

// One block lays the pairs out expert by expert: counts[e], then place[pair] = first row of the pair's expert + the
// pair's turn there, and list[place] = pair. The turns come from shared-memory counters, so which of an expert's rows
// a pair gets may differ from run to run; every pair's result is computed from its own row alone, so nothing else does.
// With `tiles`: also the experts' row tiles of `tile_rows` rows for the grouped product: [0] = their number, then
// (expert, first row, rows) each.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ choice, int* __restrict__ counts,
                                                         int* __restrict__ place, int* __restrict__ list, int pairs, int E,
                                                         int* __restrict__ tiles, int tile_rows) {
  pdl_enter();
  extern __shared__ int sh[];          // [E] counts, then [E] first rows / cursors
  int* cnt = sh;
  int* cur = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[choice[p]], 1);
  __syncthreads();
  if (threadIdx.x < 32) {              // exclusive scan over the experts, 32 at a time
    int run = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + threadIdx.x;
      const int c = e < E ? cnt[e] : 0;
      int inc = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if ((int)threadIdx.x >= o) inc += v;
      }
      if (e < E) cur[e] = run + inc - c;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    __syncwarp();
    if (tiles != nullptr && threadIdx.x == 0) {
      int n = 0;
      for (int e = 0; e < E; ++e)
        for (int r = 0; r < cnt[e]; r += tile_rows) {
          tiles[1 + 3 * n] = e;
          tiles[2 + 3 * n] = cur[e] + r;
          tiles[3 + 3 * n] = min(tile_rows, cnt[e] - r);
          ++n;
        }
      tiles[0] = n;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = cnt[e];
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int at = atomicAdd(&cur[choice[p]], 1);
    place[p] = at;
    list[at] = p;
  }
}

// Which expert and which of its row tiles (of `tile` rows) block `b` takes; false when the counts leave it nothing.
__device__ __forceinline__ bool moe_find_tile(const int* counts, int E, int b, int& expert, int& row0, int& rows,
                                              int tile = kMoeTile) {
  int first = 0;
  for (int e = 0; e < E; ++e) {
    const int c = counts[e];
    const int tiles = (c + tile - 1) / tile;
    if (b < tiles) {
      expert = e;
      row0 = first + b * tile;
      rows = min(tile, c - b * tile);
      return true;
    }
    b -= tiles;
    first += c;
  }
  return false;
}

// A 32 x 64 tile of  C = A B^T  on 256 threads (thread: 2 rows x 4 columns), float32 sums, k ascending.
// A rows come through `a_row(r)` (a pointer to the r-th row), B rows through `b_row(c)`.
template <typename T, typename ARow, typename BRow>
__device__ __forceinline__ void moe_tile_product(ARow a_row, BRow b_row, int rows, int cols, int K, float (&acc)[2][4],
                                                 float* As, float* Bs) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // ty: rows ty*2.., tx: columns tx*4..
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kMoeK) {
    const int nk = min(kMoeK, K - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < kMoeTile * kMoeK; i += blockDim.x) {
      const int r = i / kMoeK, k = i % kMoeK;
      As[k * (kMoeTile + 1) + r] = (r < rows && k < nk) ? to_f32(a_row(r)[k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < kMoeCols * kMoeK; i += blockDim.x) {
      const int c = i / kMoeK, k = i % kMoeK;
      Bs[k * (kMoeCols + 1) + c] = (c < cols && k < nk) ? to_f32(b_row(c)[k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kMoeK; ++k) {
      const float a0 = As[k * (kMoeTile + 1) + ty * 2], a1 = As[k * (kMoeTile + 1) + ty * 2 + 1];
      const float* bp = Bs + k * (kMoeCols + 1) + tx * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float bv = bp[j];
        acc[0][j] = fmaf(a0, bv, acc[0][j]);
        acc[1][j] = fmaf(a1, bv, acc[1][j]);
      }
    }
  }
}

// grid (row tiles, column tiles of 32 gate + 32 up columns). w_gu [E, 2 * ff, dim]: gate rows then up rows.
template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu,
                                                          const int* __restrict__ counts, const int* __restrict__ list,
                                                          T* __restrict__ act, int E, int top, int dim, int ff, GateAct gate) {
  pdl_enter();
  __shared__ float As[kMoeK * (kMoeTile + 1)];
  __shared__ float Bs[kMoeK * (kMoeCols + 1)];
  __shared__ int toks[kMoeTile];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows)) return;
  if (threadIdx.x < kMoeTile) toks[threadIdx.x] = threadIdx.x < rows ? list[row0 + threadIdx.x] / top : 0;
  __syncthreads();
  const int j0 = blockIdx.y * 32;
  const int nj = min(32, ff - j0);
  const T* w = w_gu + (size_t)expert * 2 * ff * dim;
  float acc[2][4];
  // tile columns 0..31: gate rows j0.., columns 32..63: up rows j0..
  moe_tile_product<T>([&](int r) { return h + (size_t)toks[r] * dim; },
                      [&](int c) { return w + (size_t)((c < 32 ? 0 : ff) + j0 + min(c & 31, nj - 1)) * dim; }, rows, 64,
                      dim, acc, As, Bs);
  // a thread holds four gate columns or four up columns: pair them through shared memory
  __syncthreads();
  float* Cs = Bs;      // [32 rows][65]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) Cs[(ty * 2 + i) * 65 + tx * 4 + j] = acc[i][j];
  __syncthreads();
  for (int i = threadIdx.x; i < kMoeTile * 32; i += blockDim.x) {
    const int r = i / 32, j = i % 32;
    if (r >= rows || j >= nj) continue;
    const float g = Cs[r * 65 + j], u = Cs[r * 65 + 32 + j];
    act[(size_t)(row0 + r) * ff + j0 + j] = from_f32<T>(gated(gate, g, u));
  }
}

// grid (row tiles, column tiles of 64). w_down [E, dim, ff]. y[pair, :] float32.
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                       const int* __restrict__ counts, const int* __restrict__ list,
                                                       const float* __restrict__ weight, float* __restrict__ y, int E,
                                                       int dim, int ff) {
  pdl_enter();
  __shared__ float As[kMoeK * (kMoeTile + 1)];
  __shared__ float Bs[kMoeK * (kMoeCols + 1)];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows)) return;
  const int n0 = blockIdx.y * kMoeCols;
  const int nn = min(kMoeCols, dim - n0);
  const T* w = w_down + (size_t)expert * dim * ff;
  float acc[2][4];
  moe_tile_product<T>([&](int r) { return act + (size_t)(row0 + r) * ff; },
                      [&](int c) { return w + (size_t)(n0 + min(c, nn - 1)) * ff; }, rows, nn, ff, acc, As, Bs);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
    const int pair = list[row0 + r];
    const float wt = weight[pair];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tx * 4 + j;
      if (c < nn) y[(size_t)pair * dim + n0 + c] = wt * acc[i][j];
    }
  }
}

// ---- the same two products on the warp-level tensor cores (bfloat16, inner sizes that are multiples of 8) ----
// A block of four warps takes 64 rows x 128 columns; a warp 16 rows x all columns (mma.sync m16n8k16, float32 sums).
// The inner dimension goes through shared memory 32 values at a time, two buffers filled by 16-byte asynchronous
// copies; rows are padded to 40 values, which keeps ldmatrix free of bank conflicts. GATED: the 128 columns are 64
// gate rows and the 64 up rows that belong to them, so that a thread holds both halves of each of its outputs.
constexpr int kMmaRows = 64, kMmaCols = 128, kMmaK = 32, kMmaPad = 40;

template <bool GATED>
__global__ void __launch_bounds__(128) moe_mma_kernel(const __nv_bfloat16* __restrict__ a_rows, const __nv_bfloat16* __restrict__ w,
                                                      const int* __restrict__ counts, const int* __restrict__ list,
                                                      const float* __restrict__ weight, __nv_bfloat16* __restrict__ act,
                                                      float* __restrict__ y, int E, int top, int K, int N, GateAct gate) {
  pdl_enter();
  __shared__ __align__(16) __nv_bfloat16 As[2][kMmaRows * kMmaPad];
  __shared__ __align__(16) __nv_bfloat16 Bs[2][kMmaCols * kMmaPad];
  __shared__ int src_row[kMmaRows];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows, kMmaRows)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  // GATED: N = ff, the block's columns are gate rows n0 .. n0 + 63 and up rows N + n0 .. ; A rows are token rows of h.
  // else:  N = the output width, columns n0 .. n0 + 127; A rows are the expert-ordered rows of act.
  const int n0 = blockIdx.y * (GATED ? 64 : kMmaCols);
  const int ncols = min(GATED ? 64 : kMmaCols, N - n0);
  if (tid < kMmaRows) src_row[tid] = tid < rows ? (GATED ? list[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* wb = w + (size_t)expert * (GATED ? 2 : 1) * N * K;

  auto load = [&](int stage, int k0) {
    // 64 rows x 4 sixteen-byte pieces of A, 128 rows x 4 of B
    for (int i = tid; i < kMmaRows * 4; i += 128) {
      const int r = i >> 2, c = (i & 3) * 8;
      __nv_bfloat16* dst = &As[stage][r * kMmaPad + c];
      if (src_row[r] >= 0 && k0 + c < K) cp_async16(smem_u32(dst), a_rows + (size_t)src_row[r] * K + k0 + c);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < kMmaCols * 4; i += 128) {
      const int r = i >> 2, c = (i & 3) * 8;
      __nv_bfloat16* dst = &Bs[stage][r * kMmaPad + c];
      int col;      // the weight row behind tile column r
      if (GATED) col = (r & 63) < ncols ? (r < 64 ? 0 : N) + n0 + (r & 63) : -1;
      else col = r < ncols ? n0 + r : -1;
      if (col >= 0 && k0 + c < K) cp_async16(smem_u32(dst), wb + (size_t)col * K + k0 + c);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  float acc[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int steps = (K + kMmaK - 1) / kMmaK;
  load(0, 0);
  for (int s = 0; s < steps; ++s) {
    const int stage = s & 1;
    if (s + 1 < steps) {
      load(stage ^ 1, (s + 1) * kMmaK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t a_base = smem_u32(&As[stage][0]), b_base = smem_u32(&Bs[stage][0]);
#pragma unroll
    for (int kb = 0; kb < kMmaK / 16; ++kb) {
      uint32_t af[4];
      ldmatrix_x4(af, a_base + 2 * ((warp * 16 + (lane & 15)) * kMmaPad + kb * 16 + ((lane >> 4) << 3)));
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {       // 16 columns at a time
        uint32_t bf[4];
        ldmatrix_x4(bf, b_base + 2 * ((jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kMmaPad + kb * 16 + (((lane >> 3) & 1) << 3)));
        mma_bf16(acc[2 * jp], af, bf[0], bf[1]);
        mma_bf16(acc[2 * jp + 1], af, bf[2], bf[3]);
      }
    }
    __syncthreads();
  }
  // a thread holds rows g and g + 8 of its warp, columns j * 8 + 2 * t4 (+1) of every column tile j
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = warp * 16 + g + 8 * half;
    if (r >= rows) continue;
    if (GATED) {
      __nv_bfloat16* dst = act + (size_t)(row0 + r) * N + n0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = j * 8 + 2 * t4 + e;
          if (c >= ncols) continue;
          const float gv = acc[j][2 * half + e], uv = acc[j + 8][2 * half + e];
          dst[c] = __float2bfloat16_rn(gated(gate, gv, uv));
        }
      }
    } else {
      const int pair = list[row0 + r];
      const float wt = weight[pair];
      float* dst = y + (size_t)pair * N + n0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = j * 8 + 2 * t4 + e;
          if (c < ncols) dst[c] = wt * acc[j][2 * half + e];
        }
      }
    }
  }
}

// ---- few pairs (single-token steps): a warp per output, every weight row streamed once per pair that uses it ----
// (act rows lie in the order of the pairs here: nothing needs the expert order, so a step of few pairs skips the layout.)
// grid (pairs, column groups of 8): act[pair, j] = f(gate_e[j] . h[token]) * (up_e[j] . h[token]).
template <typename T>
__global__ void __launch_bounds__(256) moe_few_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu,
                                                              const int* __restrict__ choice, T* __restrict__ act, int top,
                                                              int dim, int ff, GateAct gate) {
  pdl_enter();
  const int pair = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  if (j >= ff) return;
  const int e = choice[pair];
  const T* x = h + (size_t)(pair / top) * dim;
  const T* wg = w_gu + ((size_t)e * 2 * ff + j) * dim;
  const T* wu = wg + (size_t)ff * dim;
  float g = 0.f, u = 0.f;
  if constexpr (sizeof(T) == 2) {
    if (dim % 8 == 0) {
      for (int k = lane * 8; k < dim; k += 256) {
        float xf[8], gf[8], uf[8];
        unpack8(*reinterpret_cast<const Bf16x8*>(x + k), xf);
        unpack8(*reinterpret_cast<const Bf16x8*>(wg + k), gf);
        unpack8(*reinterpret_cast<const Bf16x8*>(wu + k), uf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          g = fmaf(xf[i], gf[i], g);
          u = fmaf(xf[i], uf[i], u);
        }
      }
    } else {
      for (int k = lane; k < dim; k += 32) {
        const float xv = to_f32(x[k]);
        g = fmaf(xv, to_f32(wg[k]), g);
        u = fmaf(xv, to_f32(wu[k]), u);
      }
    }
  } else {
    for (int k = lane; k < dim; k += 32) {
      const float xv = to_f32(x[k]);
      g = fmaf(xv, to_f32(wg[k]), g);
      u = fmaf(xv, to_f32(wu[k]), u);
    }
  }
  g = warp_sum(g);
  u = warp_sum(u);
  if (lane == 0) {
    act[(size_t)pair * ff + j] = from_f32<T>(gated(gate, g, u));
  }
}

// grid (tokens, column groups of 8): x[t, n] += sum over the token's choices, in their order, of
// weight[pair] * (down_e[n] . act[pair]).
template <typename T>
__global__ void __launch_bounds__(256) moe_few_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                           const int* __restrict__ choice, const float* __restrict__ weight,
                                                           float* __restrict__ x, int top, int dim, int ff) {
  pdl_enter();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y * 8 + warp;
  if (n >= dim) return;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    const int pair = t * top + k;
    const T* a = act + (size_t)pair * ff;
    const T* w = w_down + ((size_t)choice[pair] * dim + n) * ff;
    float s = 0.f;
    if constexpr (sizeof(T) == 2) {
      if (ff % 8 == 0) {
        for (int i = lane * 8; i < ff; i += 256) {
          float af[8], wf[8];
          unpack8(*reinterpret_cast<const Bf16x8*>(a + i), af);
          unpack8(*reinterpret_cast<const Bf16x8*>(w + i), wf);
#pragma unroll
          for (int u = 0; u < 8; ++u) s = fmaf(af[u], wf[u], s);
        }
      } else {
        for (int i = lane; i < ff; i += 32) s = fmaf(to_f32(a[i]), to_f32(w[i]), s);
      }
    } else {
      for (int i = lane; i < ff; i += 32) s = fmaf(to_f32(a[i]), to_f32(w[i]), s);
    }
    total = fmaf(weight[pair], warp_sum(s), total);
  }
  if (lane == 0) x[(size_t)t * dim + n] += total;
}

__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, int top, int dim, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / dim, d = i - t * dim;
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += y[(t * top + k) * dim + d];
    x[i] += s;
  }
}

// xs[r, :] = h[list[r] / top, :]: the tokens' rows in the expert order (16 bytes a lane).
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ list, __nv_bfloat16* __restrict__ xs,
                                  int pairs, int dim, int top) {
  pdl_enter();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= pairs) return;
  const uint4* src = reinterpret_cast<const uint4*>(h + (size_t)(list[r] / top) * dim);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)r * dim);
  for (int i = lane; i < dim / 8; i += 32) dst[i] = src[i];
}

// x[t, :] += sum over the token's choices, in their order, of weight[pair] * y[place[pair], :] (y in the expert order).
__global__ void moe_combine_sorted_kernel(float* __restrict__ x, const float* __restrict__ y, const int* __restrict__ place,
                                          const float* __restrict__ weight, int top, int dim, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / dim, d = i - t * dim;
    float s = 0.f;
    for (int k = 0; k < top; ++k) s = fmaf(weight[t * top + k], y[(size_t)place[t * top + k] * dim + d], s);
    x[i] += s;
  }
}

}  // namespace slb

using namespace slb;

extern "C" int slb_gemm_tc_grouped_gated(const void* X, const void* W, void* C, int M, int N, int K, int groups, int mode,
                                         const int* group_tiles, int max_row_tiles, int kind, float limit, float alpha,
                                         int* status, void* stream);

// The experts of a step of many pairs on the tcgen05 tensor cores (bfloat16, any of the gated activations): the tokens' rows gathered into the
// expert order (xs [pairs, dim]), the grouped product with the gated activation in its epilogue (act [pairs, ff]), the
// grouped down product (y [pairs, dim] float32, expert order, unweighted), and the weighted sum into the stream.
extern "C" int slb_moe_experts_tc(const void* h, const void* w_gu, const void* w_down, const int* list, const int* place,
                                  const float* weight, const int* tiles, void* xs, void* act, float* y, float* x, int tokens,
                                  int dim, int ff, int E, int top, int act_kind, float act_limit, float act_alpha,
                                  int* status, void* stream) {
  SLB_REQUIRE(tokens > 0 && dim > 0 && ff > 0 && E > 0 && top > 0 && dim % 8 == 0 && ff % 8 == 0,
              "moe_experts_tc: tokens=%d dim=%d ff=%d experts=%d top=%d (inner sizes must be multiples of 8)", tokens, dim, ff, E, top);
  SLB_REQUIRE(tiles != nullptr && status != nullptr, "moe_experts_tc: the row tiles and the status word are needed");
  cudaStream_t s = (cudaStream_t)stream;
  const long long pairs = (long long)tokens * top;
  const long long max_tiles = pairs / 128 + (pairs < E ? pairs : E);
  SLB_REQUIRE(pairs < (1LL << 30), "moe_experts_tc: too many pairs (%lld)", pairs);
  launch(moe_gather_kernel, dim3((unsigned)((pairs + 7) / 8)), dim3(256), 0, s, (const __nv_bfloat16*)h, list, (__nv_bfloat16*)xs,
         (int)pairs, dim, top);
  int rc = check_launch("moe_gather");
  if (rc) return rc;
  rc = slb_gemm_tc_grouped_gated(xs, w_gu, act, (int)pairs, ff, dim, E, 3, tiles, (int)max_tiles, act_kind, act_limit, act_alpha,
                                 status, stream);
  if (rc) return rc;
  rc = slb_gemm_tc_grouped_gated(act, w_down, y, (int)pairs, dim, ff, E, 1, tiles, (int)max_tiles, kGateSilu, 0.0f, 1.0f, status,
                                 stream);
  if (rc) return rc;
  const size_t total = (size_t)tokens * dim;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(moe_combine_sorted_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, (const float*)y, place, weight, top, dim, total);
  return check_launch("moe_combine");
}

// choice, place, list: int32 [tokens * top]; weight: float32 [tokens * top]; counts: int32 [E] (written here).
// logits: float32 scratch [tokens, E], or null (then every token's block forms its own logits); with logits_ready they
// hold the logits already (a matrix product formed them) and nothing is computed from h. tiles: int32
// [1 + 3 * (tokens * top / 128 + min(tokens * top, E))] for the grouped tensor-memory product, or null.
extern "C" int slb_moe_route(const void* h, const float* w_router, const float* bias, const float* pick_bias, int* choice, float* weight,
                             int* rank, int* counts, int* place, int* list, float* logits, int* tiles, int layout,
                             int tokens, int dim, int E, int top, int scoring, int groups, int keep, float route_scale,
                             int logits_ready, int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && E > 0 && top > 0 && top <= E, "moe_route: tokens=%d dim=%d experts=%d top=%d",
              tokens, dim, E, top);
  SLB_REQUIRE(E <= 4096, "moe_route: at most 4096 experts, got %d", E);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "moe_route: unknown dtype %d", dtype);
  SLB_REQUIRE(scoring >= 0 && scoring <= 3, "moe_route: unknown scoring %d", scoring);
  SLB_REQUIRE(pick_bias == nullptr || scoring >= 2, "moe_route: a choice correction goes with the softmax scoring over all experts");
  if (groups <= 0) groups = 1;
  if (keep <= 0 || keep > groups) keep = groups;
  SLB_REQUIRE(E % groups == 0, "moe_route: %d experts do not form %d equal groups", E, groups);
  SLB_REQUIRE(scoring == 1 || groups == 1, "moe_route: groups of experts go with the sigmoid scoring");
  SLB_REQUIRE((long long)keep * (E / groups) >= top, "moe_route: %d groups of %d experts cannot give %d choices", keep, E / groups, top);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  (void)rank;      // kept in the signature: callers hand over a table that older versions filled
  const RouteRule rule{scoring, groups, keep, route_scale};
  const size_t smem = (size_t)(E + 2 * groups + (scoring >= 2 ? E : 0)) * sizeof(float);
  const dim3 grid(tokens);
  // from a few tokens on the logits are formed 32 tokens and 16 experts at a time, each weight read once a block
  const float* given = nullptr;
  if (logits_ready) {                             // a product in front of this call has formed the logits
    SLB_REQUIRE(logits != nullptr && bias == nullptr, "moe_route: ready logits must be given, and hold their bias already");
    given = logits;
  } else if (logits != nullptr && tokens < 16) {         // few tokens: a warp per (token, expert)
    const dim3 lg((tokens * E + 7) / 8), lb(256);
    if (dtype == kF32) launch(moe_logits_few_kernel<float>, lg, lb, 0, s, (const float*)h, w_router, bias, logits, tokens, dim, E);
    else launch(moe_logits_few_kernel<__nv_bfloat16>, lg, lb, 0, s, (const __nv_bfloat16*)h, w_router, bias, logits, tokens, dim, E);
    int rc0 = check_launch("moe_logits");
    if (rc0) return rc0;
    given = logits;
  } else if (logits != nullptr) {
    const dim3 lg((tokens + 31) / 32, (E + 15) / 16), lb(256);
    if (dtype == kF32) launch(moe_logits_kernel<float>, lg, lb, 0, s, (const float*)h, w_router, bias, logits, tokens, dim, E);
    else launch(moe_logits_kernel<__nv_bfloat16>, lg, lb, 0, s, (const __nv_bfloat16*)h, w_router, bias, logits, tokens, dim, E);
    int rc0 = check_launch("moe_logits");
    if (rc0) return rc0;
    given = logits;
  }
  // with the logits given only the choosing warp has work: a block of one warp, so that many tokens are resident at once
  const dim3 block(given != nullptr && tokens >= 256 ? 32 : 256);
  if (dtype == kF32)
    launch(moe_route_kernel<float>, grid, block, smem, s, (const float*)h, w_router, bias, pick_bias, given, choice, weight, tokens, dim, E, top, rule);
  else
    launch(moe_route_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)h, w_router, bias, pick_bias, given, choice, weight,
           tokens, dim, E, top, rule);
  int rc = check_launch("moe_route");
  if (rc || !layout) return rc;        // a step of few pairs needs no counts and no expert order
  const int pairs = tokens * top;
  launch(moe_group_kernel, dim3(1), dim3(pairs >= 1024 ? 1024 : 256), 2 * sizeof(int) * E, s, (const int*)choice, counts, place, list,
         pairs, E, tiles, 128);
  return check_launch("moe_group");
}

// act: [tokens * top, ff] in the run dtype; y: float32 [tokens * top, dim]; x: the float32 stream [tokens, dim].
// choice (from slb_moe_route) serves steps of few pairs, which run a warp per output instead of tiles and need neither
// the counts nor the expert-ordered list (`place` is accepted for callers that have it and is not read).
extern "C" int slb_moe_experts(const void* h, const void* w_gu, const void* w_down, const int* counts, const int* list,
                               const int* choice, const int* place, const float* weight, void* act, float* y, float* x,
                               int tokens, int dim, int ff, int E, int top, int act_kind, float act_limit, float act_alpha,
                               int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && ff > 0 && E > 0 && top > 0, "moe_experts: tokens=%d dim=%d ff=%d experts=%d top=%d",
              tokens, dim, ff, E, top);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "moe_experts: unknown dtype %d", dtype);
  SLB_REQUIRE(act_kind >= kGateSilu && act_kind <= kGateLast, "moe_experts: unknown activation %d", act_kind);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const GateAct gate{act_kind, act_limit, act_alpha};
  const long long pairs = (long long)tokens * top;
  // every expert with a pair has at most pairs/tile + 1 tiles more than full ones: an upper bound the host knows
  const long long tiles = pairs / kMoeTile + (pairs < E ? pairs : E);
  SLB_REQUIRE(tiles < (1LL << 31), "moe_experts: too many pairs (%lld)", pairs);
  const dim3 block(256);
  const dim3 g1((unsigned)tiles, (ff + 31) / 32), g2((unsigned)tiles, (dim + kMoeCols - 1) / kMoeCols);
  const bool aligned = ((uintptr_t)h | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)act) % 16 == 0;
  if (pairs <= kMoeFewPairs && choice != nullptr && (dtype == kF32 || aligned)) {
    const dim3 f1((unsigned)pairs, (ff + 7) / 8), f2((unsigned)tokens, (dim + 7) / 8);
    if (dtype == kF32) {
      launch(moe_few_gate_up_kernel<float>, f1, block, 0, s, (const float*)h, (const float*)w_gu, choice, (float*)act, top, dim, ff, gate);
      launch(moe_few_down_kernel<float>, f2, block, 0, s, (const float*)act, (const float*)w_down, choice, weight, x, top, dim, ff);
    } else {
      launch(moe_few_gate_up_kernel<__nv_bfloat16>, f1, block, 0, s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gu, choice,
             (__nv_bfloat16*)act, top, dim, ff, gate);
      launch(moe_few_down_kernel<__nv_bfloat16>, f2, block, 0, s, (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, choice,
             weight, x, top, dim, ff);
    }
    return check_launch("moe_experts");          // the down kernel has added into the stream already
  } else if (dtype == kBF16 && dim % 8 == 0 && ff % 8 == 0 && aligned) {
    const long long tiles64 = pairs / kMmaRows + (pairs < E ? pairs : E);
    launch(moe_mma_kernel<true>, dim3((unsigned)tiles64, (ff + 63) / 64), dim3(128), 0, s, (const __nv_bfloat16*)h,
           (const __nv_bfloat16*)w_gu, counts, list, weight, (__nv_bfloat16*)act, (float*)nullptr, E, top, dim, ff, gate);
    launch(moe_mma_kernel<false>, dim3((unsigned)tiles64, (dim + kMmaCols - 1) / kMmaCols), dim3(128), 0, s,
           (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, counts, list, weight, (__nv_bfloat16*)nullptr, y, E, top, ff,
           dim, gate);
  } else if (dtype == kF32) {
    launch(moe_gate_up_kernel<float>, g1, block, 0, s, (const float*)h, (const float*)w_gu, counts, list, (float*)act, E, top, dim, ff, gate);
    launch(moe_down_kernel<float>, g2, block, 0, s, (const float*)act, (const float*)w_down, counts, list, weight, y, E, dim, ff);
  } else {
    launch(moe_gate_up_kernel<__nv_bfloat16>, g1, block, 0, s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gu, counts, list,
           (__nv_bfloat16*)act, E, top, dim, ff, gate);
    launch(moe_down_kernel<__nv_bfloat16>, g2, block, 0, s, (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, counts, list,
           weight, y, E, dim, ff);
  }
  int rc = check_launch("moe_experts");
  if (rc) return rc;
  const size_t total = (size_t)tokens * dim;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(moe_combine_kernel, dim3((unsigned)blocks), block, 0, s, x, (const float*)y, top, dim, total);
  return check_launch("moe_combine");
}
