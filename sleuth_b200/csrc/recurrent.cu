// Recurrent mixers: element-wise gated recurrences over a sequence's tokens, with a float32 state per sequence.
//
// minGRU. From the stacked projection's float32 result p[t] = [z' | u' | g'] (three runs of W values) and two biases:
//   z = sigmoid(z' + b_z),  u = u' + b_u,  c = u + 1/2 where u >= 0 and sigmoid(u) below,
//   S_t = (1 - z) S_(t-1) + z c,  y[t] = S_t * silu(g')            (all float32, one rounding at the store of y)
// The state S of a sequence lives in state[slot] between steps.
//
//   mingru_step_kernel    a thread per (sequence, channel) walks the sequence's tokens of this step one after another:
//                         single tokens and short portions
//   mingru_fold_kernel    long portions, first pass: a block takes a chunk of kScanChunk tokens and 128 channels and
//                         reduces it to the pair (A, B) with S_end = A S_start + B; chunk 0 also copies the state the
//                         step starts from
//   mingru_scan_kernel    second pass: a chunk's block finds its start state by walking the pairs of the chunks before
//                         it (at most a few dozen multiply-adds), then walks its own tokens and stores y; the block of
//                         the last chunk stores the state the step ends with
// The order of operations inside a token is the same in both forms; cutting a sequence into chunks changes the
// rounding of S only.
#include "common.cuh"

namespace slb {

constexpr int kScanChunk = 64;      // tokens of a chunk of the two-pass form
constexpr int kScanThreads = 128;   // channels of a block

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }

// The token's decay a = 1 - z and input b = z * c.
__device__ __forceinline__ void mingru_gates(float zr, float ur, float bz, float bu, float& a, float& b) {
  const float z = sigmoid_f32(zr + bz);
  const float u = ur + bu;
  const float c = u >= 0.0f ? u + 0.5f : sigmoid_f32(u);
  a = 1.0f - z;
  b = z * c;
}

template <typename TO>
__global__ void __launch_bounds__(kScanThreads) mingru_step_kernel(const float* __restrict__ p, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ seq_start,
                                                                   TO* __restrict__ y, int W) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int seq = blockIdx.y;
  const int t0 = seq_start[seq], t1 = seq_start[seq + 1];
  float* st = state + (size_t)slots[seq] * W + ch;
  float S = *st;
  const float cz = bz[ch], cu = bu[ch];
  for (int t = t0; t < t1; ++t) {
    const float* row = p + (size_t)t * 3 * W;
    float a, b;
    mingru_gates(row[ch], row[W + ch], cz, cu, a, b);
    S = fmaf(a, S, b);
    const float g = row[2 * W + ch];
    y[(size_t)t * W + ch] = from_f32<TO>(S * (g * sigmoid_f32(g)));
  }
  *st = S;
}

// pairs: [n_seqs, max_chunks, 2, W]; start: [n_seqs, W] (the state each sequence's step starts from).
__global__ void __launch_bounds__(kScanThreads) mingru_fold_kernel(const float* __restrict__ p, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, const float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ seq_start,
                                                                   float* __restrict__ pairs, float* __restrict__ start, int W,
                                                                   int max_chunks) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int chunk = blockIdx.y, seq = blockIdx.z;
  const int t0 = seq_start[seq] + chunk * kScanChunk, t_end = seq_start[seq + 1];
  if (t0 >= t_end) return;
  const int t1 = min(t_end, t0 + kScanChunk);
  if (chunk == 0) start[(size_t)seq * W + ch] = state[(size_t)slots[seq] * W + ch];
  const float cz = bz[ch], cu = bu[ch];
  float A = 1.0f, B = 0.0f;
  for (int t = t0; t < t1; ++t) {
    const float* row = p + (size_t)t * 3 * W;
    float a, b;
    mingru_gates(row[ch], row[W + ch], cz, cu, a, b);
    A *= a;
    B = fmaf(a, B, b);
  }
  float* out = pairs + (((size_t)seq * max_chunks + chunk) * 2) * W;
  out[ch] = A;
  out[W + ch] = B;
}

template <typename TO>
__global__ void __launch_bounds__(kScanThreads) mingru_scan_kernel(const float* __restrict__ p, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ seq_start,
                                                                   const float* __restrict__ pairs, const float* __restrict__ start,
                                                                   TO* __restrict__ y, int W, int max_chunks) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int chunk = blockIdx.y, seq = blockIdx.z;
  const int t0 = seq_start[seq] + chunk * kScanChunk, t_end = seq_start[seq + 1];
  if (t0 >= t_end) return;
  const int t1 = min(t_end, t0 + kScanChunk);
  float S = start[(size_t)seq * W + ch];
  const float* pr = pairs + ((size_t)seq * max_chunks * 2) * W;
  for (int c = 0; c < chunk; ++c) S = fmaf(pr[(size_t)(2 * c) * W + ch], S, pr[(size_t)(2 * c + 1) * W + ch]);
  const float cz = bz[ch], cu = bu[ch];
  for (int t = t0; t < t1; ++t) {
    const float* row = p + (size_t)t * 3 * W;
    float a, b;
    mingru_gates(row[ch], row[W + ch], cz, cu, a, b);
    S = fmaf(a, S, b);
    const float g = row[2 * W + ch];
    y[(size_t)t * W + ch] = from_f32<TO>(S * (g * sigmoid_f32(g)));
  }
  if (t1 == t_end) state[(size_t)slots[seq] * W + ch] = S;
}

}  // namespace slb

using namespace slb;

// Floats of scratch memory that a step needs (0: the one-pass form serves it).
extern "C" long long slb_mingru_scratch_floats(int n_seqs, int max_count, int W) {
  if (max_count <= kScanChunk) return 0;
  const long long chunks = (max_count + kScanChunk - 1) / kScanChunk;
  return (long long)n_seqs * W * (2 * chunks + 1);
}

// p: float32 [T, 3 * W]; bz, bu: float32 [W]; state: float32 [slots, W]; y: [T, W] in `dtype`; scratch: float32, as many
// as slb_mingru_scratch_floats says.
extern "C" int slb_mingru(const float* p, const float* bz, const float* bu, float* state, const int* slots,
                          const int* seq_start, void* y, float* scratch, int n_seqs, int max_count, int W, int dtype,
                          void* stream) {
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && W > 0, "mingru: seqs=%d max=%d width=%d", n_seqs, max_count, W);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "mingru: unknown dtype %d", dtype);
  if (n_seqs == 0 || max_count == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int bx = (W + kScanThreads - 1) / kScanThreads;
  if (max_count <= kScanChunk) {
    const dim3 grid(bx, n_seqs);
    if (dtype == kF32)
      launch(mingru_step_kernel<float>, grid, dim3(kScanThreads), 0, s, p, bz, bu, state, slots, seq_start, (float*)y, W);
    else
      launch(mingru_step_kernel<__nv_bfloat16>, grid, dim3(kScanThreads), 0, s, p, bz, bu, state, slots, seq_start,
             (__nv_bfloat16*)y, W);
    return check_launch("mingru");
  }
  SLB_REQUIRE(scratch != nullptr, "mingru: a step of %d tokens a sequence needs scratch memory", max_count);
  const int chunks = (max_count + kScanChunk - 1) / kScanChunk;
  SLB_REQUIRE(chunks <= 65535 && n_seqs <= 65535, "mingru: %d chunks of %d sequences", chunks, n_seqs);
  float* pairs = scratch;
  float* start = scratch + (size_t)n_seqs * chunks * 2 * W;
  const dim3 grid(bx, chunks, n_seqs);
  launch(mingru_fold_kernel, grid, dim3(kScanThreads), 0, s, p, bz, bu, (const float*)state, slots, seq_start, pairs, start, W,
         chunks);
  int rc = check_launch("mingru_fold");
  if (rc) return rc;
  if (dtype == kF32)
    launch(mingru_scan_kernel<float>, grid, dim3(kScanThreads), 0, s, p, bz, bu, state, slots, seq_start, (const float*)pairs,
           (const float*)start, (float*)y, W, chunks);
  else
    launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(kScanThreads), 0, s, p, bz, bu, state, slots, seq_start,
           (const float*)pairs, (const float*)start, (__nv_bfloat16*)y, W, chunks);
  return check_launch("mingru_scan");
}
