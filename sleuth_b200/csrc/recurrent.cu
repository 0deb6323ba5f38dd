// Recurrent mixers: element-wise gated recurrences over a sequence's tokens, with a float32 state per sequence.
//
// minGRU. From the stacked projection's float32 result p[t] = [z' | u' | g'] (three runs of W values at the head of a row
// of `stride` values) and two biases:
//   z = sigmoid(z' + b_z),  u = u' + b_u,  c = u + 1/2 where u >= 0 and sigmoid(u) below,
//   S_t = (1 - z) S_(t-1) + z c,  y[t] = S_t * silu(g')            (all float32, one rounding at the store of y)
// The state S of a sequence lives in state[slot] between steps.
//
//   mingru_step_kernel    a thread per (sequence, channel) walks the sequence's tokens of this step one after another:
//                         single tokens and short portions
//   mingru_fold_kernel    long portions, first pass: a block takes a chunk of kScanChunk tokens and 128 channels and
//                         reduces it to the pair (A, B) with S_end = A S_start + B
//   mingru_starts_kernel  second pass: a block takes 32 channels of a sequence and cuts the chunks' pairs into 32 runs; a
//                         thread per (channel, run) folds its run to one pair, walks the runs before its own from the
//                         sequence's state (pairs compose: (a, b) after (A, B) is (a A, a B + b)), then walks its own
//                         chunks and leaves every chunk's start state in the place of its A
//   mingru_scan_kernel    third pass: a chunk's block walks its own tokens from its start state and stores y; the block
//                         of the last chunk stores the state the step ends with
// The order of operations inside a token is the same in all forms; cutting a sequence into chunks changes the
// rounding of S only. A token's loads do not depend on the state, so every walk fetches kAhead tokens' values before it
// runs their (dependent) updates: the chain of multiply-adds never waits for memory.
#include "common.cuh"

namespace slb {

constexpr int kStepMax = 32;        // the most tokens a sequence may bring for the one-pass form
constexpr int kScanChunk = 16;      // tokens of a chunk of the three-pass form: all of a chunk's values are in flight at once
constexpr int kScanThreads = 128;   // channels of a block
constexpr int kAhead = 8;           // tokens (or pairs) whose values are in flight at once in the walks that may be long
constexpr int kStartRuns = 32;      // runs of chunks that a block of the second pass folds side by side

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }

// The token's decay a = 1 - z and input b = z * c.
__device__ __forceinline__ void mingru_gates(float zr, float ur, float bz, float bu, float& a, float& b) {
  const float z = sigmoid_f32(zr + bz);
  const float u = ur + bu;
  const float c = u >= 0.0f ? u + 0.5f : sigmoid_f32(u);
  a = 1.0f - z;
  b = z * c;
}

// Tokens t0 .. t1 - 1 of channel ch from state S: y[t] = S_t * silu(g_t). Returns the last state.
template <typename TO, int AHEAD>
__device__ __forceinline__ float mingru_walk(const float* __restrict__ p, long long stride, TO* __restrict__ y, int W, int ch,
                                             int t0, int t1, float cz, float cu, float S) {
  for (int t = t0; t < t1; t += AHEAD) {
    float zr[AHEAD], ur[AHEAD], gr[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      if (t + k < t1) {
        const float* row = p + (size_t)(t + k) * stride;
        zr[k] = row[ch];
        ur[k] = row[W + ch];
        gr[k] = row[2 * W + ch];
      }
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      if (t + k < t1) {
        float a, b;
        mingru_gates(zr[k], ur[k], cz, cu, a, b);
        S = fmaf(a, S, b);
        y[(size_t)(t + k) * W + ch] = from_f32<TO>(S * (gr[k] * sigmoid_f32(gr[k])));
      }
    }
  }
  return S;
}

template <typename TO>
__global__ void __launch_bounds__(kScanThreads) mingru_step_kernel(const float* __restrict__ p, long long stride, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ seq_start,
                                                                   TO* __restrict__ y, int W) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int seq = blockIdx.y;
  float* st = state + (size_t)slots[seq] * W + ch;
  *st = mingru_walk<TO, kAhead>(p, stride, y, W, ch, seq_start[seq], seq_start[seq + 1], bz[ch], bu[ch], *st);
}

// pairs: [n_seqs, max_chunks, 2, W].
__global__ void __launch_bounds__(kScanThreads) mingru_fold_kernel(const float* __restrict__ p, long long stride, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, const int* __restrict__ seq_start,
                                                                   float* __restrict__ pairs, int W, int max_chunks) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int chunk = blockIdx.y, seq = blockIdx.z;
  const int t0 = seq_start[seq] + chunk * kScanChunk, t_end = seq_start[seq + 1];
  if (t0 >= t_end) return;
  const int t1 = min(t_end, t0 + kScanChunk);
  const float cz = bz[ch], cu = bu[ch];
  float A = 1.0f, B = 0.0f;
  for (int t = t0; t < t1; t += kScanChunk) {
    float zr[kScanChunk], ur[kScanChunk];
#pragma unroll
    for (int k = 0; k < kScanChunk; ++k) {
      if (t + k < t1) {
        const float* row = p + (size_t)(t + k) * stride;
        zr[k] = row[ch];
        ur[k] = row[W + ch];
      }
    }
#pragma unroll
    for (int k = 0; k < kScanChunk; ++k) {
      if (t + k < t1) {
        float a, b;
        mingru_gates(zr[k], ur[k], cz, cu, a, b);
        A *= a;
        B = fmaf(a, B, b);
      }
    }
  }
  float* out = pairs + (((size_t)seq * max_chunks + chunk) * 2) * W;
  out[ch] = A;
  out[W + ch] = B;
}

// Every chunk's A becomes the state its chunk starts from. Block: 32 channels (x) by kStartRuns runs of chunks (y).
__global__ void __launch_bounds__(32 * kStartRuns) mingru_starts_kernel(const float* __restrict__ state, const int* __restrict__ slots,
                                                                        const int* __restrict__ seq_start, float* __restrict__ pairs,
                                                                        int W, int max_chunks) {
  pdl_enter();
  __shared__ float runA[kStartRuns][33], runB[kStartRuns][33];
  const int ch = blockIdx.x * 32 + threadIdx.x, run = threadIdx.y, seq = blockIdx.y;
  const bool live = ch < W;
  const int chunks = (seq_start[seq + 1] - seq_start[seq] + kScanChunk - 1) / kScanChunk;
  const int per = (chunks + kStartRuns - 1) / kStartRuns;
  const int c0 = min(chunks, run * per), c1 = min(chunks, c0 + per);
  float* pr = pairs + ((size_t)seq * max_chunks * 2) * W + ch;
  float RA = 1.0f, RB = 0.0f;       // this run's chunks as one pair
  if (live) {
    for (int c = c0; c < c1; c += kAhead) {
      float A[kAhead], B[kAhead];
#pragma unroll
      for (int k = 0; k < kAhead; ++k) {
        if (c + k < c1) {
          A[k] = pr[(size_t)(2 * (c + k)) * W];
          B[k] = pr[(size_t)(2 * (c + k) + 1) * W];
        }
      }
#pragma unroll
      for (int k = 0; k < kAhead; ++k) {
        if (c + k < c1) {
          RA *= A[k];
          RB = fmaf(A[k], RB, B[k]);
        }
      }
    }
  }
  runA[run][threadIdx.x] = RA;
  runB[run][threadIdx.x] = RB;
  __syncthreads();
  if (!live || c0 >= c1) return;
  float S = state[(size_t)slots[seq] * W + ch];
  for (int j = 0; j < run; ++j) S = fmaf(runA[j][threadIdx.x], S, runB[j][threadIdx.x]);
  for (int c = c0; c < c1; c += kAhead) {
    float A[kAhead], B[kAhead];
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      if (c + k < c1) {
        A[k] = pr[(size_t)(2 * (c + k)) * W];
        B[k] = pr[(size_t)(2 * (c + k) + 1) * W];
      }
    }
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      if (c + k < c1) {
        pr[(size_t)(2 * (c + k)) * W] = S;
        S = fmaf(A[k], S, B[k]);
      }
    }
  }
}

template <typename TO>
__global__ void __launch_bounds__(kScanThreads) mingru_scan_kernel(const float* __restrict__ p, long long stride, const float* __restrict__ bz,
                                                                   const float* __restrict__ bu, float* __restrict__ state,
                                                                   const int* __restrict__ slots, const int* __restrict__ seq_start,
                                                                   const float* __restrict__ pairs, TO* __restrict__ y, int W,
                                                                   int max_chunks) {
  pdl_enter();
  const int ch = blockIdx.x * kScanThreads + threadIdx.x;
  if (ch >= W) return;
  const int chunk = blockIdx.y, seq = blockIdx.z;
  const int t0 = seq_start[seq] + chunk * kScanChunk, t_end = seq_start[seq + 1];
  if (t0 >= t_end) return;
  const int t1 = min(t_end, t0 + kScanChunk);
  const float S = mingru_walk<TO, kScanChunk>(p, stride, y, W, ch, t0, t1, bz[ch], bu[ch], pairs[(((size_t)seq * max_chunks + chunk) * 2) * W + ch]);
  if (t1 == t_end) state[(size_t)slots[seq] * W + ch] = S;
}

}  // namespace slb

using namespace slb;

// Floats of scratch memory that a step needs (0: the one-pass form serves it).
extern "C" long long slb_mingru_scratch_floats(int n_seqs, int max_count, int W) {
  if (max_count <= kStepMax) return 0;
  const long long chunks = (max_count + kScanChunk - 1) / kScanChunk;
  return (long long)n_seqs * W * 2 * chunks;
}

// p: float32 [T, 3 * W] with row stride `stride` (in floats); bz, bu: float32 [W]; state: float32 [slots, W]; y: [T, W] in `dtype`; scratch: float32, as many
// as slb_mingru_scratch_floats says.
extern "C" int slb_mingru(const float* p, long long stride, const float* bz, const float* bu, float* state, const int* slots,
                          const int* seq_start, void* y, float* scratch, int n_seqs, int max_count, int W, int dtype,
                          void* stream) {
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && W > 0, "mingru: seqs=%d max=%d width=%d", n_seqs, max_count, W);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "mingru: unknown dtype %d", dtype);
  SLB_REQUIRE(stride >= 3LL * W, "mingru: a row stride of %lld for 3 * %d values", stride, W);
  if (n_seqs == 0 || max_count == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int bx = (W + kScanThreads - 1) / kScanThreads;
  if (max_count <= kStepMax) {
    const dim3 grid(bx, n_seqs);
    if (dtype == kF32)
      launch(mingru_step_kernel<float>, grid, dim3(kScanThreads), 0, s, p, stride, bz, bu, state, slots, seq_start, (float*)y, W);
    else
      launch(mingru_step_kernel<__nv_bfloat16>, grid, dim3(kScanThreads), 0, s, p, stride, bz, bu, state, slots, seq_start,
             (__nv_bfloat16*)y, W);
    return check_launch("mingru");
  }
  SLB_REQUIRE(scratch != nullptr, "mingru: a step of %d tokens a sequence needs scratch memory", max_count);
  const int chunks = (max_count + kScanChunk - 1) / kScanChunk;
  SLB_REQUIRE(chunks <= 65535 && n_seqs <= 65535, "mingru: %d chunks of %d sequences", chunks, n_seqs);
  float* pairs = scratch;
  const dim3 grid(bx, chunks, n_seqs);
  launch(mingru_fold_kernel, grid, dim3(kScanThreads), 0, s, p, stride, bz, bu, seq_start, pairs, W, chunks);
  int rc = check_launch("mingru_fold");
  if (rc) return rc;
  launch(mingru_starts_kernel, dim3((W + 31) / 32, n_seqs), dim3(32, kStartRuns), 0, s, (const float*)state, slots, seq_start, pairs, W, chunks);
  rc = check_launch("mingru_starts");
  if (rc) return rc;
  if (dtype == kF32)
    launch(mingru_scan_kernel<float>, grid, dim3(kScanThreads), 0, s, p, stride, bz, bu, state, slots, seq_start, (const float*)pairs,
           (float*)y, W, chunks);
  else
    launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(kScanThreads), 0, s, p, stride, bz, bu, state, slots, seq_start,
           (const float*)pairs, (__nv_bfloat16*)y, W, chunks);
  return check_launch("mingru_scan");
}
