// Mixers that carry a fixed-size state per sequence instead of a growing cache: short causal convolutions over time and
// recurrences with a matrix state and a decay (state-space duality, gated linear attention). All arithmetic is float32;
// the states live in the cache's per-sequence regions [slots, ...] and are indexed by the step's slots.
//
//   causal_conv_kernel      y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c] (+ bias, then silu): inputs before the step's
//                           first token come from the sequence's state (its last taps - 1 inputs), zeros at its start
//   conv_state_kernel       the state after the step: the sequence's last taps - 1 inputs
//   decay_scan_kernel       S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head; a_t one factor per key channel
//                           or one per head; v may carry a factor per (token, head)
//   step_decay_kernel       dt = softplus(raw + bias_h), a = exp(-exp(A_log_h) * dt)   (state-space step sizes and decays)
//   channel_decay_kernel    a = sigmoid(z + bias)^(1 / tau) = exp(-softplus(-(z + bias)) / tau)
//   gated_group_norm_kernel rows cut into equal groups, each divided by its root mean square, times a gain, with a
//                           silu gate in front of or behind the norm and an optional skip term D_h * x
#include <math.h>

#include "common.cuh"

namespace slb {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// One thread per (token, channel). in: [tokens, in_stride] float32, state: [slots, taps - 1, C] (oldest first).
__global__ void __launch_bounds__(256) causal_conv_kernel(const float* __restrict__ in, long long in_stride,
                                                          const float* __restrict__ w, const float* __restrict__ bias,
                                                          const float* __restrict__ state, const int* __restrict__ slots,
                                                          const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                                                          float* __restrict__ out, long long out_stride, int tokens, int C,
                                                          int taps, int act) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * C) return;
  const int t = (int)(i / C), c = (int)(i - (long long)t * C);
  const int seq = tok_seq[t];
  const int at = t - seq_start[seq];                 // index of the token within its sequence's share of the step
  const float* st = state + ((size_t)slots[seq] * (taps - 1)) * C + c;
  float acc = bias ? bias[c] : 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int src = at - (taps - 1) + j;
    const float u = src >= 0 ? in[(size_t)(t - (taps - 1) + j) * in_stride + c] : st[(size_t)(taps - 1 + src) * C];
    acc = fmaf(w[(size_t)c * taps + j], u, acc);
  }
  out[(size_t)t * out_stride + c] = act ? silu_f(acc) : acc;
}

// One thread per (sequence, channel): the last taps - 1 inputs of the sequence, old ones kept where the step was short.
__global__ void __launch_bounds__(256) conv_state_kernel(const float* __restrict__ in, long long in_stride,
                                                         float* __restrict__ state, const int* __restrict__ slots,
                                                         const int* __restrict__ seq_start, int n_seqs, int C, int taps) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_seqs * C) return;
  const int seq = (int)(i / C), c = (int)(i - (long long)seq * C);
  const int first = seq_start[seq], count = seq_start[seq + 1] - first;
  float* st = state + ((size_t)slots[seq] * (taps - 1)) * C + c;
  float keep[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k < taps - 1) {
      const int src = count - (taps - 1) + k;
      keep[k] = src >= 0 ? in[(size_t)(first + src) * in_stride + c] : st[(size_t)(taps - 1 + src) * C];
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k)
    if (k < taps - 1) st[(size_t)k * C] = keep[k];
}

// Steps that bring few tokens a sequence (single tokens above all): one thread per (sequence, channel) walks the
// sequence's tokens with the window of the last taps inputs in registers, writes the outputs and leaves the new tail, in
// one launch. The sums run in the same order as in causal_conv_kernel.
__global__ void __launch_bounds__(128) causal_conv_short_kernel(const float* __restrict__ in, long long in_stride,
                                                                const float* __restrict__ w, const float* __restrict__ bias,
                                                                float* __restrict__ state, const int* __restrict__ slots,
                                                                const int* __restrict__ seq_start, float* __restrict__ out,
                                                                long long out_stride, int n_seqs, int C, int taps, int act) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n_seqs * C) return;
  const int seq = (int)(i / C), c = (int)(i - (long long)seq * C);
  float* st = state + ((size_t)slots[seq] * (taps - 1)) * C + c;
  float win[kMaxTaps], wt[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    win[k] = k < taps - 1 ? st[(size_t)k * C] : 0.0f;          // win[0 .. taps-2]: the tail, oldest first
    wt[k] = k < taps ? w[(size_t)c * taps + k] : 0.0f;
  }
  const float b = bias ? bias[c] : 0.0f;
  for (int t = seq_start[seq]; t < seq_start[seq + 1]; ++t) {
    const float u = in[(size_t)t * in_stride + c];
    float acc = b;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k)
      if (k < taps - 1) acc = fmaf(wt[k], win[k], acc);
    acc = fmaf(wt[taps - 1], u, acc);
    out[(size_t)t * out_stride + c] = act ? silu_f(acc) : acc;
#pragma unroll
    for (int k = 0; k < kMaxTaps - 1; ++k)
      if (k < taps - 2) win[k] = win[k + 1];
    if (taps > 1) win[taps - 2] = u;
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k)
    if (k < taps - 1) st[(size_t)k * C] = win[k];
}

struct ScanArgs {
  const float *q, *k, *v, *a, *vs;     // rows of tokens; vs may be null
  long long q_stride, k_stride, v_stride, a_stride, vs_stride;
  float* state;                        // [slots, heads, N, P]
  const int* slots;
  const int* seq_start;
  float* out;                          // [tokens, heads * P]
  int n_seqs, heads, groups, N, P;
  int a_per_channel;                   // 1: a is [tokens, heads * N]; 0: [tokens, heads]
  float q_scale;
  // Long portions in chunks (chunk_len > 0): every sequence's tokens of the step are cut into `chunks` chunks of chunk_len
  // tokens (the last ones may be short or empty). mode 1 walks each chunk from a zero state and leaves its end state in
  // `starts` [n_seqs, chunks, heads, N, P]; scan_starts_kernel then turns those into the chunks' true start states and
  // updates the sequences' states; mode 2 walks each chunk from its start state and writes the outputs.
  int chunk_len, chunks, mode;
  float* starts;
};

// One thread per (sequence, head, value channel p) keeps column p of the head's state, N values, in registers and walks
// the sequence's tokens of the step. Neighbouring threads hold neighbouring p, so state and value accesses are whole
// lines and the key, query and decay values of a token are the same addresses for a whole warp. A token's loads do not
// depend on the state, so the compiler keeps several tokens' loads in flight. Above 64 rows two neighbouring lanes
// share a column (SPLIT = 2). LOCAL: the pass that walks a chunk from a
// zero state for its end state alone (no queries, no outputs). VEC: rows of keys, queries and decays are read four
// values at a time (N a multiple of 4, rows 16-byte aligned).
template <int NB, bool LOCAL, bool VEC, int SPLIT>
__global__ void __launch_bounds__(128) decay_scan_kernel(ScanArgs a) {
  pdl_enter();
  // SPLIT = 2: two neighbouring lanes share a column of the state, each holds half of its rows (NB of them at most) and
  // the two halves of an output are joined by one shuffle: half the registers a thread, twice the threads
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int pieces = a.mode == 0 ? 1 : a.chunks;
  const long long total = (long long)a.n_seqs * pieces * a.heads * a.P * SPLIT;
  if (i >= total) return;
  const int half = (int)(i % SPLIT);
  const long long col = i / SPLIT;
  const int p = (int)(col % a.P);
  const int h = (int)((col / a.P) % a.heads);
  const int piece = (int)((col / ((long long)a.P * a.heads)) % pieces);
  const int seq = (int)(col / ((long long)a.P * a.heads * pieces));
  const int g = h / (a.heads / a.groups);
  const int N = a.N / SPLIT, n0 = half * N;          // this thread's rows: n0 .. n0 + N - 1
  int t0 = a.seq_start[seq], t1 = a.seq_start[seq + 1];
  float* st = a.state + (((size_t)a.slots[seq] * a.heads + h) * a.N + n0) * a.P + p;
  if (a.mode != 0) {
    t0 += piece * a.chunk_len;
    t1 = min(t1, t0 + a.chunk_len);
    if (t0 >= t1) return;                       // a chunk beyond the sequence's tokens (both lanes of a pair leave)
    st = a.starts + ((((size_t)seq * a.chunks + piece) * a.heads + h) * a.N + n0) * a.P + p;
  }
  float S[NB];
#pragma unroll
  for (int n = 0; n < NB; ++n) S[n] = (n < N && !LOCAL) ? st[(size_t)n * a.P] : 0.0f;
  for (int t = t0; t < t1; ++t) {
    const float* qr = a.q + (size_t)t * a.q_stride + (size_t)g * a.N + n0;
    const float* kr = a.k + (size_t)t * a.k_stride + (size_t)g * a.N + n0;
    const float* ar = a.a + (size_t)t * a.a_stride + (a.a_per_channel ? (size_t)h * a.N + n0 : (size_t)h);
    float v = a.v[(size_t)t * a.v_stride + (size_t)h * a.P + p];
    if (a.vs) v *= a.vs[(size_t)t * a.vs_stride + h];
    const float a_head = a.a_per_channel ? 1.0f : ar[0];
    float o = 0.0f;
    if constexpr (VEC) {
#pragma unroll
      for (int n = 0; n < NB; n += 4) {
        if (n < N) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + n);
          float4 a4 = make_float4(a_head, a_head, a_head, a_head);
          if (a.a_per_channel) a4 = *reinterpret_cast<const float4*>(ar + n);
          S[n] = fmaf(a4.x, S[n], k4.x * v);
          S[n + 1] = fmaf(a4.y, S[n + 1], k4.y * v);
          S[n + 2] = fmaf(a4.z, S[n + 2], k4.z * v);
          S[n + 3] = fmaf(a4.w, S[n + 3], k4.w * v);
          if constexpr (!LOCAL) {
            const float4 q4 = *reinterpret_cast<const float4*>(qr + n);
            o = fmaf(S[n], q4.x, o);
            o = fmaf(S[n + 1], q4.y, o);
            o = fmaf(S[n + 2], q4.z, o);
            o = fmaf(S[n + 3], q4.w, o);
          }
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < NB; ++n) {
        if (n < N) {
          const float an = a.a_per_channel ? ar[n] : a_head;
          S[n] = fmaf(an, S[n], kr[n] * v);
          if constexpr (!LOCAL) o = fmaf(S[n], qr[n], o);
        }
      }
    }
    if constexpr (!LOCAL) {
      // lower rows + upper rows, in both lanes; only the pair takes part (other lanes of the warp may walk other chunks)
      if constexpr (SPLIT == 2) o += __shfl_xor_sync(3u << (threadIdx.x & 30), o, 1);
      if (half == 0) a.out[(size_t)t * ((size_t)a.heads * a.P) + (size_t)h * a.P + p] = o * a.q_scale;
    }
  }
  if (a.mode == 2) return;
#pragma unroll
  for (int n = 0; n < NB; ++n)
    if (n < N) st[(size_t)n * a.P] = S[n];
}

// The product of a chunk's decays: one thread per (sequence, chunk, head, key channel or 0). prod: [n_seqs, chunks, heads, Nn].
__global__ void __launch_bounds__(256) scan_decay_kernel(ScanArgs a, float* __restrict__ prod) {
  pdl_enter();
  const int Nn = a.a_per_channel ? a.N : 1;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)a.n_seqs * a.chunks * a.heads * Nn) return;
  const int n = (int)(i % Nn);
  const int h = (int)((i / Nn) % a.heads);
  const int piece = (int)((i / ((long long)Nn * a.heads)) % a.chunks);
  const int seq = (int)(i / ((long long)Nn * a.heads * a.chunks));
  const int t0 = a.seq_start[seq] + piece * a.chunk_len, t1 = min(a.seq_start[seq + 1], t0 + a.chunk_len);
  float v = 1.0f;
  for (int t = t0; t < t1; ++t) v *= a.a[(size_t)t * a.a_stride + (a.a_per_channel ? (size_t)h * a.N + n : (size_t)h)];
  prod[i] = v;
}

// One thread per (sequence, head, n, p) walks the chunks in order: a chunk's end state (from zero) is replaced by its true
// start state, and the state after the last chunk goes back to the sequence's slot.
__global__ void __launch_bounds__(256) scan_starts_kernel(ScanArgs a, const float* __restrict__ prod) {
  pdl_enter();
  const int Nn = a.a_per_channel ? a.N : 1;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long per_seq = (long long)a.heads * a.N * a.P;
  if (i >= (long long)a.n_seqs * per_seq) return;
  const int seq = (int)(i / per_seq);
  const long long r = i - (long long)seq * per_seq;          // (h, n, p)
  const int h = (int)(r / ((long long)a.N * a.P)), n = (int)((r / a.P) % a.N);
  const int count = a.seq_start[seq + 1] - a.seq_start[seq];
  float* st = a.state + (size_t)a.slots[seq] * per_seq + r;
  float s = *st;
  const int live = min(a.chunks, (count + a.chunk_len - 1) / a.chunk_len);      // chunks that hold tokens
  float* e = a.starts + (size_t)seq * a.chunks * per_seq + r;
  const float* pr = prod + ((size_t)seq * a.chunks * a.heads + h) * Nn + (a.a_per_channel ? n : 0);
  // eight chunks' end states and decay products are asked for before the dependent chain of eight updates runs
  for (int c0 = 0; c0 < live; c0 += 8) {
    float end[8], dec[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = c0 + j < live;
      end[j] = in ? e[(size_t)(c0 + j) * per_seq] : 0.0f;
      dec[j] = in ? pr[(size_t)(c0 + j) * a.heads * Nn] : 1.0f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 + j < live) {
        e[(size_t)(c0 + j) * per_seq] = s;
        s = fmaf(dec[j], s, end[j]);
      }
    }
  }
  *st = s;
}

// raw: [tokens, raw_stride] (the step sizes' pre-activations of head h at raw[t * raw_stride + h]).
__global__ void __launch_bounds__(256) step_decay_kernel(const float* __restrict__ raw, long long raw_stride,
                                                         const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                                         float* __restrict__ dt, float* __restrict__ decay, int tokens,
                                                         int heads) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * heads) return;
  const int t = (int)(i / heads), h = (int)(i - (long long)t * heads);
  const float d = softplus_f(raw[(size_t)t * raw_stride + h] + dt_bias[h]);
  dt[i] = d;
  decay[i] = expf(-expf(a_log[h]) * d);
}

// z: [tokens, C] float32, overwritten by the decays.
__global__ void __launch_bounds__(256) channel_decay_kernel(float* __restrict__ z, const float* __restrict__ bias,
                                                            long long total, int C, float inv_tau) {
  pdl_enter();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = z[i] + (bias ? bias[i % C] : 0.0f);
  z[i] = expf(-softplus_f(-v) * inv_tau);
}

struct GroupNormArgs {
  const float* y;        // [tokens, inner] the recurrence's result
  const float* skip;     // null, or [tokens, skip_stride]: D[h] * skip[t, c] is added first (h = c / head_width)
  long long skip_stride;
  const float* skip_gain;
  int head_width;
  const float* gate;     // [tokens, gate_stride] pre-activations of the silu gate
  long long gate_stride;
  const float* gain;     // [gain_len]; channel c reads gain[c % gain_len]
  int gain_len;
  void* out;             // [tokens, inner] in the run dtype
  int tokens, inner, groups;
  int gate_first;        // 1: (y * silu(gate)) is normalised; 0: the normalised row is multiplied by silu(gate)
  float eps;
};

// One block per (token, group).
template <typename T>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(GroupNormArgs a) {
  pdl_enter();
  __shared__ float scratch[33];
  const int t = blockIdx.x / a.groups, grp = blockIdx.x % a.groups;
  const int width = a.inner / a.groups, c0 = grp * width;
  const float* y = a.y + (size_t)t * a.inner;
  const float* gate = a.gate + (size_t)t * a.gate_stride;
  float ss = 0.0f;
  for (int c = c0 + threadIdx.x; c < c0 + width; c += blockDim.x) {
    float v = y[c];
    if (a.skip) v = fmaf(a.skip_gain[c / a.head_width], a.skip[(size_t)t * a.skip_stride + c], v);
    if (a.gate_first) v *= silu_f(gate[c]);
    ss = fmaf(v, v, ss);
  }
  const float r = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + a.eps);
  T* out = (T*)a.out + (size_t)t * a.inner;
  for (int c = c0 + threadIdx.x; c < c0 + width; c += blockDim.x) {
    float v = y[c];
    if (a.skip) v = fmaf(a.skip_gain[c / a.head_width], a.skip[(size_t)t * a.skip_stride + c], v);
    if (a.gate_first) v *= silu_f(gate[c]);
    v = v * r * a.gain[c % a.gain_len];
    if (!a.gate_first) v *= silu_f(gate[c]);
    out[c] = from_f32<T>(v);
  }
}

}  // namespace slb

using namespace slb;

extern "C" int slb_causal_conv(const float* in, long long in_stride, const float* w, const float* bias, float* state,
                               const int* slots, const int* tok_seq, const int* seq_start, float* out,
                               long long out_stride, int tokens, int n_seqs, int C, int taps, int act, int max_count, void* stream) {
  SLB_REQUIRE(tokens >= 0 && n_seqs >= 0 && C > 0 && taps >= 1 && taps <= kMaxTaps, "causal_conv: tokens=%d channels=%d taps=%d",
              tokens, C, taps);
  SLB_REQUIRE(in_stride >= C && out_stride >= C, "causal_conv: rows are narrower than the channels");
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (max_count >= 1 && max_count <= 4 && taps > 1) {       // few tokens a sequence: outputs and the new tail in one launch
    const long long st = (long long)n_seqs * C;
    launch(causal_conv_short_kernel, dim3((unsigned)((st + 127) / 128)), dim3(128), 0, s, in, in_stride, w, bias, state, slots, seq_start,
           out, out_stride, n_seqs, C, taps, act);
    return check_launch("causal_conv (short steps)");
  }
  const long long total = (long long)tokens * C;
  launch(causal_conv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, in, in_stride, w, bias,
         (const float*)state, slots, tok_seq, seq_start, out, out_stride, tokens, C, taps, act);
  int rc = check_launch("causal_conv");
  if (rc || taps == 1) return rc;
  const long long st = (long long)n_seqs * C;
  launch(conv_state_kernel, dim3((unsigned)((st + 255) / 256)), dim3(256), 0, s, in, in_stride, state, slots, seq_start,
         n_seqs, C, taps);
  return check_launch("conv_state");
}

template <int NB, int SPLIT>
static void launch_scan_nb(const ScanArgs& g, dim3 grid, dim3 block, bool vec, cudaStream_t s) {
  if (g.mode == 1) {
    if (vec) launch(decay_scan_kernel<NB, true, true, SPLIT>, grid, block, 0, s, g);
    else launch(decay_scan_kernel<NB, true, false, SPLIT>, grid, block, 0, s, g);
  } else {
    if (vec) launch(decay_scan_kernel<NB, false, true, SPLIT>, grid, block, 0, s, g);
    else launch(decay_scan_kernel<NB, false, false, SPLIT>, grid, block, 0, s, g);
  }
}

static void launch_scan(const ScanArgs& g, cudaStream_t s) {
  // above 64 rows (an even number of them) two lanes share a column, so a thread holds at most 128 rows; measured on a
  // B200 with 2,048-token prompts: 128 rows 806 + 470 us a layer with one lane a column, 494 + 290 us with two; 64 rows
  // 128 + 90 us with one lane, 144 + 101 us with two
  const int split = (g.N > 64 && g.N % 2 == 0) ? 2 : 1;
  const int rows = g.N / split;
  const long long total = (long long)g.n_seqs * (g.mode == 0 ? 1 : g.chunks) * g.heads * g.P * split;
  const dim3 grid((unsigned)((total + 127) / 128)), block(128);
  // four values a load where every row of keys, queries and decays starts on a 16-byte boundary (the sum's order is the same)
  const bool vec = rows % 4 == 0 && g.N % 4 == 0 && g.q_stride % 4 == 0 && g.k_stride % 4 == 0 && ((uintptr_t)g.q % 16 == 0) &&
                   ((uintptr_t)g.k % 16 == 0) && (!g.a_per_channel || (g.a_stride % 4 == 0 && (uintptr_t)g.a % 16 == 0));
  if (split == 1) {                      // up to 64 rows, or an odd number of them (at most 255 then)
    if (rows <= 16) launch_scan_nb<16, 1>(g, grid, block, vec, s);
    else if (rows <= 32) launch_scan_nb<32, 1>(g, grid, block, vec, s);
    else if (rows <= 64) launch_scan_nb<64, 1>(g, grid, block, vec, s);
    else if (rows <= 128) launch_scan_nb<128, 1>(g, grid, block, vec, s);
    else if (g.mode == 1) launch(decay_scan_kernel<256, true, false, 1>, grid, block, 0, s, g);      // (registers spill here)
    else launch(decay_scan_kernel<256, false, false, 1>, grid, block, 0, s, g);
  } else {
    if (rows <= 64) launch_scan_nb<64, 2>(g, grid, block, vec, s);          // 33 to 64 rows a lane
    else launch_scan_nb<128, 2>(g, grid, block, vec, s);
  }
}

// Portions of more than kScanWhole tokens run in chunks (three passes); the chunk length grows with the portion so that
// the middle pass, which walks the chunks one after another, stays short.
constexpr int kScanWhole = 48;
static int scan_chunk_len(int max_count) { return max_count <= 4096 ? 32 : 128; }

// Floats of scratch memory that a step whose longest portion has max_count tokens needs (0: it runs in one pass).
extern "C" long long slb_decay_scan_scratch_floats(int n_seqs, int max_count, int heads, int N, int P, int a_per_channel) {
  if (max_count <= kScanWhole) return 0;
  const long long chunks = (max_count + scan_chunk_len(max_count) - 1) / scan_chunk_len(max_count);
  return (long long)n_seqs * chunks * heads * ((long long)N * P + (a_per_channel ? N : 1));
}

extern "C" int slb_decay_scan(const float* q, long long q_stride, const float* k, long long k_stride, const float* v,
                              long long v_stride, const float* a, long long a_stride, int a_per_channel, const float* vs,
                              long long vs_stride, float* state, const int* slots, const int* seq_start, float* out,
                              int n_seqs, int heads, int groups, int N, int P, float q_scale, int max_count, float* scratch,
                              long long scratch_floats, void* stream) {
  SLB_REQUIRE(n_seqs >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && N > 0 && N <= 256 && P > 0,
              "decay_scan: heads=%d groups=%d state rows=%d (at most 256) columns=%d", heads, groups, N, P);
  if (n_seqs == 0) return 0;
  ScanArgs g{q, k, v, a, vs, q_stride, k_stride, v_stride, a_stride, vs_stride, state, slots, seq_start, out,
             n_seqs, heads, groups, N, P, a_per_channel, q_scale, 0, 1, 0, nullptr};
  cudaStream_t s = (cudaStream_t)stream;
  const long long need = slb_decay_scan_scratch_floats(n_seqs, max_count, heads, N, P, a_per_channel);
  if (need == 0) {
    launch_scan(g, s);
    return check_launch("decay_scan");
  }
  SLB_REQUIRE(scratch != nullptr && scratch_floats >= need, "decay_scan: %lld floats of scratch memory are needed, %lld were given",
              need, scratch_floats);
  g.chunk_len = scan_chunk_len(max_count);
  g.chunks = (max_count + g.chunk_len - 1) / g.chunk_len;
  g.starts = scratch;
  float* prod = scratch + (size_t)n_seqs * g.chunks * heads * N * P;
  g.mode = 1;
  launch_scan(g, s);
  int rc = check_launch("decay_scan (chunks from zero)");
  if (rc) return rc;
  const long long np = (long long)n_seqs * g.chunks * heads * (a_per_channel ? N : 1);
  launch(scan_decay_kernel, dim3((unsigned)((np + 255) / 256)), dim3(256), 0, s, g, prod);
  rc = check_launch("decay_scan (decay products)");
  if (rc) return rc;
  const long long ns = (long long)n_seqs * heads * N * P;
  launch(scan_starts_kernel, dim3((unsigned)((ns + 255) / 256)), dim3(256), 0, s, g, (const float*)prod);
  rc = check_launch("decay_scan (chunk starts)");
  if (rc) return rc;
  g.mode = 2;
  launch_scan(g, s);
  return check_launch("decay_scan (chunks from their starts)");
}

extern "C" int slb_step_decay(const float* raw, long long raw_stride, const float* dt_bias, const float* a_log, float* dt,
                              float* decay, int tokens, int heads, void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && raw_stride >= heads, "step_decay: tokens=%d heads=%d", tokens, heads);
  if (tokens == 0) return 0;
  const long long total = (long long)tokens * heads;
  launch(step_decay_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, raw, raw_stride,
         dt_bias, a_log, dt, decay, tokens, heads);
  return check_launch("step_decay");
}

extern "C" int slb_channel_decay(float* z, const float* bias, int tokens, int C, float tau, void* stream) {
  SLB_REQUIRE(tokens >= 0 && C > 0 && tau > 0.0f, "channel_decay: tokens=%d channels=%d tau=%g", tokens, C, (double)tau);
  if (tokens == 0) return 0;
  const long long total = (long long)tokens * C;
  launch(channel_decay_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, z, bias, total, C,
         1.0f / tau);
  return check_launch("channel_decay");
}

extern "C" int slb_gated_group_norm(const float* y, const float* skip, long long skip_stride, const float* skip_gain,
                                    int head_width, const float* gate, long long gate_stride, const float* gain,
                                    int gain_len, void* out, int tokens, int inner, int groups, int gate_first, float eps,
                                    int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && inner > 0 && groups > 0 && inner % groups == 0 && gain_len > 0 && head_width > 0,
              "gated_group_norm: inner=%d groups=%d gain=%d", inner, groups, gain_len);
  SLB_REQUIRE(gate != nullptr && gate_stride >= inner && (skip == nullptr || (skip_gain != nullptr && skip_stride >= inner)),
              "gated_group_norm: gate or skip rows");
  if (tokens == 0) return 0;
  GroupNormArgs a{y, skip, skip_stride, skip_gain, head_width, gate, gate_stride, gain, gain_len, out, tokens, inner, groups,
                  gate_first, eps};
  const dim3 grid((unsigned)(tokens * groups)), block(128);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch(gated_group_norm_kernel<float>, grid, block, 0, s, a);
  else if (dtype == kBF16) launch(gated_group_norm_kernel<__nv_bfloat16>, grid, block, 0, s, a);
  else return fail(1, "gated_group_norm: unknown dtype %d", dtype);
  return check_launch("gated_group_norm");
}
