// Attention through low-rank latents over a paged latent cache.
//
// A token's cache row holds W = R + P values: its normed latent c (R values) and one rotated key part (P values)
// that all heads share. With the key up-projection moved onto the query (q_lat[h] = W_uk[h]^T q_plain[h]) the score
// of head h is (q_lat[h] . c + q_rot[h] . k_rot) * scale, and the value up-projection can wait until after the
// weighted sum: o_lat[h] = sum_j p_j c_j, value[h] = W_uv[h] o_lat[h]. So every head reads the same rows, as keys
// (all W values) and as values (the first R).
//
// Kernels here:
//   latent_post_kernel    the down-projections' float32 output -> normed query latent, normed latent and rotated key
//                         part into the cache (norms and rotation in float32, one rounding at the store)
//   latent_attn_kernel    causal softmax attention of all heads of a tile of tokens over the cache rows, float32
//                         arithmetic; the rotation of the query's rotated part happens as the queries are loaded;
//                         a long sequence's keys may be cut into slices whose partial results latent_merge_kernel joins
//   latent_attn_mma_kernel  the same on the warp-level tensor cores (bfloat16, widths that are multiples of 16)
//   head_prompt_mma_kernel  whole prompts (every sequence starts at 0): per-head keys and values formed from the step's
//                         latents by one product, then ordinary causal attention per head on the tensor cores
//   latent_gate_kernel    y[t, h, :] = value[h, t, :] * sigmoid(g[t, h, :])
#include "mma_sync.cuh"

namespace slb {

constexpr int kLatRows = 32;      // (token, head) rows of a block of the general kernel
constexpr size_t kLatMaxSmem = 227 * 1024;      // dynamic shared memory a block may ask for
constexpr int kLatWarps = 8;
constexpr int kLatRowsPerWarp = kLatRows / kLatWarps;

// One block per token. lat[t] = [q_rank | R | P | anything] float32, rows `lat_stride` values apart; q_rank may be 0 (the
// queries do not pass through a latent: nothing is written to cq).
template <typename TO>
__global__ void latent_post_kernel(const float* __restrict__ lat, const float* __restrict__ q_gain,
                                   const float* __restrict__ c_gain, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, TO* __restrict__ cq, TO* __restrict__ pool,
                                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                   const int* __restrict__ table, int stride, int q_rank, int R, int P, int rot,
                                   float eps, TO* __restrict__ c_out, TO* __restrict__ k_out, int lat_stride) {
  pdl_enter();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* row = lat + (size_t)t * lat_stride;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
  for (int i = threadIdx.x; i < R; i += blockDim.x) sc = fmaf(row[q_rank + i], row[q_rank + i], sc);
  if (q_rank > 0) sq = block_sum(sq, scratch);
  sc = block_sum(sc, scratch);
  const float inv_q = q_rank > 0 ? 1.0f / sqrtf(sq / (float)q_rank + eps) : 0.0f;
  const float inv_c = 1.0f / sqrtf(sc / (float)R + eps);
  TO* qo = cq + (size_t)t * q_rank;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) qo[i] = from_f32<TO>((row[i] * inv_q) * q_gain[i]);
  if (pool == nullptr && c_out == nullptr) return;
  const int pos = tok_pos[t];
  TO* dst = nullptr;
  if (pool != nullptr) {
    const int page = table[(size_t)tok_seq[t] * stride + pos / kPageTokens];
    dst = pool + ((size_t)page * kPageTokens + pos % kPageTokens) * (R + P);
  }
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const TO v = from_f32<TO>((row[q_rank + i] * inv_c) * c_gain[i]);
    if (dst) dst[i] = v;
    if (c_out) c_out[(size_t)t * R + i] = v;      // the same values side by side, for products over the step's own tokens
  }
  const float* kr = row + q_rank + R;
  const int half = rot / 2;
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    float v = kr[i];
    if (i < rot) {
      const int f = i < half ? i : i - half;
      const float c = cos_t[(size_t)pos * half + f], s = sin_t[(size_t)pos * half + f];
      v = i < half ? kr[i] * c - kr[i + half] * s : kr[i] * c + kr[i - half] * s;
    }
    if (dst) dst[R + i] = from_f32<TO>(v);
    if (k_out) k_out[(size_t)t * P + i] = from_f32<TO>(v);
  }
}

struct LatentAttnArgs {
  const void* q_lat;      // [H, T, R]
  const void* q_raw;      // [T, H, dn + P]; the rotated part starts at dn
  const void* pool;       // [pages, 64, R + P]
  void* out;              // [H, T, R]
  float* parts;           // splits > 1: [splits, T * H, R + 2] (sum, then running maximum and mass)
  const float* cos_t;
  const float* sin_t;
  const int* seq_start;
  const int* past;
  const int* counts;
  const int* table;
  int stride, T, H, R, P, dn, rot, window, splits, chunk, tq, hb, kstride;
  float scale;
};

// Block (x: tile of tq tokens, y: sequence, z: head chunk * splits + slice), 8 warps, 4 (token, head) rows a warp.
// The keys are walked in chunks of `chunk` (16, 32 or 64) rows staged in shared memory as float32 with an odd row
// stride; a lane takes a key (two with 64), then a value column (RV of them).
template <typename T, int RV>
__global__ void __launch_bounds__(kLatWarps * 32) latent_attn_kernel(const LatentAttnArgs a) {
  pdl_enter();
  extern __shared__ float smem[];
  const int W = a.R + a.P;
  float* Qs = smem;                                   // [32][W]
  float* Ks = Qs + (size_t)kLatRows * W;              // [chunk][kstride]
  float* Ps = Ks + (size_t)a.chunk * a.kstride;       // [warps][64][4]
  const int seq = blockIdx.y;
  const int slice = blockIdx.z % a.splits, hc = blockIdx.z / a.splits;
  const int count = a.counts[seq], past = a.past[seq];
  const int t0 = blockIdx.x * a.tq;
  if (t0 >= count) return;
  const int nt = min(a.tq, count - t0);
  const int h0 = hc * a.hb, nh = min(a.hb, a.H - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q_lat = (const T*)a.q_lat;
  const T* q_raw = (const T*)a.q_raw;
  const T* pool = (const T*)a.pool;
  const int tok0 = a.seq_start[seq] + t0;             // first token row of the tile

  // queries: latent part as it is, rotated part turned by the token's angle
  const int half = a.rot / 2;
  for (int r = warp; r < kLatRows; r += kLatWarps) {
    const int tq = r / a.hb, hh = r % a.hb;
    const bool live = tq < nt && hh < nh;
    float* qs = Qs + (size_t)r * W;
    if (!live) {
      for (int i = lane; i < W; i += 32) qs[i] = 0.f;
      continue;
    }
    const int tok = tok0 + tq, h = h0 + hh, pos = past + t0 + tq;
    const T* ql = q_lat + ((size_t)h * a.T + tok) * a.R;
    for (int i = lane; i < a.R; i += 32) qs[i] = to_f32(ql[i]);
    const T* qr = q_raw + ((size_t)tok * a.H + h) * (a.dn + a.P) + a.dn;
    for (int i = lane; i < a.P; i += 32) {
      float v = to_f32(qr[i]);
      if (i < a.rot) {
        const int f = i < half ? i : i - half;
        const float c = a.cos_t[(size_t)pos * half + f], s = a.sin_t[(size_t)pos * half + f];
        v = i < half ? v * c - to_f32(qr[i + half]) * s : v * c + to_f32(qr[i - half]) * s;
      }
      qs[a.R + i] = v;
    }
  }

  // the keys this block walks
  const int last_pos = past + t0 + nt - 1;
  int key_lo = a.window > 0 ? max(0, past + t0 - a.window + 1) : 0;
  key_lo = key_lo / a.chunk * a.chunk;
  const int n_chunks = (last_pos - key_lo) / a.chunk + 1;
  const int per = (n_chunks + a.splits - 1) / a.splits;
  const int c_lo = slice * per, c_hi = min(n_chunks, c_lo + per);

  float acc[kLatRowsPerWarp][RV];
  float m[kLatRowsPerWarp], l[kLatRowsPerWarp];
  int row_pos[kLatRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kLatRowsPerWarp; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
    const int row = warp * kLatRowsPerWarp + r;
    const int tq = row / a.hb, hh = row % a.hb;
    row_pos[r] = (tq < nt && hh < nh) ? past + t0 + tq : -1;
#pragma unroll
    for (int i = 0; i < RV; ++i) acc[r][i] = 0.f;
  }
  const int* trow = a.table + (size_t)seq * a.stride;
  const float* qw = Qs + (size_t)warp * kLatRowsPerWarp * W;
  float* pw = Ps + (size_t)warp * 64 * kLatRowsPerWarp;
  const int keys_per_lane = a.chunk > 32 ? 2 : 1;

  for (int c = c_lo; c < c_hi; ++c) {
    const int k0 = key_lo + c * a.chunk;
    const int nk = min(a.chunk, last_pos - k0 + 1);
    __syncthreads();
    // stage the chunk: rows k0 .. k0 + nk - 1 of one page (a chunk never straddles pages: 64 is a multiple of it)
    {
      const int page = trow[k0 / kPageTokens];
      const T* src = pool + ((size_t)page * kPageTokens + k0 % kPageTokens) * W;
      const int total = nk * W;
      for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int j = i / W, d = i - j * W;
        Ks[(size_t)j * a.kstride + d] = to_f32(src[i]);
      }
      for (int i = threadIdx.x + total; i < a.chunk * W; i += blockDim.x) {
        const int j = i / W, d = i - j * W;
        Ks[(size_t)j * a.kstride + d] = 0.f;
      }
    }
    __syncthreads();

    // scores: lane = key (and key + 32)
    float s[kLatRowsPerWarp][2];
#pragma unroll
    for (int r = 0; r < kLatRowsPerWarp; ++r) s[r][0] = s[r][1] = 0.f;
    const int ja = min(lane, a.chunk - 1);
    const float* ka = Ks + (size_t)ja * a.kstride;
    const float* kb = Ks + (size_t)min(lane + 32, a.chunk - 1) * a.kstride;
    if (keys_per_lane == 2) {
      for (int d = 0; d < W; ++d) {
        const float x0 = ka[d], x1 = kb[d];
#pragma unroll
        for (int r = 0; r < kLatRowsPerWarp; ++r) {
          const float qv = qw[(size_t)r * W + d];
          s[r][0] = fmaf(qv, x0, s[r][0]);
          s[r][1] = fmaf(qv, x1, s[r][1]);
        }
      }
    } else {
      for (int d = 0; d < W; ++d) {
        const float x0 = ka[d];
#pragma unroll
        for (int r = 0; r < kLatRowsPerWarp; ++r) s[r][0] = fmaf(qw[(size_t)r * W + d], x0, s[r][0]);
      }
    }
    // softmax bookkeeping per row, probabilities to shared memory as [key][row]
    float alpha[kLatRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kLatRowsPerWarp; ++r) {
      float mx = -INFINITY;
      float sv[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = lane + 32 * u;
        const int kpos = k0 + j;
        const bool seen = u < keys_per_lane && j < nk && row_pos[r] >= 0 && kpos <= row_pos[r] &&
                          (a.window <= 0 || kpos > row_pos[r] - a.window);
        sv[u] = seen ? s[r][u] * a.scale : -INFINITY;
        mx = fmaxf(mx, sv[u]);
      }
      mx = warp_max(mx);
      const float m_new = fmaxf(m[r], mx);
      float psum = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float p = (m_new == -INFINITY || sv[u] == -INFINITY) ? 0.f : expf(sv[u] - m_new);
        psum += p;
        if (u < keys_per_lane) pw[(size_t)(lane + 32 * u) * kLatRowsPerWarp + r] = p;
      }
      psum = warp_sum(psum);
      alpha[r] = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
      if (m_new == -INFINITY) alpha[r] = 1.f;
      l[r] = l[r] * alpha[r] + psum;
      m[r] = m_new;
    }
    __syncwarp();
    // weighted sum of the latents: lane = value column
#pragma unroll
    for (int r = 0; r < kLatRowsPerWarp; ++r)
#pragma unroll
      for (int i = 0; i < RV; ++i) acc[r][i] *= alpha[r];
    for (int j = 0; j < nk; ++j) {
      const float4 p4 = *reinterpret_cast<const float4*>(pw + (size_t)j * kLatRowsPerWarp);
      const float pr[4] = {p4.x, p4.y, p4.z, p4.w};
      const float* kv = Ks + (size_t)j * a.kstride;
#pragma unroll
      for (int i = 0; i < RV; ++i) {
        const int d = lane + 32 * i;
        const float v = d < a.R ? kv[d] : 0.f;
#pragma unroll
        for (int r = 0; r < kLatRowsPerWarp; ++r) acc[r][i] = fmaf(pr[r], v, acc[r][i]);
      }
    }
    __syncwarp();
  }

  // results
#pragma unroll
  for (int r = 0; r < kLatRowsPerWarp; ++r) {
    if (row_pos[r] < 0) continue;
    const int row = warp * kLatRowsPerWarp + r;
    const int tok = tok0 + row / a.hb, h = h0 + row % a.hb;
    if (a.splits == 1) {
      const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
      T* o = (T*)a.out + ((size_t)h * a.T + tok) * a.R;
#pragma unroll
      for (int i = 0; i < RV; ++i) {
        const int d = lane + 32 * i;
        if (d < a.R) o[d] = from_f32<T>(acc[r][i] * inv);
      }
    } else {
      float* o = a.parts + ((size_t)slice * a.T * a.H + (size_t)tok * a.H + h) * (a.R + 2);
#pragma unroll
      for (int i = 0; i < RV; ++i) {
        const int d = lane + 32 * i;
        if (d < a.R) o[d] = acc[r][i];
      }
      if (lane == 0) {
        o[a.R] = m[r];
        o[a.R + 1] = l[r];
      }
    }
  }
}

// The same attention on the warp-level tensor cores, for bfloat16 and widths that are multiples of 16.
// Block: 64 (token, head) rows on four warps, 16 rows a warp, so that a row's softmax stays inside its warp. Queries
// (latent part and rotated part, turned as they are loaded) and one chunk of 64 cache rows lie in shared memory as
// bfloat16 with rows padded by 16 bytes, which keeps ldmatrix free of bank conflicts. Scores = Q K^T over all W
// columns (mma.sync m16n8k16, float32 sums), online softmax in registers, then P times the chunk's first columns, read
// from the same shared rows through transposing loads. A block takes at most NTM * 16 value columns (its sums live in
// registers); a wider latent is shared by several blocks (grid z), each of which forms the scores again.
template <int NTM>
__global__ void __launch_bounds__(128) latent_attn_mma_kernel(const LatentAttnArgs a, int nt16, int groups, int buffers) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char lat_raw[];
  const int W = a.R + a.P, ks = a.kstride;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lat_raw);     // [64][ks]
  __nv_bfloat16* Ks = Qs + 64 * ks;                                  // [64][ks]
  const int seq = blockIdx.y;
  int z = blockIdx.z;
  const int slice = z % a.splits;
  z /= a.splits;
  const int grp = z % groups, hc = z / groups;
  const int count = a.counts[seq], past = a.past[seq];
  const int t0 = blockIdx.x * a.tq;
  if (t0 >= count) return;
  const int nt = min(a.tq, count - t0);
  const int h0 = hc * a.hb, nh = min(a.hb, a.H - h0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const __nv_bfloat16* q_lat = (const __nv_bfloat16*)a.q_lat;
  const __nv_bfloat16* q_raw = (const __nv_bfloat16*)a.q_raw;
  const __nv_bfloat16* pool = (const __nv_bfloat16*)a.pool;
  const int tok0 = a.seq_start[seq] + t0;
  const int half = a.rot / 2;
  // queries: a warp takes every fourth row; dead rows become zeros
  for (int r = warp; r < 64; r += 4) {
    const int tq = r / a.hb, hh = r % a.hb;
    __nv_bfloat16* qs = Qs + (size_t)r * ks;
    if (!(tq < nt && hh < nh)) {
      for (int i = lane * 8; i < W; i += 256) *reinterpret_cast<uint4*>(qs + i) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int tok = tok0 + tq, h = h0 + hh, pos = past + t0 + tq;
    const __nv_bfloat16* ql = q_lat + ((size_t)h * a.T + tok) * a.R;
    for (int i = lane * 8; i < a.R; i += 256) *reinterpret_cast<uint4*>(qs + i) = *reinterpret_cast<const uint4*>(ql + i);
    const __nv_bfloat16* qr = q_raw + ((size_t)tok * a.H + h) * (a.dn + a.P) + a.dn;
    for (int i = lane; i < a.P; i += 32) {
      float v = __bfloat162float(qr[i]);
      if (i < a.rot) {
        const int f = i < half ? i : i - half;
        const float c = a.cos_t[(size_t)pos * half + f], sn = a.sin_t[(size_t)pos * half + f];
        v = i < half ? v * c - __bfloat162float(qr[i + half]) * sn : v * c + __bfloat162float(qr[i - half]) * sn;
      }
      qs[a.R + i] = __float2bfloat16_rn(v);
    }
  }
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = warp * 16 + g + 8 * h;
    const int tq = row / a.hb, hh = row % a.hb;
    pos_r[h] = (tq < nt && hh < nh) ? past + t0 + tq : -1;
    lo_r[h] = a.window > 0 ? max(0, pos_r[h] - a.window + 1) : 0;
  }
  const bool warp_active = __any_sync(0xffffffffu, pos_r[0] >= 0 || pos_r[1] >= 0);
  const int last_pos = past + t0 + nt - 1;
  int key_lo = a.window > 0 ? max(0, past + t0 - a.window + 1) : 0;
  key_lo = key_lo / 64 * 64;
  const int n_chunks = (last_pos - key_lo) / 64 + 1;
  const int per = (n_chunks + a.splits - 1) / a.splits;
  const int c_lo = slice * per, c_hi = min(n_chunks, c_lo + per);
  const int* trow = a.table + (size_t)seq * a.stride;
  const int col0 = grp * nt16 * 16;
  const float scale_log2 = a.scale * 1.4426950408889634f;

  float o[2 * NTM][4];
#pragma unroll
  for (int i = 0; i < 2 * NTM; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  const uint32_t q_base = smem_u32(Qs);
  const int pieces = W / 8;

  // a chunk of 64 cache rows into buffer `buf`: rows past the sequence become zeros, never stale values
  auto load_chunk = [&](int c, int buf) {
    const int k0 = key_lo + c * 64;
    const int nk = min(64, last_pos - k0 + 1);
    const __nv_bfloat16* src = pool + (size_t)trow[k0 / kPageTokens] * kPageTokens * W;
    __nv_bfloat16* base = Ks + (size_t)buf * 64 * ks;
    for (int i = tid; i < 64 * pieces; i += 128) {
      const int j = i / pieces, p8 = (i - j * pieces) * 8;
      __nv_bfloat16* dst = base + (size_t)j * ks + p8;
      if (j < nk) cp_async16(smem_u32(dst), src + (size_t)j * W + p8);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };
  // with two buffers the next chunk is on its way while this one is multiplied
  __syncthreads();
  if (buffers == 2 && c_lo < c_hi) load_chunk(c_lo, 0);
  for (int c = c_lo; c < c_hi; ++c) {
    const int k0 = key_lo + c * 64;
    int buf = 0;
    if (buffers == 2) {
      buf = (c - c_lo) & 1;
      if (c + 1 < c_hi) {
        load_chunk(c + 1, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
    } else {
      __syncthreads();
      load_chunk(c, 0);
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_base = smem_u32(Ks + (size_t)buf * 64 * ks);
    if (warp_active) {
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    for (int kb = 0; kb < W / 16; ++kb) {
      uint32_t qf[4];
      ldmatrix_x4(qf, q_base + 2 * ((warp * 16 + (lane & 15)) * ks + kb * 16 + ((lane >> 4) << 3)));
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        uint32_t kf[4];
        ldmatrix_x4(kf, k_base + 2 * ((jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ks + kb * 16 + (((lane >> 3) & 1) << 3)));
        mma_bf16(s[2 * jp], qf, kf[0], kf[1]);
        mma_bf16(s[2 * jp + 1], qf, kf[2], kf[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = k0 + j * 8 + 2 * t4 + (e & 1);
        float v = s[j][e] * scale_log2;
        if (key > pos_r[h] || key < lo_r[h]) v = -INFINITY;
        s[j][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_r[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = exp2f(m_r[h] - m_use[h]);
      m_r[h] = m_new;
    }
    float sum[2] = {0.f, 0.f};
    uint32_t pf[4][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
      const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
      sum[0] += p0 + p1;
      sum[1] += p2 + p3;
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_r[h] = l_r[h] * alpha[h] + sum[h];
#pragma unroll
    for (int i = 0; i < 2 * NTM; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
      for (int dp = 0; dp < NTM; ++dp) {
        if (dp < nt16 && col0 + dp * 16 < a.R) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, k_base + 2 * ((kb * 16 + (lane & 15)) * ks + col0 + dp * 16 + ((lane >> 4) << 3)));
          mma_bf16(o[2 * dp], pf[kb], vf[0], vf[1]);
          mma_bf16(o[2 * dp + 1], pf[kb], vf[2], vf[3]);
        }
      }
    }
    }
    if (buffers == 2) __syncthreads();      // this buffer is the target of the next iteration's prefetch
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (pos_r[h] < 0) continue;
    const int row = warp * 16 + g + 8 * h;
    const int tok = tok0 + row / a.hb, head = h0 + row % a.hb;
    if (a.splits == 1) {
      const float inv = l_r[h] > 0.f ? 1.0f / l_r[h] : 0.f;
      __nv_bfloat16* dst = (__nv_bfloat16*)a.out + ((size_t)head * a.T + tok) * a.R;
#pragma unroll
      for (int i = 0; i < 2 * NTM; ++i) {
        const int col = col0 + i * 8 + 2 * t4;
        if ((i >> 1) < nt16 && col < a.R)
          *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      }
    } else {
      float* dst = a.parts + ((size_t)slice * a.T * a.H + (size_t)tok * a.H + head) * (a.R + 2);
#pragma unroll
      for (int i = 0; i < 2 * NTM; ++i) {
        const int col = col0 + i * 8 + 2 * t4;
        if ((i >> 1) < nt16 && col < a.R) {
          dst[col] = o[i][2 * h];
          dst[col + 1] = o[i][2 * h + 1];
        }
      }
      if (grp == 0 && t4 == 0) {
        dst[a.R] = m_r[h] == -INFINITY ? -INFINITY : m_r[h] * 0.6931471805599453f;      // the merge works with e, not 2
        dst[a.R + 1] = l_r[h];
      }
    }
  }
}

// ---- whole prompts: attention with per-head keys and values (bfloat16) ----
// When every sequence of a step starts at position 0 its keys are the step's own tokens, and forming each head's
// unrotated key and value from the latents (one product for all tokens) costs little beside an attention that then
// multiplies d_n + d_r + d_v instead of r + d_r + r values per head and pair of tokens. Block: 64 query rows of one
// (sequence, head) on four warps; the queries stay in shared memory (the rotated part is turned as it is loaded);
// 64 keys a step in shared memory: the head's unrotated key values and the shared rotated part side by side, and the
// head's values; mma.sync m16n8k16, float32 sums, online softmax in registers.
struct HeadPromptArgs {
  const __nv_bfloat16* q;        // [T, H, dn + P] up-projected queries, rotated part not yet turned
  const __nv_bfloat16* kv;       // [T, H * dn + H * dv]: every head's unrotated key values, then every head's values
  const __nv_bfloat16* k_rot;    // [T, P] the shared key part, turned
  __nv_bfloat16* out;            // [H, T, dv]
  const float* cos_t;
  const float* sin_t;
  const int* seq_start;
  const int* counts;
  int T, H, dn, P, dv, rot, window;
  float scale;
};

template <int KQ, int NV>       // at most KQ * 16 key values and NV * 16 value columns a head
__global__ void __launch_bounds__(128, NV <= 8 ? 3 : 2) head_prompt_mma_kernel(const HeadPromptArgs a, int nbuf) {
  pdl_enter();
  extern __shared__ __align__(16) unsigned char hp_raw[];
  const int DK = a.dn + a.P, ksd = DK + 8, vsd = a.dv + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(hp_raw);   // [64][ksd]
  __nv_bfloat16* Ks = Qs + 64 * ksd;                              // nbuf buffers of [64][ksd]
  __nv_bfloat16* Vs = Ks + nbuf * 64 * ksd;                       // nbuf buffers of [64][vsd]
  const int seq = blockIdx.y, h = blockIdx.z;
  const int count = a.counts[seq];
  const int n_tiles = (count + 63) / 64;
  const int tile = n_tiles - 1 - (int)blockIdx.x;                 // the long tiles first
  if (tile < 0) return;
  const int r0 = tile * 64;
  const int tok0 = a.seq_start[seq];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int half = a.rot / 2;
  const int kv_stride = a.H * (a.dn + a.dv);
  // queries of rows r0 .. r0 + 63 (positions = rows: the sequences start at 0)
  for (int r = warp; r < 64; r += 4) {
    __nv_bfloat16* qs = Qs + r * ksd;
    const int pos = r0 + r;
    if (pos >= count) {
      for (int i = lane * 8; i < DK; i += 256) *reinterpret_cast<uint4*>(qs + i) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const __nv_bfloat16* src = a.q + ((size_t)(tok0 + pos) * a.H + h) * DK;
    for (int i = lane; i < a.dn; i += 32) qs[i] = src[i];
    const __nv_bfloat16* qr = src + a.dn;
    for (int i = lane; i < a.P; i += 32) {
      float v = __bfloat162float(qr[i]);
      if (i < a.rot) {
        const int f = i < half ? i : i - half;
        const float c = a.cos_t[(size_t)pos * half + f], sn = a.sin_t[(size_t)pos * half + f];
        v = i < half ? v * c - __bfloat162float(qr[i + half]) * sn : v * c + __bfloat162float(qr[i - half]) * sn;
      }
      qs[a.dn + i] = __float2bfloat16_rn(v);
    }
  }
  __syncthreads();
  const int kq = DK / 16, nv = a.dv / 16;
  const uint32_t q_at = smem_u32(Qs) + 2 * ((warp * 16 + (lane & 15)) * ksd + ((lane >> 4) << 3));   // this lane's part of a query fragment
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int p = r0 + warp * 16 + g + 8 * hh;
    pos_r[hh] = p < count ? p : -1;
    lo_r[hh] = a.window > 0 ? max(0, p - a.window + 1) : 0;
  }
  const bool warp_active = r0 + warp * 16 < count;
  const int last_pos = min(count, r0 + 64) - 1;
  const int key_lo = (a.window > 0 ? max(0, r0 - a.window + 1) : 0) / 64 * 64;
  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  const float scale_log2 = a.scale * 1.4426950408889634f;
  const int kp = a.dn / 8, rp = a.P / 8, vp = a.dv / 8;
  // 64 keys into buffer `buf`: the head's unrotated key values and the shared rotated part side by side, and its values.
  // Which 16-byte pieces a thread copies is the same at every step, so for heads of up to 128 key values it is worked out
  // once: per piece the place in the buffer (bits 0-19, bit 20: the value buffer, bit 21: the source is the shared key
  // part, bits 24-29: the key's row) and the source's element offset from the step's first key. (Measured at 96 + 64
  // values a head: 1,112 against 1,432 µs for eight layers. Packed into one word a piece the unpacking cost what the
  // plan saved: 1,526 µs.)
  constexpr int kMine = KQ <= 8 ? 16 : 1;
  const int per_row = kp + rp + vp;
  const bool planned = KQ <= 8 && 64 * per_row <= 128 * kMine;
  uint32_t where[kMine], from[kMine];
  if constexpr (KQ <= 8) {
#pragma unroll
    for (int q = 0; q < kMine; ++q) {
      const int i = tid + 128 * q;
      where[q] = 0xffffffffu;
      from[q] = 0;
      if (planned && i < 64 * per_row) {
        const int j = i / per_row, p = i - j * per_row;
        if (p < kp) { where[q] = (uint32_t)(2 * (j * ksd + p * 8)) | (j << 24); from[q] = j * kv_stride + h * a.dn + p * 8; }
        else if (p < kp + rp) { where[q] = (uint32_t)(2 * (j * ksd + a.dn + (p - kp) * 8)) | (1u << 21) | (j << 24); from[q] = j * a.P + (p - kp) * 8; }
        else { where[q] = (uint32_t)(2 * (j * vsd + (p - kp - rp) * 8)) | (1u << 20) | (j << 24); from[q] = j * kv_stride + a.H * a.dn + h * a.dv + (p - kp - rp) * 8; }
      }
    }
  }
  auto load_keys = [&](int k0, int buf) {
    const int nk = min(64, last_pos - k0 + 1);
    __nv_bfloat16* kb = Ks + buf * 64 * ksd;
    __nv_bfloat16* vb = Vs + buf * 64 * vsd;
    if constexpr (KQ <= 8) {
      if (planned) {
        const __nv_bfloat16* kv0 = a.kv + (size_t)(tok0 + k0) * kv_stride;
        const __nv_bfloat16* kr0 = a.k_rot + (size_t)(tok0 + k0) * a.P;
        const uint32_t kb_at = smem_u32(kb), vb_at = smem_u32(vb);
#pragma unroll
        for (int q = 0; q < kMine; ++q) {
          const uint32_t w = where[q];
          if (w == 0xffffffffu) continue;
          const uint32_t dst = ((w >> 20) & 1 ? vb_at : kb_at) + (w & 0xfffffu);
          if ((int)((w >> 24) & 63) < nk) cp_async16(dst, ((w >> 21) & 1 ? kr0 : kv0) + from[q]);
          else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0));
        }
        cp_async_commit();
        return;
      }
    }
    for (int i = tid; i < 64 * (kp + rp + vp); i += 128) {
      const int j = i / (kp + rp + vp), p = i - j * (kp + rp + vp);
      __nv_bfloat16* dst;
      const __nv_bfloat16* src;
      const size_t tok = (size_t)(tok0 + k0 + j);
      if (p < kp) { dst = kb + j * ksd + p * 8; src = a.kv + tok * kv_stride + h * a.dn + p * 8; }
      else if (p < kp + rp) { dst = kb + j * ksd + a.dn + (p - kp) * 8; src = a.k_rot + tok * a.P + (p - kp) * 8; }
      else { dst = vb + j * vsd + (p - kp - rp) * 8; src = a.kv + tok * kv_stride + a.H * a.dn + h * a.dv + (p - kp - rp) * 8; }
      if (j < nk) cp_async16(smem_u32(dst), src);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  // With two buffers the next 64 keys are on their way while these are multiplied; with one (chosen when that lets
  // more blocks share an SM) other blocks' products hide the wait.
  if (nbuf == 2) load_keys(key_lo, 0);
  int buf = 0;
  for (int k0 = key_lo; k0 <= last_pos; k0 += 64, buf = nbuf == 2 ? buf ^ 1 : 0) {
    if (nbuf == 2 && k0 + 64 <= last_pos) {
      load_keys(k0 + 64, buf ^ 1);
      cp_async_wait<1>();
    } else {
      if (nbuf == 1) load_keys(k0, 0);
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t k_base = smem_u32(Ks + buf * 64 * ksd), v_base = smem_u32(Vs + buf * 64 * vsd);
    if (warp_active && k0 <= r0 + warp * 16 + 15) {       // else: keys after all of this warp's rows
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kb = 0; kb < KQ; ++kb) {
      if (kb < kq) {
        uint32_t qf[4];          // fetched again every step: keeping all of them would cost the registers of a block more an SM
        ldmatrix_x4(qf, q_at + 2 * kb * 16);
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {
          uint32_t kf[4];
          ldmatrix_x4(kf, k_base + 2 * ((jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * ksd + kb * 16 + (((lane >> 3) & 1) << 3)));
          mma_bf16(s[2 * jp], qf, kf[0], kf[1]);
          mma_bf16(s[2 * jp + 1], qf, kf[2], kf[3]);
        }
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int hh = e >> 1;
        const int key = k0 + j * 8 + 2 * t4 + (e & 1);
        float v = s[j][e] * scale_log2;
        if (key > pos_r[hh] || key < lo_r[hh]) v = -INFINITY;
        s[j][e] = v;
        mx[hh] = fmaxf(mx[hh], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
      const float m_new = fmaxf(m_r[hh], mx[hh]);
      m_use[hh] = m_new == -INFINITY ? 0.f : m_new;
      alpha[hh] = exp2f(m_r[hh] - m_use[hh]);
      m_r[hh] = m_new;
    }
    float sum[2] = {0.f, 0.f};
    uint32_t pf[4][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
      const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
      sum[0] += p0 + p1;
      sum[1] += p2 + p3;
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) l_r[hh] = l_r[hh] * alpha[hh] + sum[hh];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
      for (int dp = 0; dp < NV; ++dp) {
        if (dp < nv) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, v_base + 2 * ((kb * 16 + (lane & 15)) * vsd + dp * 16 + ((lane >> 4) << 3)));
          mma_bf16(o[2 * dp], pf[kb], vf[0], vf[1]);
          mma_bf16(o[2 * dp + 1], pf[kb], vf[2], vf[3]);
        }
      }
    }
    }
    __syncthreads();      // this buffer is the target of the next iteration's fetch
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_r[hh] += __shfl_xor_sync(0xffffffffu, l_r[hh], 1);
    l_r[hh] += __shfl_xor_sync(0xffffffffu, l_r[hh], 2);
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    if (pos_r[hh] < 0) continue;
    const float inv = l_r[hh] > 0.f ? 1.0f / l_r[hh] : 0.f;
    __nv_bfloat16* dst = a.out + ((size_t)h * a.T + tok0 + pos_r[hh]) * a.dv;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
      if ((i >> 1) < nv)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][2 * hh] * inv, o[i][2 * hh + 1] * inv);
  }
}

// One block per (token, head): the slices' factors exp(m_s - m) / mass are formed once, then every thread joins its
// columns over the slices in slice order.
template <typename T>
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ parts, T* __restrict__ out, int rows, int Tn,
                                                           int H, int R, int splits) {
  pdl_enter();
  __shared__ float factor[64];
  const int row = blockIdx.x;
  const int tok = row / H, h = row % H;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = lane < splits ? parts[((size_t)lane * rows + row) * (R + 2) + R] : -INFINITY;
    float m1 = lane + 32 < splits ? parts[((size_t)(lane + 32) * rows + row) * (R + 2) + R] : -INFINITY;
    const float mx = warp_max(fmaxf(m0, m1));
    float f0 = m0 == -INFINITY ? 0.f : expf(m0 - mx), f1 = m1 == -INFINITY ? 0.f : expf(m1 - mx);
    float l0 = lane < splits ? parts[((size_t)lane * rows + row) * (R + 2) + R + 1] : 0.f;
    float l1 = lane + 32 < splits ? parts[((size_t)(lane + 32) * rows + row) * (R + 2) + R + 1] : 0.f;
    // the mass is summed in slice order by one lane, so that the result does not depend on the lanes' tree
    factor[lane] = f0 * l0;
    factor[lane + 32] = f1 * l1;
    __syncwarp();
    float mass = 0.f;
    if (lane == 0)
      for (int s = 0; s < splits; ++s) mass += factor[s];
    mass = __shfl_sync(0xffffffffu, mass, 0);
    const float inv = mass > 0.f ? 1.0f / mass : 0.f;
    __syncwarp();
    factor[lane] = f0 * inv;
    factor[lane + 32] = f1 * inv;
  }
  __syncthreads();
  T* o = out + ((size_t)h * Tn + tok) * R;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float f = factor[s];
      if (f != 0.f) v = fmaf(parts[((size_t)s * rows + row) * (R + 2) + d], f, v);
    }
    o[d] = from_f32<T>(v);
  }
}

// One gate value per head: y[t, h * dv + j] = val[h, t, j] * sigmoid(g[t * g_stride + h]), g float32.
template <typename T>
__global__ void latent_head_gate_kernel(const T* __restrict__ val, const float* __restrict__ g, long long g_stride,
                                        T* __restrict__ y, int Tn, int H, int dv, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / ((size_t)H * dv);
    const int rest = (int)(i - t * H * dv), h = rest / dv, j = rest - h * dv;
    const float v = to_f32(val[((size_t)h * Tn + t) * dv + j]);
    const float z = g[t * g_stride + h];
    y[i] = from_f32<T>(v * (1.0f / (1.0f + expf(-z))));
  }
}

// The bfloat16 form for value widths that are multiples of 8: a thread moves eight values (16 bytes) at a time; the
// arithmetic of a value is the one above.
__global__ void latent_head_gate_bf16x8_kernel(const uint4* __restrict__ val, const float* __restrict__ g, long long g_stride,
                                               uint4* __restrict__ y, int Tn, int H, int dv8, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / ((size_t)H * dv8);
    const int rest = (int)(i - t * H * dv8), h = rest / dv8, j = rest - h * dv8;
    uint4 raw = val[((size_t)h * Tn + t) * dv8 + j];
    const float z = g[t * g_stride + h];
    const float sig = 1.0f / (1.0f + expf(-z));
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(pr[k]);
      pr[k] = __floats2bfloat162_rn(f.x * sig, f.y * sig);
    }
    y[i] = raw;
  }
}

// y[t, h * dv + j] = val[h, t, j] * sigmoid(g[t, h * dv + j])
template <typename T>
__global__ void latent_gate_kernel(const T* __restrict__ val, const T* __restrict__ g, T* __restrict__ y, int Tn, int H,
                                   int dv, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / ((size_t)H * dv);
    const int rest = (int)(i - t * H * dv), h = rest / dv, j = rest - h * dv;
    const float v = to_f32(val[((size_t)h * Tn + t) * dv + j]);
    const float z = to_f32(g[i]);
    y[i] = from_f32<T>(v * (1.0f / (1.0f + expf(-z))));
  }
}

static int lat_rv(int R) {
  const int need = (R + 31) / 32;
  for (int v : {1, 2, 3, 4, 6, 8, 12, 16, 24, 32})
    if (need <= v) return v;
  return 0;
}

static int lat_chunk_for(int W, int& kstride, size_t& bytes) {
  kstride = (W % 2 == 0) ? W + 1 : W;
  for (int chunk : {64, 32, 16}) {
    bytes = ((size_t)kLatRows * W + (size_t)chunk * kstride + (size_t)kLatWarps * 64 * kLatRowsPerWarp) * sizeof(float);
    if (bytes <= 200 * 1024) return chunk;
  }
  return 0;
}

}  // namespace slb

using namespace slb;

extern "C" int slb_latent_post(const float* lat, const float* q_gain, const float* c_gain, const float* cos_t,
                               const float* sin_t, void* cq, void* pool, const int* tok_seq, const int* tok_pos,
                               const int* table, int stride, int tokens, int q_rank, int R, int P, int rot, float eps,
                               int dtype, void* c_out, void* k_out, int lat_stride, void* stream) {
  SLB_REQUIRE(tokens >= 0 && q_rank >= 0 && R > 0 && P >= 0 && rot >= 0 && rot <= P && rot % 2 == 0 && eps > 0.f,
              "latent_post: tokens=%d q_rank=%d rank=%d rot_dim=%d rotated=%d", tokens, q_rank, R, P, rot);
  if (lat_stride <= 0) lat_stride = q_rank + R + P;
  SLB_REQUIRE(lat_stride >= q_rank + R + P && (q_rank == 0 || cq != nullptr), "latent_post: rows of %d values hold %d + %d + %d",
              lat_stride, q_rank, R, P);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "latent_post: unknown dtype %d", dtype);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int widest = q_rank > R ? q_rank : R;
  const int threads = widest > 512 ? 256 : (widest > 128 ? 128 : 64);
  if (dtype == kF32)
    launch(latent_post_kernel<float>, dim3(tokens), dim3(threads), 0, s, lat, q_gain, c_gain, cos_t, sin_t, (float*)cq,
           (float*)pool, tok_seq, tok_pos, table, stride, q_rank, R, P, rot, eps, (float*)c_out, (float*)k_out, lat_stride);
  else
    launch(latent_post_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, s, lat, q_gain, c_gain, cos_t, sin_t,
           (__nv_bfloat16*)cq, (__nv_bfloat16*)pool, tok_seq, tok_pos, table, stride, q_rank, R, P, rot, eps, (__nv_bfloat16*)c_out,
           (__nv_bfloat16*)k_out, lat_stride);
  return check_launch("latent_post");
}

// Whether the attention kernel takes these sizes (latent width and rotated width).
extern "C" int slb_latent_attention_supported(int R, int P) {
  int kstride;
  size_t bytes;
  return R > 0 && P >= 0 && lat_rv(R) > 0 && lat_chunk_for(R + P, kstride, bytes) > 0 ? 1 : 0;
}

// Tests set this to compare the tensor-core kernel with the general one on the same inputs.
static int slb_latent_force_generic = 0;
extern "C" int slb_latent_attention_general_only(int on) {
  slb_latent_force_generic = on;
  return 0;
}

extern "C" int slb_latent_attention(const void* q_lat, const void* q_raw, const void* pool, void* out, float* parts,
                                    const float* cos_t, const float* sin_t, const int* seq_start, const int* past,
                                    const int* counts, const int* table, int stride, int n_seqs, int max_count, int T,
                                    int H, int R, int P, int dn, int rot, int window, float scale, int splits,
                                    int dtype, void* stream) {
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && T >= 0 && H > 0 && R > 0 && P >= 0 && dn >= 0 && rot >= 0 && rot <= P &&
                  rot % 2 == 0 && splits >= 1 && window >= 0,
              "latent_attention: seqs=%d max=%d heads=%d rank=%d rot_dim=%d splits=%d", n_seqs, max_count, H, R, P, splits);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "latent_attention: unknown dtype %d", dtype);
  SLB_REQUIRE(splits == 1 || parts != nullptr, "latent_attention: slices need scratch memory");
  SLB_REQUIRE(splits <= 64, "latent_attention: at most 64 slices, got %d", splits);
  if (n_seqs == 0 || max_count == 0 || T == 0) return 0;
  LatentAttnArgs a;
  a.q_lat = q_lat; a.q_raw = q_raw; a.pool = pool; a.out = out; a.parts = parts; a.cos_t = cos_t; a.sin_t = sin_t;
  a.seq_start = seq_start; a.past = past; a.counts = counts; a.table = table; a.stride = stride; a.T = T; a.H = H;
  a.R = R; a.P = P; a.dn = dn; a.rot = rot; a.window = window; a.splits = splits; a.scale = scale;
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned = ((uintptr_t)q_lat | (uintptr_t)q_raw | (uintptr_t)pool | (uintptr_t)out) % 16 == 0;
  if (dtype == kBF16 && R % 16 == 0 && (R + P) % 16 == 0 && aligned && (size_t)128 * (R + P + 8) * 2 <= kLatMaxSmem &&
      !slb_latent_force_generic) {
    const int tiles16 = R / 16;
    const int groups = (tiles16 + 15) / 16;
    const int nt16 = (tiles16 + groups - 1) / groups;
    a.chunk = 64;
    a.kstride = R + P + 8;
    a.hb = H < 64 ? H : 64;
    a.tq = 64 / a.hb;
    const int head_chunks = (H + a.hb - 1) / a.hb;
    const int buffers = (size_t)192 * a.kstride * 2 <= kLatMaxSmem ? 2 : 1;
    const size_t smem = (size_t)(64 + 64 * buffers) * a.kstride * 2;
    const dim3 grid((max_count + a.tq - 1) / a.tq, n_seqs, head_chunks * groups * splits), block(128);
#define SLB_LATM(V)                                                                                              \
  do {                                                                                                           \
    static bool raised = false;                                                                                  \
    if (!raised) {                                                                                               \
      cudaFuncSetAttribute(latent_attn_mma_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLatMaxSmem);   \
      raised = true;                                                                                             \
    }                                                                                                            \
    launch(latent_attn_mma_kernel<V>, grid, block, smem, s, a, nt16, groups, buffers);                                   \
  } while (0)
    if (nt16 <= 4) SLB_LATM(4); else if (nt16 <= 8) SLB_LATM(8); else SLB_LATM(16);
#undef SLB_LATM
    int rc = check_launch("latent_attention");
    if (rc || splits == 1) return rc;
    const int rows = T * H;
    launch(latent_merge_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s, (const float*)parts,
           (__nv_bfloat16*)out, rows, T, H, R, splits);
    return check_launch("latent_merge");
  }
  size_t bytes;
  a.chunk = lat_chunk_for(R + P, a.kstride, bytes);
  const int rv = lat_rv(R);
  SLB_REQUIRE(a.chunk > 0 && rv > 0, "latent_attention: a cache row of %d values (latent %d) is too wide", R + P, R);
  a.hb = H < kLatRows ? H : kLatRows;
  a.tq = kLatRows / a.hb;
  const int head_chunks = (H + a.hb - 1) / a.hb;
  const dim3 grid((max_count + a.tq - 1) / a.tq, n_seqs, head_chunks * splits), block(kLatWarps * 32);
#define SLB_LAT(TT, V)                                                                                   \
  do {                                                                                                   \
    static bool raised_##V = false;                                                                      \
    if (!raised_##V) {                                                                                   \
      cudaFuncSetAttribute(latent_attn_kernel<TT, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
      raised_##V = true;                                                                                 \
    }                                                                                                    \
    launch(latent_attn_kernel<TT, V>, grid, block, bytes, s, a);                                         \
  } while (0)
#define SLB_LAT_RV(TT)                                                                   \
  switch (rv) {                                                                          \
    case 1: SLB_LAT(TT, 1); break;   case 2: SLB_LAT(TT, 2); break;                      \
    case 3: SLB_LAT(TT, 3); break;   case 4: SLB_LAT(TT, 4); break;                      \
    case 6: SLB_LAT(TT, 6); break;   case 8: SLB_LAT(TT, 8); break;                      \
    case 12: SLB_LAT(TT, 12); break; case 16: SLB_LAT(TT, 16); break;                    \
    case 24: SLB_LAT(TT, 24); break; default: SLB_LAT(TT, 32); break;                    \
  }
  if (dtype == kF32) { SLB_LAT_RV(float) } else { SLB_LAT_RV(__nv_bfloat16) }
#undef SLB_LAT_RV
#undef SLB_LAT
  int rc = check_launch("latent_attention");
  if (rc || splits == 1) return rc;
  const int rows = T * H;
  if (dtype == kF32)
    launch(latent_merge_kernel<float>, dim3(rows), dim3(128), 0, s, (const float*)parts, (float*)out, rows, T, H, R, splits);
  else
    launch(latent_merge_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s, (const float*)parts,
           (__nv_bfloat16*)out, rows, T, H, R, splits);
  return check_launch("latent_merge");
}

// Whether the per-head prompt kernel takes these head sizes (bfloat16 only).
extern "C" int slb_head_prompt_supported(int dn, int P, int dv) {
  const int DK = dn + P;
  return dn > 0 && dv > 0 && dn % 8 == 0 && P % 8 == 0 && DK % 16 == 0 && dv % 16 == 0 && DK <= 256 && dv <= 256 ? 1 : 0;
}

// Attention of whole prompts (every sequence starts at position 0) with per-head keys and values; see HeadPromptArgs.
extern "C" int slb_head_prompt_attention(const void* q, const void* kv, const void* k_rot, void* out, const float* cos_t,
                                         const float* sin_t, const int* seq_start, const int* counts, int n_seqs,
                                         int max_count, int T, int H, int dn, int P, int dv, int rot, int window,
                                         float scale, void* stream) {
  SLB_REQUIRE(slb_head_prompt_supported(dn, P, dv), "head_prompt_attention: head sizes %d + %d, %d are not taken", dn, P, dv);
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && T >= 0 && H > 0 && rot >= 0 && rot <= P && rot % 2 == 0 && window >= 0,
              "head_prompt_attention: seqs=%d max=%d heads=%d", n_seqs, max_count, H);
  SLB_REQUIRE((((uintptr_t)q | (uintptr_t)kv | (uintptr_t)k_rot | (uintptr_t)out) % 16 == 0) && (H * (dn + dv)) % 8 == 0,
              "head_prompt_attention: 16-byte alignment");
  if (n_seqs == 0 || max_count == 0 || T == 0) return 0;
  HeadPromptArgs a;
  a.q = (const __nv_bfloat16*)q; a.kv = (const __nv_bfloat16*)kv; a.k_rot = (const __nv_bfloat16*)k_rot;
  a.out = (__nv_bfloat16*)out; a.cos_t = cos_t; a.sin_t = sin_t; a.seq_start = seq_start; a.counts = counts;
  a.T = T; a.H = H; a.dn = dn; a.P = P; a.dv = dv; a.rot = rot; a.window = window; a.scale = scale;
  // two key buffers where four blocks still fit an SM's shared memory with them, else one
  const size_t smem2 = (size_t)(192 * (dn + P + 8) + 128 * (dv + 8)) * 2, smem1 = (size_t)(128 * (dn + P + 8) + 64 * (dv + 8)) * 2;
  const int nbuf = smem2 * 3 <= kLatMaxSmem ? 2 : 1;
  const size_t smem = nbuf == 2 ? smem2 : smem1;
  const dim3 grid((max_count + 63) / 64, n_seqs, H), block(128);
  cudaStream_t s = (cudaStream_t)stream;
  const int kq = (dn + P) / 16, nv = dv / 16;
#define SLB_HP(KQ, NV)                                                                                          \
  do {                                                                                                          \
    static bool raised = false;                                                                                 \
    if (!raised) {                                                                                              \
      cudaFuncSetAttribute(head_prompt_mma_kernel<KQ, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLatMaxSmem); \
      raised = true;                                                                                            \
    }                                                                                                           \
    launch(head_prompt_mma_kernel<KQ, NV>, grid, block, smem, s, a, nbuf);                                         \
  } while (0)
  if (kq <= 8) {
    if (nv <= 4) SLB_HP(8, 4); else if (nv <= 8) SLB_HP(8, 8); else SLB_HP(8, 16);
  } else {
    if (nv <= 4) SLB_HP(16, 4); else if (nv <= 8) SLB_HP(16, 8); else SLB_HP(16, 16);
  }
#undef SLB_HP
  return check_launch("head_prompt_attention");
}

extern "C" int slb_latent_gate(const void* val, const void* g, void* y, int tokens, int H, int dv, int dtype,
                               void* stream) {
  SLB_REQUIRE(tokens >= 0 && H > 0 && dv > 0, "latent_gate: tokens=%d heads=%d width=%d", tokens, H, dv);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)tokens * H * dv;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  if (dtype == kF32)
    launch(latent_gate_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)val, (const float*)g, (float*)y, tokens, H, dv, total);
  else if (dtype == kBF16)
    launch(latent_gate_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, (const __nv_bfloat16*)val,
           (const __nv_bfloat16*)g, (__nv_bfloat16*)y, tokens, H, dv, total);
  else
    return fail(1, "latent_gate: unknown dtype %d", dtype);
  return check_launch("latent_gate");
}

// val [H, tokens, dv] and y [tokens, H * dv] in `dtype`; g float32, one value per (token, head), rows g_stride apart.
extern "C" int slb_latent_head_gate(const void* val, const float* g, long long g_stride, void* y, int tokens, int H, int dv,
                                    int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && H > 0 && dv > 0 && g_stride >= H, "latent_head_gate: tokens=%d heads=%d width=%d", tokens, H, dv);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)tokens * H * dv;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  if (dtype == kBF16 && dv % 8 == 0 && (uintptr_t)val % 16 == 0 && (uintptr_t)y % 16 == 0) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + 255) / 256;
    if (b8 > (size_t)sm_count() * 16) b8 = (size_t)sm_count() * 16;
    launch(latent_head_gate_bf16x8_kernel, dim3((int)b8), dim3(256), 0, s, (const uint4*)val, g, g_stride, (uint4*)y, tokens, H, dv / 8,
           total8);
    return check_launch("latent_head_gate");
  }
  if (dtype == kF32)
    launch(latent_head_gate_kernel<float>, dim3((int)blocks), dim3(256), 0, s, (const float*)val, g, g_stride, (float*)y, tokens, H, dv, total);
  else if (dtype == kBF16)
    launch(latent_head_gate_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, s, (const __nv_bfloat16*)val, g, g_stride,
           (__nv_bfloat16*)y, tokens, H, dv, total);
  else
    return fail(1, "latent_head_gate: unknown dtype %d", dtype);
  return check_launch("latent_head_gate");
}
