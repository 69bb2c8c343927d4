// Sliding-window attention with pooled blocks and a sink, over the paged cache.  Compiled for one key size D
// (DRYFT_QK_DIM), one value size DV (DRYFT_V_DIM) and REP query heads per key/value head (DRYFT_GROUP).
//
// The query at position i of its sequence sees the tokens j with 0 <= i - j < size and, beside them, ONE key and value
// for every block of P positions that lies wholly before the window (block b = positions bP .. bP + P - 1, seen when
// bP + P - 1 <= i - size): the mean of the block's P cached keys and the mean of its P cached values, kept in pages of
// their own, one row per block.  Tokens and blocks share one softmax, whose denominator also holds exp(sink_h), a
// number per head without key or value.  Scores, weights and sums are 32-bit; q, k, v and the pooled rows have the
// activation type T.
//
//   pool_attn_prep    per token: q, k (+ bias) rotated over their first `rot` dims (dims i and i + rot/2 turn together by
//                     the angle pos * inv_freq[i], evaluated in 32-bit), THEN divided by their root mean square over D
//                     (no weight; skipped when eps < 0); v (+ bias); k and v written into the cache at the token's position.  One warp a vector.
//   pool_attn_prep_tok  the same per token for projections that are normed as a whole: q (all H * D values at once) and k (all
//                     G * D) are divided by their root mean square and multiplied by a weight per entry BEFORE the rotation,
//                     and the rotation pairs either dims i and i + rot/2 or (interleaved) dims 2i and 2i + 1.  One block a
//                     token: the two sums of squares first, then a warp a vector.
//   pool_attn_blocks  every token that completes a block (pos % P == P - 1) averages the block's P cached keys and
//                     values into the pooled pages.  One block per (token, kv head); all others return at once.
//   pool_attn_rows    one block per (token, kv head, split): the REP query heads of the kv head over the visible pooled
//                     rows and tokens (one list of keys; a lane a key for the scores, a lane a value column for the
//                     weighted sum), online softmax per warp, warps combined in shared memory; with one split the sink
//                     joins there and the output is written, else partial (max, sum, weighted sum) go to memory and
//   pool_attn_combine joins the splits and the sink.
// Tokens with slot -1 (padding) are skipped.  No block waits on another block.
#include "common.cuh"
#include <math.h>

#ifndef DRYFT_QK_DIM
#error "compile with -DDRYFT_QK_DIM, -DDRYFT_V_DIM and -DDRYFT_GROUP"
#endif

namespace {
constexpr int D = DRYFT_QK_DIM, DV = DRYFT_V_DIM, REP = DRYFT_GROUP;
constexpr int DR = (D + 31) / 32, DVR = (DV + 31) / 32;
constexpr int ROWS_WARPS = 4;
constexpr int BLOCKS_THREADS = (D + DV + 31) / 32 * 32 < 1024 ? (D + DV + 31) / 32 * 32 : 1024;   // a thread a column of a key or a value
constexpr int PREP_WARPS = 4;
constexpr int PREP_TOK_WARPS = 8;    // pool_attn_prep_tok: a block a token, its vectors dealt to the warps

// sin and cos of  pos * (f_hi + f_lo): the product is formed in 32-bit, and what its rounding drops (recovered exactly with
// one fused multiply-add) plus the low half of the frequency are applied as a first-order turn.  f_lo = 0 gives the plain
// 32-bit angle to within that correction.
__device__ __forceinline__ void sincos_split(float pos, float f_hi, float f_lo, float* sn, float* cs) {
  const float a = pos * f_hi;
  const float e = fmaf(pos, f_hi, -a) + pos * f_lo;
  float s, c;
  sincosf(a, &s, &c);
  *sn = fmaf(e, c, s);
  *cs = fmaf(-e, s, c);
}

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32) pool_attn_prep_kernel(
    const T* __restrict__ proj, int ld, const float* __restrict__ qb, const float* __restrict__ kb, const float* __restrict__ vb,
    const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, int rot, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages,
    int page_size, int n_tokens, int H, int G, float eps, int write_kv) {
  __shared__ float sm[PREP_WARPS][D > DV ? D : DV];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_tok = H + (write_kv ? 2 * G : 0);
  const long long item = (long long)blockIdx.x * PREP_WARPS + warp;
  if (item >= (long long)n_tokens * per_tok) return;
  const int t = (int)(item / per_tok), vec = (int)(item % per_tok);
  const int slot = tok_slot[t];
  if (slot < 0) return;
  const int pos = tok_pos[t];
  const T* row = proj + (size_t)t * ld;
  size_t cache_row = 0;
  if (vec >= H) {
    const int g = (vec - H) % G;
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    cache_row = ((size_t)page * G + g) * page_size + pos % page_size;
  }
  if (vec >= H + G) {     // a value vector: bias, cache
    const int g = vec - H - G;
    const T* src = row + (size_t)H * D + (size_t)G * D + (size_t)g * DV;
    for (int c = lane; c < DV; c += 32)
      v_pages[cache_row * DV + c] = from_f32<T>(to_f32<T>(src[c]) + (vb != nullptr ? vb[g * DV + c] : 0.f));
    return;
  }
  const bool is_q = vec < H;
  const int hd = is_q ? vec : vec - H;
  const T* src = row + (is_q ? (size_t)hd * D : (size_t)H * D + (size_t)hd * D);
  const float* bias = is_q ? qb : kb;
  float* s = sm[warp];
  for (int c = lane; c < D; c += 32) s[c] = to_f32<T>(src[c]) + (bias != nullptr ? bias[hd * D + c] : 0.f);
  __syncwarp();
  const int half = rot / 2;
  const float fpos = (float)pos;
  float o[DR];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < DR; ++r) {
    const int c = lane + 32 * r;
    float v = 0.f;
    if (c < D) {
      if (c < half) {
        float sn, cs;
        sincos_split(fpos, inv_freq[c], inv_freq_lo != nullptr ? inv_freq_lo[c] : 0.f, &sn, &cs);
        v = s[c] * cs - s[c + half] * sn;
      } else if (c < rot) {
        float sn, cs;
        sincos_split(fpos, inv_freq[c - half], inv_freq_lo != nullptr ? inv_freq_lo[c - half] : 0.f, &sn, &cs);
        v = s[c] * cs + s[c - half] * sn;
      } else {
        v = s[c];
      }
    }
    o[r] = v;
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float rinv = eps >= 0.f ? 1.f / sqrtf(ss / (float)D + eps) : 1.f;    // eps < 0: no unit norm
  T* dst = is_q ? q_out + ((size_t)t * H + hd) * D : k_pages + cache_row * D;
#pragma unroll
  for (int r = 0; r < DR; ++r) {
    const int c = lane + 32 * r;
    if (c < D) dst[c] = from_f32<T>(o[r] * rinv);
  }
}

// One block per token.  q_w [H * D] / k_w [G * D]: the weights of a norm over the whole projection (nullptr: no such norm).
template <typename T>
__global__ void __launch_bounds__(PREP_TOK_WARPS * 32) pool_attn_prep_tok_kernel(
    const T* __restrict__ proj, int ld, const float* __restrict__ q_w, const float* __restrict__ k_w, float norm_eps,
    const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, int rot, int interleaved, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const int* __restrict__ page_table, int max_pages, int page_size, int H, int G, float eps, int write_kv) {
  __shared__ float sm[PREP_TOK_WARPS][D];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int slot = tok_slot[t];
  if (slot < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = tok_pos[t];
  const T* row = proj + (size_t)t * ld;
  float rq = 1.f, rk = 1.f;
  if (q_w != nullptr) {
    float a = 0.f;
    for (int c = threadIdx.x; c < H * D; c += PREP_TOK_WARPS * 32) { const float v = to_f32<T>(row[c]); a = fmaf(v, v, a); }
    rq = 1.f / sqrtf(block_sum(a, scratch) / (float)(H * D) + norm_eps);
  }
  if (k_w != nullptr && write_kv) {
    float a = 0.f;
    for (int c = threadIdx.x; c < G * D; c += PREP_TOK_WARPS * 32) { const float v = to_f32<T>(row[(size_t)H * D + c]); a = fmaf(v, v, a); }
    rk = 1.f / sqrtf(block_sum(a, scratch) / (float)(G * D) + norm_eps);
  }
  size_t cache_row0 = 0;
  if (write_kv) cache_row0 = (size_t)page_table[(size_t)slot * max_pages + pos / page_size];
  const int per_tok = H + (write_kv ? 2 * G : 0);
  const int half = rot / 2;
  const float fpos = (float)pos;
  float* s = sm[warp];
  for (int vec = warp; vec < per_tok; vec += PREP_TOK_WARPS) {
    if (vec >= H + G) {     // a value vector: into the cache as it is
      const int g = vec - H - G;
      const size_t cr = (cache_row0 * G + g) * page_size + pos % page_size;
      const T* src = row + (size_t)H * D + (size_t)G * D + (size_t)g * DV;
      for (int c = lane; c < DV; c += 32) v_pages[cr * DV + c] = src[c];
      continue;
    }
    const bool is_q = vec < H;
    const int hd = is_q ? vec : vec - H;
    const T* src = row + (is_q ? (size_t)hd * D : (size_t)H * D + (size_t)hd * D);
    const float* w = is_q ? q_w : k_w;
    const float r = is_q ? rq : rk;
    __syncwarp();
    for (int c = lane; c < D; c += 32) s[c] = w != nullptr ? to_f32<T>(src[c]) * r * w[hd * D + c] : to_f32<T>(src[c]);
    __syncwarp();
    float o[DR];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < DR; ++k) {
      const int c = lane + 32 * k;
      float v = 0.f;
      if (c < D) {
        if (c < rot) {
          // the entry this one turns with, the pair's frequency, and which of the two it is
          const int i = interleaved ? (c >> 1) : (c < half ? c : c - half);
          const bool first = interleaved ? !(c & 1) : c < half;
          const int other = interleaved ? (c ^ 1) : (first ? c + half : c - half);
          float sn, cs;
          sincos_split(fpos, inv_freq[i], inv_freq_lo != nullptr ? inv_freq_lo[i] : 0.f, &sn, &cs);
          v = first ? s[c] * cs - s[other] * sn : s[c] * cs + s[other] * sn;
        } else {
          v = s[c];
        }
      }
      o[k] = v;
      ss = fmaf(v, v, ss);
    }
    float rinv = 1.f;
    if (eps >= 0.f) rinv = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);    // eps < 0: no unit norm
    T* dst = is_q ? q_out + ((size_t)t * H + hd) * D : k_pages + ((cache_row0 * G + hd) * page_size + pos % page_size) * D;
#pragma unroll
    for (int k = 0; k < DR; ++k) {
      const int c = lane + 32 * k;
      if (c < D) dst[c] = from_f32<T>(o[k] * rinv);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(BLOCKS_THREADS) pool_attn_blocks_kernel(
    const T* __restrict__ k_pages, const T* __restrict__ v_pages, const int* __restrict__ page_table, int max_pages, int page_size,
    T* __restrict__ pk_pages, T* __restrict__ pv_pages, const int* __restrict__ pool_table, int pool_max_pages,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int G, int P) {
  const int t = blockIdx.x, g = blockIdx.y;
  const int slot = tok_slot[t];
  if (slot < 0) return;
  const int pos = tok_pos[t];
  if (pos % P != P - 1) return;
  const int b = pos / P, p0 = pos - (P - 1);
  const int ppage = pool_table[(size_t)slot * pool_max_pages + b / page_size];
  const size_t prow = ((size_t)ppage * G + g) * page_size + b % page_size;
  const float inv = 1.f / (float)P;
  for (int c = threadIdx.x; c < D + DV; c += blockDim.x) {
    float acc = 0.f;
#pragma unroll 8
    for (int j = 0; j < P; ++j) {   // rows in order: the sum does not depend on how the loads are scheduled
      const int pj = p0 + j;
      const int page = page_table[(size_t)slot * max_pages + pj / page_size];
      const size_t r = ((size_t)page * G + g) * page_size + pj % page_size;
      acc += c < D ? to_f32<T>(k_pages[r * D + c]) : to_f32<T>(v_pages[r * DV + (c - D)]);
    }
    if (c < D) pk_pages[prow * D + c] = from_f32<T>(acc * inv);
    else pv_pages[prow * DV + (c - D)] = from_f32<T>(acc * inv);
  }
}

template <typename T> __device__ __forceinline__ void dot_row(const T* __restrict__ kr, const float (*qs)[D], float* dots) {
  constexpr int V = 16 / sizeof(T);
  if (D % V == 0) {
#pragma unroll 2
    for (int c = 0; c < D; c += V) {
      const uint4 kv = *reinterpret_cast<const uint4*>(kr + c);
      const T* ke = reinterpret_cast<const T*>(&kv);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float kf = to_f32<T>(ke[e]);
#pragma unroll
        for (int h = 0; h < REP; ++h) dots[h] = fmaf(kf, qs[h][c + e], dots[h]);
      }
    }
  } else {
    for (int c = 0; c < D; ++c) {
      const float kf = to_f32<T>(kr[c]);
#pragma unroll
      for (int h = 0; h < REP; ++h) dots[h] = fmaf(kf, qs[h][c], dots[h]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(ROWS_WARPS * 32) pool_attn_rows_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, const int* __restrict__ page_table,
    int max_pages, int page_size, const T* __restrict__ pk_pages, const T* __restrict__ pv_pages, const int* __restrict__ pool_table,
    int pool_max_pages, const float* __restrict__ sink, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int G, int n_splits, float scale, int size, int P) {
  __shared__ float qs[REP][D];
  __shared__ float wo[ROWS_WARPS][REP][DV];
  __shared__ float wml[ROWS_WARPS][REP][2];
  const int t = blockIdx.x, g = blockIdx.y, sp = blockIdx.z;
  const int slot = tok_slot[t];
  if (slot < 0) return;
  const int H = G * REP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = tok_pos[t];
  const int lo = max(0, i - size + 1);
  const int nb = (P > 0 && i - size + 1 >= P) ? (i - size + 1) / P : 0;
  const int nkeys = nb + (i - lo + 1);
  int chunk = (nkeys + n_splits - 1) / n_splits;
  chunk = (chunk + 31) / 32 * 32;
  const int u0 = sp * chunk, u1 = min(nkeys, u0 + chunk);
  for (int c = threadIdx.x; c < REP * D; c += blockDim.x) qs[c / D][c % D] = to_f32<T>(q[((size_t)t * H + (size_t)g * REP) * D + c]);
  __syncthreads();

  float m[REP], l[REP], o[REP][DVR];
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int r = 0; r < DVR; ++r) o[h][r] = 0.f;
  }
  for (int tile = u0 + warp * 32; tile < u1; tile += ROWS_WARPS * 32) {
    const int u = tile + lane;
    const bool valid = u < u1;
    const T* kr = k_pages;
    const T* vr = v_pages;
    if (valid) {
      if (u < nb) {
        const int page = pool_table[(size_t)slot * pool_max_pages + u / page_size];
        const size_t r = ((size_t)page * G + g) * page_size + u % page_size;
        kr = pk_pages + r * D;
        vr = pv_pages + r * DV;
      } else {
        const int j = lo + (u - nb);
        const int page = page_table[(size_t)slot * max_pages + j / page_size];
        const size_t r = ((size_t)page * G + g) * page_size + j % page_size;
        kr = k_pages + r * D;
        vr = v_pages + r * DV;
      }
    }
    float dots[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) dots[h] = 0.f;
    if (valid) dot_row<T>(kr, qs, dots);
    float pr[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float sc = valid ? dots[h] * scale : -INFINITY;
      const float mn = fmaxf(m[h], warp_max(sc));          // finite: the tile holds at least one key
      const float corr = expf(m[h] - mn);                  // exp(-inf) = 0 for the first tile
      const float pv = valid ? expf(sc - mn) : 0.f;
      l[h] = fmaf(l[h], corr, warp_sum(pv));
      m[h] = mn;
      pr[h] = pv;
#pragma unroll
      for (int r = 0; r < DVR; ++r) o[h][r] *= corr;
    }
    const int cnt = min(32, u1 - tile);
    const unsigned long long vaddr = reinterpret_cast<unsigned long long>(vr);
    for (int jj = 0; jj < cnt; ++jj) {
      const T* vj = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, vaddr, jj));
      float vv[DVR];
#pragma unroll
      for (int r = 0; r < DVR; ++r) {
        const int c = lane + 32 * r;
        vv[r] = c < DV ? to_f32<T>(vj[c]) : 0.f;
      }
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float pj = __shfl_sync(0xffffffffu, pr[h], jj);
#pragma unroll
        for (int r = 0; r < DVR; ++r) o[h][r] = fmaf(pj, vv[r], o[h][r]);
      }
    }
  }
  // the warps' partial results meet in shared memory
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    if (lane == 0) { wml[warp][h][0] = m[h]; wml[warp][h][1] = l[h]; }
#pragma unroll
    for (int r = 0; r < DVR; ++r) {
      const int c = lane + 32 * r;
      if (c < DV) wo[warp][h][c] = o[h][r];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < REP * DV; e += blockDim.x) {
    const int h = e / DV, c = e % DV;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ROWS_WARPS; ++w) M = fmaxf(M, wml[w][h][0]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < ROWS_WARPS; ++w) {
      const float mw = wml[w][h][0];
      const float f = mw == -INFINITY ? 0.f : expf(mw - M);
      L = fmaf(wml[w][h][1], f, L);
      O = fmaf(wo[w][h][c], f, O);
    }
    const int head = g * REP + h;
    if (n_splits == 1) {
      const float sk = sink != nullptr ? sink[head] : -INFINITY;
      const float Mx = fmaxf(M, sk);
      const float f = M == -INFINITY ? 0.f : expf(M - Mx);
      const float den = L * f + (sk == -INFINITY ? 0.f : expf(sk - Mx));
      out[((size_t)t * H + head) * DV + c] = from_f32<T>(den > 0.f ? O * f / den : 0.f);
    } else {
      const size_t pi = ((size_t)t * H + head) * n_splits + sp;
      part_o[pi * DV + c] = O;
      if (c == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) pool_attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                const float* __restrict__ sink, const int* __restrict__ tok_slot,
                                                                T* __restrict__ out, int H, int n_splits) {
  const int t = blockIdx.x, head = blockIdx.y;
  if (tok_slot[t] < 0) return;
  const size_t base = ((size_t)t * H + head) * n_splits;
  const float sk = sink != nullptr ? sink[head] : -INFINITY;
  float Mx = sk;
  for (int s = 0; s < n_splits; ++s) Mx = fmaxf(Mx, part_ml[(base + s) * 2]);
  float den = sk == -INFINITY ? 0.f : expf(sk - Mx);
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) den = fmaf(part_ml[(base + s) * 2 + 1], expf(ms - Mx), den);
  }
  for (int c = threadIdx.x; c < DV; c += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) O = fmaf(part_o[(base + s) * DV + c], expf(ms - Mx), O);
    }
    out[((size_t)t * H + head) * DV + c] = from_f32<T>(den > 0.f ? O / den : 0.f);
  }
}

template <typename T>
int prep_launch(const void* proj, int ld, const float* qb, const float* kb, const float* vb, const float* inv_freq,
                const float* inv_freq_lo, int rot, const int* tok_slot, const int* tok_pos, void* q_out, void* k_pages, void* v_pages, const int* page_table,
                int max_pages, int page_size, int n, int H, int G, float eps, int write_kv, cudaStream_t st) {
  const long long items = (long long)n * (H + (write_kv ? 2 * G : 0));
  const long long blocks = (items + PREP_WARPS - 1) / PREP_WARPS;
  if (blocks > 0x7fffffffLL) return DRYFT_ERR_UNSUPPORTED;
  pool_attn_prep_kernel<T><<<(unsigned)blocks, PREP_WARPS * 32, 0, st>>>(
      (const T*)proj, ld, qb, kb, vb, inv_freq, inv_freq_lo, rot, tok_slot, tok_pos, (T*)q_out, (T*)k_pages, (T*)v_pages, page_table, max_pages,
      page_size, n, H, G, eps, write_kv);
  return launch_status();
}

template <typename T>
int rows_launch(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages, int page_size,
                const void* pk, const void* pv, const int* pool_table, int pool_max_pages, const float* sink, const int* tok_slot,
                const int* tok_pos, void* out, float* part_o, float* part_ml, int n, int G, int n_splits, float scale, int size, int P,
                cudaStream_t st) {
  dim3 grid(n, G, n_splits);
  pool_attn_rows_kernel<T><<<grid, ROWS_WARPS * 32, 0, st>>>((const T*)q, (const T*)k_pages, (const T*)v_pages, page_table, max_pages,
                                                            page_size, (const T*)pk, (const T*)pv, pool_table, pool_max_pages, sink,
                                                            tok_slot, tok_pos, (T*)out, part_o, part_ml, G, n_splits, scale, size, P);
  int rc = launch_status();
  if (rc || n_splits == 1) return rc;
  dim3 cgrid(n, G * REP);
  pool_attn_combine_kernel<T><<<cgrid, 128, 0, st>>>(part_o, part_ml, sink, tok_slot, (T*)out, G * REP, n_splits);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_pool_attn_qk_dim() { return D; }
DRYFT_API int dryft_pool_attn_v_dim() { return DV; }
DRYFT_API int dryft_pool_attn_group() { return REP; }

DRYFT_API int dryft_pool_attn_prep(int is_bf16, const void* proj, int ld, const float* qb, const float* kb, const float* vb,
                                   const float* inv_freq, const float* inv_freq_lo, int rot, const int* tok_slot, const int* tok_pos,
                                   void* q_out, void* k_pages, void* v_pages, const int* page_table, int max_pages, int page_size, int n, int H, int G, float eps,
                                   int write_kv, cudaStream_t st) {
  if (n <= 0) return 0;
  if (H != G * REP || rot < 0 || rot % 2 || rot > D || (rot > 0 && inv_freq == nullptr) || (write_kv && page_size < 1))
    return DRYFT_ERR_UNSUPPORTED;
  return is_bf16 ? prep_launch<__nv_bfloat16>(proj, ld, qb, kb, vb, inv_freq, inv_freq_lo, rot, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table,
                                              max_pages, page_size, n, H, G, eps, write_kv, st)
                 : prep_launch<float>(proj, ld, qb, kb, vb, inv_freq, inv_freq_lo, rot, tok_slot, tok_pos, q_out, k_pages, v_pages, page_table,
                                      max_pages, page_size, n, H, G, eps, write_kv, st);
}

DRYFT_API int dryft_pool_attn_prep_tok(int is_bf16, const void* proj, int ld, const float* q_w, const float* k_w, float norm_eps,
                                       const float* inv_freq, const float* inv_freq_lo, int rot, int interleaved, const int* tok_slot,
                                       const int* tok_pos, void* q_out, void* k_pages, void* v_pages, const int* page_table, int max_pages,
                                       int page_size, int n, int H, int G, float eps, int write_kv, cudaStream_t st) {
  if (n <= 0) return 0;
  if (H != G * REP || rot < 0 || rot % 2 || rot > D || (rot > 0 && inv_freq == nullptr) || (write_kv && page_size < 1))
    return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  if (is_bf16)
    pool_attn_prep_tok_kernel<bf><<<n, PREP_TOK_WARPS * 32, 0, st>>>((const bf*)proj, ld, q_w, k_w, norm_eps, inv_freq, inv_freq_lo, rot, interleaved,
                                                                 tok_slot, tok_pos, (bf*)q_out, (bf*)k_pages, (bf*)v_pages, page_table, max_pages,
                                                                 page_size, H, G, eps, write_kv);
  else
    pool_attn_prep_tok_kernel<float><<<n, PREP_TOK_WARPS * 32, 0, st>>>((const float*)proj, ld, q_w, k_w, norm_eps, inv_freq, inv_freq_lo, rot,
                                                                    interleaved, tok_slot, tok_pos, (float*)q_out, (float*)k_pages,
                                                                    (float*)v_pages, page_table, max_pages, page_size, H, G, eps, write_kv);
  return launch_status();
}

DRYFT_API int dryft_pool_attn_blocks(int is_bf16, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
                                     int page_size, void* pk, void* pv, const int* pool_table, int pool_max_pages, const int* tok_slot,
                                     const int* tok_pos, int n, int G, int P, cudaStream_t st) {
  if (n <= 0 || P <= 0) return 0;
  if (G < 1 || G > 65535 || page_size < 1) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(n, G);
  if (is_bf16)
    pool_attn_blocks_kernel<__nv_bfloat16><<<grid, BLOCKS_THREADS, 0, st>>>((const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table,
                                                                 max_pages, page_size, (__nv_bfloat16*)pk, (__nv_bfloat16*)pv, pool_table,
                                                                 pool_max_pages, tok_slot, tok_pos, G, P);
  else
    pool_attn_blocks_kernel<float><<<grid, BLOCKS_THREADS, 0, st>>>((const float*)k_pages, (const float*)v_pages, page_table, max_pages, page_size,
                                                         (float*)pk, (float*)pv, pool_table, pool_max_pages, tok_slot, tok_pos, G, P);
  return launch_status();
}

DRYFT_API int dryft_pool_attn_rows(int is_bf16, const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                                   int max_pages, int page_size, const void* pk, const void* pv, const int* pool_table,
                                   int pool_max_pages, const float* sink, const int* tok_slot, const int* tok_pos, void* out,
                                   float* part_o, float* part_ml, int n, int G, int n_splits, float scale, int size, int P,
                                   cudaStream_t st) {
  if (n <= 0) return 0;
  if (G < 1 || G > 65535 || n_splits < 1 || n_splits > 65535 || size < 1 || page_size < 1 || (P > 0 && pk == nullptr) ||
      (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
    return DRYFT_ERR_UNSUPPORTED;
  return is_bf16 ? rows_launch<__nv_bfloat16>(q, k_pages, v_pages, page_table, max_pages, page_size, pk, pv, pool_table, pool_max_pages,
                                              sink, tok_slot, tok_pos, out, part_o, part_ml, n, G, n_splits, scale, size, P, st)
                 : rows_launch<float>(q, k_pages, v_pages, page_table, max_pages, page_size, pk, pv, pool_table, pool_max_pages, sink,
                                      tok_slot, tok_pos, out, part_o, part_ml, n, G, n_splits, scale, size, P, st);
}
