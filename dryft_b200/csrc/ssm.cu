// A selective state-space mixer (state-space duality form), all of it in 32-bit.
//
// The mixer's input product leaves, per token, [z | x (heads * dv) | B (groups * N) | C (groups * N) | dt (heads)] as
// floats (row stride ld).  x, B and C ("xbc", CH channels from column x_off) pass a short causal convolution per channel
// and silu; then per head h (its B and C are those of group h / (heads / groups)):
//
//     dt_t = softplus(dt_t + dt_bias_h) ;  S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D_h x_t
//
// with S an N x dv matrix per head.  Per-sequence state, indexed by cache slot and zero when a sequence starts: S
// [slots, heads, N, dv], and the convolution's last taps - 1 inputs `tail` [slots, taps - 1, CH].  A prompt, a piece of
// one and a single token are the same operation.
//
//   ssm_conv    out[t, c] = silu(cb[c] + sum_j cw[c, j] * in[t - (taps - 1) + j, c]) (and, if asked, a bfloat16 copy); inputs before the step's first
//               token come from the tail (zeros before the sequence's start).  A thread a (token, channel).
//   ssm_tail    the tail after the step (run after ssm_conv, which reads the old one).  A thread a (sequence, channel).
//   ssm_scan    one block per (sequence, head, slice of WARPS x COLS value columns); a warp owns COLS columns of S, a lane the
//               rows n = lane, lane + 32, ...; tokens in order, the next token's operands requested before the current
//               token's arithmetic; y_t[p] is a warp sum.
//   chunked     a step of many tokens is cut into chunks of `cht` tokens that run side by side, in three launches: (1) every
//               chunk walks its tokens from a ZERO state and leaves that state and the product of its decays; (2) a prefix
//               over each sequence's chunks, S_start(c+1) = decay(c) S_start(c) + S_own(c), turns these into the state every
//               chunk starts from and leaves the sequence's final state in the slot; (3) every chunk walks its tokens again
//               from its start state and writes y.  Twice the arithmetic, 1 / chunks of the dependent steps.
// Sequences with slot -1 (padding) are skipped.  No block waits on another block.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int CONV_THREADS = 128;
constexpr int SCAN_WARPS = 4;
constexpr int MAX_NR = 16;     // state rows a lane holds at most: N <= 512
constexpr int COLS = 4;        // value columns of the state a warp owns
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ int seq_of(const int* __restrict__ cu_q, int n_seqs, int t) {
  int lo = 0, hi = n_seqs - 1;        // largest b with cu_q[b] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(CONV_THREADS) ssm_conv_kernel(
    const float* __restrict__ proj, int ld, int x_off, int CH, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
    int n_seqs, const float* __restrict__ cw, const float* __restrict__ cb, int taps, const float* __restrict__ tail,
    float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16) {
  const int t = blockIdx.x;
  const int b = seq_of(cu_q, n_seqs, t);
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const int i = t - cu_q[b];          // index of the token within this step's part of its sequence
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c < CH) {
    float acc = cb[c];
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j, src = i - back;
      const float v = src >= 0 ? proj[(size_t)(t - back) * ld + x_off + c]
                               : tail[((size_t)slot * (taps - 1) + (taps - 1 + src)) * CH + c];
      acc = fmaf(cw[(size_t)c * taps + j], v, acc);
    }
    const float v = acc / (1.f + expf(-acc));
    out[(size_t)t * CH + c] = v;
    if (out_bf16 != nullptr) out_bf16[(size_t)t * CH + c] = __float2bfloat16_rn(v);   // the operand of a bfloat16 product behind it
  }
}

__global__ void __launch_bounds__(CONV_THREADS) ssm_tail_kernel(
    const float* __restrict__ proj, int ld, int x_off, int CH, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
    int taps, float* __restrict__ tail) {
  const int b = blockIdx.x;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const int t0 = cu_q[b], q = cu_q[b + 1] - t0;
  if (q <= 0) return;
  float* tl = tail + (size_t)slot * (taps - 1) * CH;
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  if (c < CH) {
    // ascending k: an old entry is read at k + q > k, before it is overwritten
    for (int k = 0; k < taps - 1; ++k) {
      const int src = q - (taps - 1) + k;
      tl[(size_t)k * CH + c] = src >= 0 ? proj[(size_t)(t0 + src) * ld + x_off + c] : tl[(size_t)(k + q) * CH + c];
    }
  }
}

__device__ __forceinline__ float softplusf_(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// chunk `ci` of the step (chunks counted through the sequences in order) -> its sequence and its index within it
__device__ __forceinline__ bool chunk_of(const int* __restrict__ cu_q, int n_seqs, int cht, int ci, int* b_out, int* c_out) {
  int base = 0;
  for (int b = 0; b < n_seqs; ++b) {
    const int nc = (cu_q[b + 1] - cu_q[b] + cht - 1) / cht;
    if (ci < base + nc) { *b_out = b; *c_out = ci - base; return true; }
    base += nc;
  }
  return false;
}

// MODE 0: block x = sequence; its tokens in order from the slot's state, which is left advanced.
// MODE 1: block x = chunk; from a zero state; leaves the chunk's own state in cstate[chunk] and its decays' product in cdec.
// MODE 2: block x = chunk; from the start state in cstate[chunk]; writes y.
// A warp owns COLS neighbouring value columns of S (B_t and C_t, once in registers, serve all of them); a lane the rows
// n = lane, lane + 32, ... (NR of them: N <= 32 NR).
template <int MODE, int NR>
__global__ void __launch_bounds__(SCAN_WARPS * 32) ssm_scan_kernel(
    const float* __restrict__ xbc, int CH, const float* __restrict__ proj, int ld, int dt_off, const float* __restrict__ dt_bias,
    const float* __restrict__ a_log, const float* __restrict__ Dp, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
    int n_seqs, int cht, int heads, int groups, int N, int dv, float* __restrict__ state, float* __restrict__ cstate,
    float* __restrict__ cdec, float* __restrict__ y) {
  const int hd = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = (blockIdx.z * SCAN_WARPS + warp) * COLS;
  int b = blockIdx.x, c = 0;
  if (MODE != 0 && !chunk_of(cu_q, n_seqs, cht, blockIdx.x, &b, &c)) return;
  const int slot = seq_slot[b];
  if (slot < 0 || p0 >= dv) return;
  int t0 = cu_q[b], t1 = cu_q[b + 1];
  if (MODE != 0) { t0 += c * cht; t1 = min(t1, t0 + cht); }
  if (t1 <= t0) return;
  const int inner = heads * dv, g = hd / (heads / groups);
  const int xo = hd * dv + p0, bo = inner + g * N, co = inner + groups * N + g * N;
  const float rate = expf(a_log[hd]), bias = dt_bias[hd], dskip = Dp[hd];
  float* sp = MODE == 0 ? state + (((size_t)slot * heads + hd) * N) * dv + p0
                        : cstate + (((size_t)blockIdx.x * heads + hd) * N) * dv + p0;
  float S[NR][COLS];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int n = lane + 32 * r;
#pragma unroll
    for (int j = 0; j < COLS; ++j) S[r][j] = (MODE != 1 && n < N && p0 + j < dv) ? sp[(size_t)n * dv + j] : 0.f;
  }
  float dprod = 1.f;
  float Bn[NR], Cn[NR], xv[COLS], dtr;
  auto fetch = [&](int t) {
    const float* row = xbc + (size_t)t * CH;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int n = lane + 32 * r;
      Bn[r] = n < N ? row[bo + n] : 0.f;
      Cn[r] = n < N ? row[co + n] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < COLS; ++j) xv[j] = p0 + j < dv ? row[xo + j] : 0.f;
    dtr = proj[(size_t)t * ld + dt_off + hd];
  };
  fetch(t0);
  for (int t = t0; t < t1; ++t) {
    float Bc[NR], Cc[NR], dx[COLS], x[COLS];
#pragma unroll
    for (int r = 0; r < NR; ++r) { Bc[r] = Bn[r]; Cc[r] = Cn[r]; }
    const float dt = softplusf_(dtr + bias);
#pragma unroll
    for (int j = 0; j < COLS; ++j) { x[j] = xv[j]; dx[j] = dt * xv[j]; }
    if (t + 1 < t1) fetch(t + 1);
    const float decay = expf(-rate * dt);
    if (MODE == 1) {
      dprod *= decay;
#pragma unroll
      for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int j = 0; j < COLS; ++j) S[r][j] = fmaf(decay, S[r][j], Bc[r] * dx[j]);
    } else {
      float acc[COLS];
#pragma unroll
      for (int j = 0; j < COLS; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
          S[r][j] = fmaf(decay, S[r][j], Bc[r] * dx[j]);
          acc[j] = fmaf(S[r][j], Cc[r], acc[j]);
        }
      float mine = 0.f, xm = 0.f;      // lane j keeps column j's sum
#pragma unroll
      for (int j = 0; j < COLS; ++j) {
        const float sj = warp_sum(acc[j]);
        if (lane == j) { mine = sj; xm = x[j]; }
      }
      if (lane < COLS && p0 + lane < dv) y[(size_t)t * inner + xo + lane] = fmaf(dskip, xm, mine);
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int n = lane + 32 * r;
#pragma unroll
      for (int j = 0; j < COLS; ++j)
        if (n < N && p0 + j < dv) sp[(size_t)n * dv + j] = S[r][j];
    }
  }
  if (MODE == 1 && p0 == 0 && lane == 0) cdec[(size_t)blockIdx.x * heads + hd] = dprod;
}

// S_start(c + 1) = decay(c) S_start(c) + S_own(c) over a sequence's chunks, from the slot's state; cstate[c] turns from the
// chunk's own state into its start state, and the slot's state becomes the state after the last chunk.
__global__ void __launch_bounds__(256) ssm_chunk_prefix_kernel(const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int cht,
                                                               int heads, int per_head, float* __restrict__ state,
                                                               float* __restrict__ cstate, const float* __restrict__ cdec) {
  const int b = blockIdx.x, hd = blockIdx.y;
  const int e = blockIdx.z * 256 + threadIdx.x;
  const int slot = seq_slot[b];
  if (slot < 0 || e >= per_head) return;
  int base = 0;
  for (int i = 0; i < b; ++i) base += (cu_q[i + 1] - cu_q[i] + cht - 1) / cht;
  const int nc = (cu_q[b + 1] - cu_q[b] + cht - 1) / cht;
  float* sp = state + ((size_t)slot * heads + hd) * per_head + e;
  float carry = *sp;
  const size_t step = (size_t)heads * per_head;
  float* cs = cstate + ((size_t)base * heads + hd) * per_head + e;
  const float* dp = cdec + (size_t)base * heads + hd;
  float own = nc > 0 ? *cs : 0.f, dec = nc > 0 ? *dp : 0.f;
  for (int c = 0; c < nc; ++c) {     // the next chunk's values are requested before this chunk's store
    const float own_next = c + 1 < nc ? cs[step] : 0.f, dec_next = c + 1 < nc ? dp[heads] : 0.f;
    *cs = carry;
    carry = fmaf(dec, carry, own);
    own = own_next;
    dec = dec_next;
    cs += step;
    dp += heads;
  }
  *sp = carry;
}
}  // namespace

DRYFT_API int dryft_ssm_conv(const float* proj, int ld, int x_off, int CH, const int* cu_q, const int* seq_slot, int n_seqs,
                             const float* cw, const float* cb, int taps, float* tail, float* out, void* out_bf16, int n_tokens,
                             cudaStream_t st) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS || CH < 1 || (taps > 1 && tail == nullptr)) return DRYFT_ERR_UNSUPPORTED;
  const dim3 grid_c(n_tokens, (CH + CONV_THREADS - 1) / CONV_THREADS), grid_t(n_seqs, (CH + CONV_THREADS - 1) / CONV_THREADS);
  if (grid_c.y > 65535) return DRYFT_ERR_UNSUPPORTED;
  ssm_conv_kernel<<<grid_c, CONV_THREADS, 0, st>>>(proj, ld, x_off, CH, cu_q, seq_slot, n_seqs, cw, cb, taps, tail, out,
                                                   (__nv_bfloat16*)out_bf16);
  int rc = launch_status();
  if (rc || taps == 1) return rc;
  ssm_tail_kernel<<<grid_t, CONV_THREADS, 0, st>>>(proj, ld, x_off, CH, cu_q, seq_slot, taps, tail);
  return launch_status();
}

namespace {
template <int MODE>
void launch_scan(dim3 grid, cudaStream_t st, const float* xbc, int CH, const float* proj, int ld, int dt_off, const float* dt_bias,
                 const float* a_log, const float* Dp, const int* cu_q, const int* seq_slot, int n_seqs, int cht, int heads, int groups,
                 int N, int dv, float* state, float* cstate, float* cdec, float* y) {
#define DRYFT_SCAN(NR)                                                                                                         \
  ssm_scan_kernel<MODE, NR><<<grid, SCAN_WARPS * 32, 0, st>>>(xbc, CH, proj, ld, dt_off, dt_bias, a_log, Dp, cu_q, seq_slot, n_seqs, \
                                                             cht, heads, groups, N, dv, state, cstate, cdec, y)
  const int nr = (N + 31) / 32;
  if (nr <= 1) DRYFT_SCAN(1);
  else if (nr <= 2) DRYFT_SCAN(2);
  else if (nr <= 4) DRYFT_SCAN(4);
  else if (nr <= 8) DRYFT_SCAN(8);
  else DRYFT_SCAN(16);
#undef DRYFT_SCAN
}
}  // namespace

DRYFT_API int dryft_ssm_scan(const float* xbc, int CH, const float* proj, int ld, int dt_off, const float* dt_bias, const float* a_log,
                             const float* Dp, const int* cu_q, const int* seq_slot, int n_seqs, int heads, int groups, int N, int dv,
                             float* state, float* y, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || N < 1 || N > 32 * MAX_NR || dv < 1 || heads > 65535) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(n_seqs, heads, (dv + SCAN_WARPS * COLS - 1) / (SCAN_WARPS * COLS));
  if (grid.z > 65535) return DRYFT_ERR_UNSUPPORTED;
  launch_scan<0>(grid, st, xbc, CH, proj, ld, dt_off, dt_bias, a_log, Dp, cu_q, seq_slot, n_seqs, 0, heads, groups, N, dv, state, nullptr,
                 nullptr, y);
  return launch_status();
}

// The same recurrence with the step cut into chunks of `cht` tokens (three launches).  `n_chunks` bounds the step's chunks
// (tokens / cht + sequences); cstate [n_chunks, heads, N, dv] and cdec [n_chunks, heads] are scratch.
DRYFT_API int dryft_ssm_scan_chunked(const float* xbc, int CH, const float* proj, int ld, int dt_off, const float* dt_bias,
                                     const float* a_log, const float* Dp, const int* cu_q, const int* seq_slot, int n_seqs, int cht,
                                     int n_chunks, int heads, int groups, int N, int dv, float* state, float* cstate, float* cdec,
                                     float* y, cudaStream_t st) {
  if (n_seqs <= 0 || n_chunks <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || N < 1 || N > 32 * MAX_NR || dv < 1 || heads > 65535 || cht < 1 || n_seqs > 65535)
    return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(n_chunks, heads, (dv + SCAN_WARPS * COLS - 1) / (SCAN_WARPS * COLS));
  const int per_head = N * dv;
  dim3 grid_b(n_seqs, heads, (per_head + 255) / 256);
  if (grid.z > 65535 || grid_b.z > 65535) return DRYFT_ERR_UNSUPPORTED;
  launch_scan<1>(grid, st, xbc, CH, proj, ld, dt_off, dt_bias, a_log, Dp, cu_q, seq_slot, n_seqs, cht, heads, groups, N, dv, state, cstate,
                 cdec, y);
  int rc = launch_status();
  if (rc) return rc;
  ssm_chunk_prefix_kernel<<<grid_b, 256, 0, st>>>(cu_q, seq_slot, cht, heads, per_head, state, cstate, cdec);
  rc = launch_status();
  if (rc) return rc;
  launch_scan<2>(grid, st, xbc, CH, proj, ld, dt_off, dt_bias, a_log, Dp, cu_q, seq_slot, n_seqs, cht, heads, groups, N, dv, state, cstate,
                 cdec, y);
  return launch_status();
}
