// A selective scan with one decay per (channel, state): the recurrence of a state-space mixer whose state is a vector of N
// numbers per channel.  Everything here is 32-bit; T is the type of the gated output only.
//
// Per token t, channel c (of `inner`) and state n (of N):
//
//     dt_c      = softplus(dtp[t, c] + dt_bias[c])
//     S[c, n]  <- exp(dt_c * A[c, n]) * S[c, n] + dt_c * x[t, c] * B[t, n] ,      A[c, n] = -exp(a_log[c, n])
//     y[t, c]   = sum_n S[c, n] * C[t, n] + D[c] * x[t, c]
//     out[t, c] = T( y[t, c] * silu(z[t, c]) )
//
// x is the convolved and activated input [tokens, inner]; B and C are columns of `low` [tokens, low_ld]; dtp the step sizes
// before bias and softplus [tokens, inner]; z columns of `zrows` [tokens, z_ld] from z_off.  The state S [slots, inner, N]
// is per sequence, indexed by cache slot, zero when a sequence starts, read and left advanced: a prompt, a piece of one and a
// single token are the same operation.
//
//   selscan<MODE 0>   a block per (sequence, group of channels): the step's tokens in order from the slot's state.
//   chunked           a step of many tokens is cut into chunks of `cht` tokens that run side by side in three launches:
//                     <MODE 1> every chunk from a ZERO state, leaving its own state and the sum of its step sizes per
//                     channel (the product of a chunk's decays is exp(A[c, n] * that sum)); selscan_prefix: per sequence,
//                     S_start(k+1) = exp(A * sum_k) S_start(k) + S_own(k), which turns the chunks' own states into their
//                     start states and leaves the sequence's final state in the slot; <MODE 2> every chunk again from its
//                     start state, writing the output.
// A thread owns a channel while its N states fit sixteen registers; beyond that they are spread over `lpc` neighbouring lanes
// (a power of two up to 32), NR neighbouring states a lane.  Tokens go by tiles of eight: the tile's B and C rows are staged
// in shared memory (every channel reads them, 16 bytes at a time), and a thread asks for its channel's step sizes, inputs
// and gates of all eight tokens before it uses the first, forms softplus, dt x, D x and silu(z) once per token and parks
// them in shared memory, so that the loop over the states is a product, an exp2, and three multiply-adds per state.  Sequences with slot -1 (padding) are skipped.
// No block waits on another block.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ float softplus_(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

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

constexpr int TILE = 8;        // tokens whose operands are staged at once

// exp2 of a number that is never positive: one instruction (results below the normal range flush to zero, which is what a
// decay that small is)
__device__ __forceinline__ float exp2_neg(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// A lane owns the NR neighbouring states n = sub * NR .. sub * NR + NR - 1 of its channel (NP = NR * lpc >= N of them exist
// in the staged rows; those beyond N hold zeros there and in A2 and S, so they stay zero without a test).
template <typename T, int MODE, int NR>
__global__ void __launch_bounds__(SCAN_THREADS) selscan_kernel(
    const float* __restrict__ xc, const float* __restrict__ low, int low_ld, int b_off, int c_off, const float* __restrict__ dtp,
    const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ Dp, const float* __restrict__ zrows,
    int z_ld, int z_off, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int n_seqs, int cht, int inner, int N,
    int lpc, float* __restrict__ state, float* __restrict__ cstate, float* __restrict__ cdt, T* __restrict__ out) {
  extern __shared__ __align__(16) float sm[];
  const int NP = NR * lpc;
  float* bc = sm;                               // [TILE][2][NP]: B and C of the tile's tokens, read by every channel
  float* ops = sm + TILE * 2 * NP;              // [4][TILE][SCAN_THREADS]: dt, dt * x, D * x, silu(z) of each thread's channel
  int b = blockIdx.x, ck = 0;
  if (MODE != 0 && !chunk_of(cu_q, n_seqs, cht, blockIdx.x, &b, &ck)) return;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  int t0 = cu_q[b], t1 = cu_q[b + 1];
  if (MODE != 0) { t0 += ck * cht; t1 = min(t1, t0 + cht); }
  if (t1 <= t0) return;
  const int cpb = SCAN_THREADS / lpc;
  const int sub = threadIdx.x & (lpc - 1);
  const int c = blockIdx.y * cpb + threadIdx.x / lpc;
  const bool live = c < inner;
  const int cc = live ? c : inner - 1;       // lanes beyond the last channel follow it (they take part in the shuffles) and store nothing
  const int n0 = sub * NR;

  // A2 = A log2(e): the decay exp(dt A) is one exp2 of a product
  float A2[NR], S[NR];
#pragma unroll
  for (int j = 0; j < NR; ++j) {
    const int n = n0 + j;
    A2[j] = n < N ? -expf(a_log[(size_t)cc * N + n]) * 1.4426950408889634f : 0.f;
    S[j] = 0.f;
    if (n < N) {
      if (MODE == 0) S[j] = state[((size_t)slot * inner + cc) * N + n];
      if (MODE == 2) S[j] = cstate[((size_t)blockIdx.x * inner + cc) * N + n];
    }
  }
  const float bias = dt_bias[cc], dsk = Dp[cc];
  float sum_dt = 0.f;
  float* my = ops + threadIdx.x;

  for (int tb = t0; tb < t1; tb += TILE) {
    const int cnt = min(TILE, t1 - tb);
    __syncthreads();                           // the tile before is used up
    for (int i = threadIdx.x; i < cnt * 2 * NP; i += SCAN_THREADS) {
      const int tt = i / (2 * NP), e = i - tt * 2 * NP, n = e < NP ? e : e - NP;
      bc[i] = n < N ? low[(size_t)(tb + tt) * low_ld + (e < NP ? b_off : c_off) + n] : 0.f;
    }
    // this channel's operands of the tile's tokens: every load is in flight before the first is used
    float dtv[TILE], xv[TILE], zv[TILE];
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
      const size_t t = (size_t)tb + (tt < cnt ? tt : 0);
      dtv[tt] = dtp[t * inner + cc];
      xv[tt] = xc[t * inner + cc];
      zv[tt] = MODE != 1 ? zrows[t * z_ld + z_off + cc] : 0.f;
    }
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
      const float dt = softplus_(dtv[tt] + bias);
      my[(0 * TILE + tt) * SCAN_THREADS] = dt;
      my[(1 * TILE + tt) * SCAN_THREADS] = dt * xv[tt];
      if (MODE != 1) {
        my[(2 * TILE + tt) * SCAN_THREADS] = dsk * xv[tt];
        my[(3 * TILE + tt) * SCAN_THREADS] = zv[tt] / (1.f + expf(-zv[tt]));
      }
    }
    __syncthreads();
#pragma unroll 2
    for (int tt = 0; tt < cnt; ++tt) {
      const float dt = my[(0 * TILE + tt) * SCAN_THREADS], dtx = my[(1 * TILE + tt) * SCAN_THREADS];
      sum_dt += dt;
      const float* Bv = bc + tt * 2 * NP + n0;
      const float* Cv = Bv + NP;
      float acc = 0.f;
      if (NR % 4 == 0) {
#pragma unroll
        for (int j = 0; j < NR; j += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(Bv + j);
          const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
          float cv[4] = {0.f, 0.f, 0.f, 0.f};
          if (MODE != 1) {
            const float4 c4 = *reinterpret_cast<const float4*>(Cv + j);
            cv[0] = c4.x; cv[1] = c4.y; cv[2] = c4.z; cv[3] = c4.w;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            S[j + u] = fmaf(exp2_neg(dt * A2[j + u]), S[j + u], dtx * bb[u]);
            if (MODE != 1) acc = fmaf(S[j + u], cv[u], acc);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
          S[j] = fmaf(exp2_neg(dt * A2[j]), S[j], dtx * Bv[j]);
          if (MODE != 1) acc = fmaf(S[j], Cv[j], acc);
        }
      }
      if (MODE != 1) {
        for (int o = lpc >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (sub == 0 && live)
          out[(size_t)(tb + tt) * inner + c] = from_f32<T>((acc + my[(2 * TILE + tt) * SCAN_THREADS]) * my[(3 * TILE + tt) * SCAN_THREADS]);
      }
    }
  }
  if (!live) return;
  if (MODE == 0) {
#pragma unroll
    for (int j = 0; j < NR; ++j)
      if (n0 + j < N) state[((size_t)slot * inner + c) * N + n0 + j] = S[j];
  }
  if (MODE == 1) {
#pragma unroll
    for (int j = 0; j < NR; ++j)
      if (n0 + j < N) cstate[((size_t)blockIdx.x * inner + c) * N + n0 + j] = S[j];
    if (sub == 0) cdt[(size_t)blockIdx.x * inner + c] = sum_dt;
  }
}

// Per sequence and (channel, state): the chunks' own states become their start states; the slot is left with the final state.
__global__ void __launch_bounds__(256) selscan_prefix_kernel(
    const float* __restrict__ a_log, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int cht, int inner, int N,
    float* __restrict__ state, float* __restrict__ cstate, const float* __restrict__ cdt) {
  const int b = blockIdx.x;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= (size_t)inner * N) return;
  const int c = (int)(e / N);
  int first = 0;
  for (int i = 0; i < b; ++i) first += (cu_q[i + 1] - cu_q[i] + cht - 1) / cht;
  const int nc = (cu_q[b + 1] - cu_q[b] + cht - 1) / cht;
  const float A2 = -expf(a_log[e]) * 1.4426950408889634f;      // as in the scan: the decay is one exp2 of a product
  float S = state[(size_t)slot * inner * N + e];
  for (int k = 0; k < nc; ++k) {
    const size_t at = (size_t)(first + k) * inner * N + e;
    const float own = cstate[at];
    cstate[at] = S;
    S = fmaf(exp2_neg(A2 * cdt[(size_t)(first + k) * inner + c]), S, own);
  }
  state[(size_t)slot * inner * N + e] = S;
}

struct Args {
  const float *xc, *low; int low_ld, b_off, c_off; const float *dtp, *dt_bias, *a_log, *Dp, *zrows; int z_ld, z_off;
  const int *cu_q, *seq_slot; int n_seqs, cht, inner, N, lpc; float *state, *cstate, *cdt; void* out;
};

template <typename T, int MODE, int NR>
int launch_mode(const Args& a, int blocks_x, cudaStream_t st) {
  const int cpb = SCAN_THREADS / a.lpc;
  dim3 grid(blocks_x, (a.inner + cpb - 1) / cpb);
  const size_t smem = sizeof(float) * ((size_t)TILE * 2 * NR * a.lpc + 4 * TILE * SCAN_THREADS);
  selscan_kernel<T, MODE, NR><<<grid, SCAN_THREADS, smem, st>>>(a.xc, a.low, a.low_ld, a.b_off, a.c_off, a.dtp, a.dt_bias, a.a_log, a.Dp,
                                                            a.zrows, a.z_ld, a.z_off, a.cu_q, a.seq_slot, a.n_seqs, a.cht, a.inner, a.N,
                                                            a.lpc, a.state, a.cstate, a.cdt, (T*)a.out);
  return launch_status();
}

template <typename T, int NR>
int launch_all(const Args& a, int n_chunks, cudaStream_t st) {
  if (n_chunks <= 0) return launch_mode<T, 0, NR>(a, a.n_seqs, st);
  int e = launch_mode<T, 1, NR>(a, n_chunks, st);
  if (e) return e;
  const size_t per = (size_t)a.inner * a.N;
  selscan_prefix_kernel<<<dim3(a.n_seqs, (unsigned)((per + 255) / 256)), 256, 0, st>>>(a.a_log, a.cu_q, a.seq_slot, a.cht, a.inner, a.N,
                                                                                      a.state, a.cstate, a.cdt);
  e = launch_status();
  if (e) return e;
  return launch_mode<T, 2, NR>(a, n_chunks, st);
}
}  // namespace

// n_chunks = 0: the tokens of each sequence in order (one launch); else the chunked form (three launches) with scratch
// cstate [n_chunks, inner, N] and cdt [n_chunks, inner], n_chunks at least the number of chunks of `cht` tokens in the step.
DRYFT_API int dryft_selscan(int out_bf16, const float* xc, const float* low, int low_ld, int b_off, int c_off, const float* dtp,
                            const float* dt_bias, const float* a_log, const float* Dp, const float* zrows, int z_ld, int z_off,
                            const int* cu_q, const int* seq_slot, int n_seqs, int cht, int n_chunks, int inner, int N, float* state,
                            float* cstate, float* cdt, void* out, cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  if (inner <= 0 || N <= 0 || N > 512 || (n_chunks > 0 && (cht <= 0 || !cstate || !cdt))) return DRYFT_ERR_UNSUPPORTED;
  int lpc = 1;
  while (lpc < 32 && (N + lpc - 1) / lpc > 16) lpc *= 2;    // a thread a channel while its states fit sixteen registers
  const int nr = (N + lpc - 1) / lpc;
  Args a{xc, low, low_ld, b_off, c_off, dtp, dt_bias, a_log, Dp, zrows, z_ld, z_off, cu_q, seq_slot, n_seqs, cht, inner, N, lpc,
         state, cstate, cdt, out};
  typedef __nv_bfloat16 bf;
#define DRYFT_SELSCAN(NR) return out_bf16 ? launch_all<bf, NR>(a, n_chunks, st) : launch_all<float, NR>(a, n_chunks, st)
  if (nr <= 1) { DRYFT_SELSCAN(1); }
  if (nr <= 2) { DRYFT_SELSCAN(2); }
  if (nr <= 4) { DRYFT_SELSCAN(4); }
  if (nr <= 6) { DRYFT_SELSCAN(6); }
  if (nr <= 8) { DRYFT_SELSCAN(8); }
  if (nr <= 12) { DRYFT_SELSCAN(12); }
  DRYFT_SELSCAN(16);
#undef DRYFT_SELSCAN
}
