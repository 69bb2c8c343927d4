// Mixture of experts for many tokens (bfloat16): the assignments (token, k) sorted by expert, and the experts' two
// products as grouped tensor-core products over the sorted rows.  Everything is decided on the device: no count ever
// reaches the host, so a step with these launches can be captured in a graph.
//
//   moe_sort       counts per expert -> offsets[E+1]; perm[p] = assignment at sorted place p (the order inside an expert
//                  is arbitrary: every row is computed on its own, so no result depends on it); the list of row tiles
//                  (expert, first sorted place) that the products walk, and their number.  One block.
//   moe_grouped<0> act[p, f] = silu(Wg_e[f] . h[token(p)]) * (Wu_e[f] . h[token(p)])   rows gathered through perm
//   moe_grouped<1> y[perm[p], c] = Wd_e[c] . act[p]                                   rows scattered back
// A block of four warps computes 64 or 128 sorted rows of one expert x 128 weight rows (64 columns of gate and of up, or
// 128 columns of down), a warp a quarter of it, with mma.sync.m16n8k16 (bf16 in, fp32 accumulate); operands through a
// cp.async ring of k slices (two stages of 64 by default: measured at 2,048 tokens x 8 of 64 experts of 768 x 2,048,
// 230 TFLOP/s against 211 with three stages and 176 with four of 32 -- the blocks an SM holds matter more than the
// ring's depth), rows and slices that do not exist filled with zeros on their way in.  Inner sizes are multiples of 16.
//
// The grid is sized for the largest number of row tiles there can be (ceil(A/rows per tile) + E); blocks beyond the actual
// number return at once.  No block waits on another block.
#include "common.cuh"
#include <math.h>
#include <stdlib.h>

namespace {
typedef __nv_bfloat16 bf16;
#ifndef DRYFT_MOE_BK
#define DRYFT_MOE_BK 64
#endif
#ifndef DRYFT_MOE_STAGES
#define DRYFT_MOE_STAGES 2
#endif
constexpr int BK = DRYFT_MOE_BK;          // k slice: 32 or 64
constexpr int LDS = BK + 8;               // padded row stride (elements): conflict-free ldmatrix
constexpr int STAGES = DRYFT_MOE_STAGES;
static_assert(BK == 32 || BK == 64, "k slices of 32 or 64");
static_assert(STAGES >= 2 && STAGES <= 6, "two to six stages");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

constexpr int SORT_THREADS = 1024;

__global__ void __launch_bounds__(SORT_THREADS) moe_sort_kernel(
    const int* __restrict__ idx, int n_assign, int E, int BM, int* __restrict__ offsets, int* __restrict__ perm,
    int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ n_tiles) {
  extern __shared__ int sh[];   // counts[E], cursor[E]
  int* counts = sh;
  int* cursor = sh + E;
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) counts[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += SORT_THREADS) atomicAdd(&counts[min(max(idx[a], 0), E - 1)], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = run;
      cursor[e] = run;
      for (int r = 0; r < counts[e]; r += BM) {
        tile_expert[tiles] = e;
        tile_row0[tiles] = run + r;
        ++tiles;
      }
      run += counts[e];
    }
    offsets[E] = run;
    *n_tiles = tiles;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < n_assign; a += SORT_THREADS) perm[atomicAdd(&cursor[min(max(idx[a], 0), E - 1)], 1)] = a;
}

// MODE 0: A rows are h[perm[p] / top], B is W_gu[e] ([2F, K]: gate rows then up rows), out is act[p, F]
// MODE 1: A rows are act[p],           B is W_d[e]  ([C, K]),                        out is y[perm[p], C]
// MODE 2: A rows are h[perm[p] / top], B is W_u[e]  ([F, K]: experts without a gate), out is act[p, F] = max(., 0)^2
// MODE 3: as MODE 0 with the assignment's weight on the expert's INPUT and a clamped activation: with s = in_w[perm[p]],
//         g = min(s * gate, limit), u = clamp(s * up, -limit, limit), act[p, f] = g * sigmoid(alpha * g) * (u + up_off)
// A block of 2 x 2 warps computes BM sorted rows x BN output columns (of gate AND up in mode 0), a warp BM/2 x BN/2.
template <int MODE, int BM, int BN>
__global__ void __launch_bounds__(128) moe_grouped_kernel(
    const bf16* __restrict__ a_in, const bf16* __restrict__ w, const int* __restrict__ offsets, const int* __restrict__ perm,
    const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, const int* __restrict__ n_tiles, int top, int K,
    int n_out, bf16* __restrict__ out, const float* __restrict__ in_w, float limit, float alpha, float up_off) {
  constexpr int NTHREADS = 128;
  constexpr int NMAT = (MODE == 0 || MODE == 3) ? 2 : 1;       // weight matrices multiplied at once (gate and up)
  constexpr int NB = NMAT * BN;                 // weight rows a block reads per k slice
  constexpr int WM = BM / 2, WN = BN / 2;       // a warp's rows and columns
  constexpr int MT = WM / 16, NT = WN / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* as = reinterpret_cast<bf16*>(smem_raw);   // [STAGES][BM][LDS]
  bf16* bs = as + STAGES * BM * LDS;              // [STAGES][NB][LDS]
  __shared__ int row_src[BM];

  const int tile = blockIdx.x;
  if (tile >= *n_tiles) return;
  const int e = tile_expert[tile], p0 = tile_row0[tile];
  const int rows = min(BM, offsets[e + 1] - p0);
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 1, wn = warp & 1;
  const int g = lane >> 2, t = lane & 3;

  for (int r = tid; r < BM; r += NTHREADS) row_src[r] = r < rows ? (MODE != 1 ? perm[p0 + r] / top : p0 + r) : -1;
  __syncthreads();
  const bf16* we = w + (size_t)e * (NMAT * n_out) * K;

  auto load = [&](int stage, int k0) {
    bf16* a_st = as + stage * BM * LDS;
    bf16* b_st = bs + stage * NB * LDS;
    constexpr int CPR = BK / 8;
    for (int i = tid; i < BM * CPR; i += NTHREADS) {
      const int r = i / CPR, c = i % CPR;
      const int src = row_src[r];
      const bool ok = src >= 0 && k0 + c * 8 < K;
      cp_async16(a_st + r * LDS + c * 8, a_in + (ok ? (size_t)src * K + k0 + c * 8 : 0), ok ? 16 : 0);
    }
    for (int i = tid; i < NB * CPR; i += NTHREADS) {
      const int r = i / CPR, c = i % CPR;
      int wr = n0 + (r % BN);
      const bool ok = wr < n_out && k0 + c * 8 < K;
      if ((MODE == 0 || MODE == 3) && r >= BN) wr += n_out;   // the matching up rows
      cp_async16(b_st + r * LDS + c * 8, we + (ok ? (size_t)wr * K + k0 + c * 8 : 0), ok ? 16 : 0);
    }
  };

  float acc[NMAT][MT][NT][4];
#pragma unroll
  for (int m = 0; m < NMAT; ++m)
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[m][i][j][x] = 0.f;

  // a ring of STAGES k slices: slice s + STAGES - 1 is requested while slice s is multiplied; one group is committed per
  // step whether or not it holds a slice, so that the number of groups in flight names the slice that has landed
  const int nk = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load(s, s * BK);
    cp_async_commit();
  }
  for (int ks = 0; ks < nk; ++ks) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();   // slice ks has landed for every thread, and every warp is done with the stage refilled next
    if (ks + STAGES - 1 < nk) load((ks + STAGES - 1) % STAGES, (ks + STAGES - 1) * BK);
    cp_async_commit();
    const bf16* a_st = as + (ks % STAGES) * BM * LDS;
    const bf16* b_st = bs + (ks % STAGES) * NB * LDS;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      unsigned a[MT][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
        ldsm_x4(a[i][0], a[i][1], a[i][2], a[i][3], a_st + (wm * WM + i * 16 + (lane & 15)) * LDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, b_st + (m * BN + wn * WN + j * 8 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            mma16816(acc[m][i][j], a[i][0], a[i][1], a[i][2], a[i][3], b0, b1);
            mma16816(acc[m][i][j + 1], a[i][0], a[i][1], a[i][2], a[i][3], b2, b3);
          }
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const int r0 = wm * WM + i * 16 + g, r1 = r0 + 8;
    size_t o0 = 0, o1 = 0;
    if (MODE != 1) {
      o0 = (size_t)(p0 + r0) * n_out;
      o1 = (size_t)(p0 + r1) * n_out;
    } else {
      if (r0 < rows) o0 = (size_t)perm[p0 + r0] * n_out;
      if (r1 < rows) o1 = (size_t)perm[p0 + r1] * n_out;
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int c = n0 + wn * WN + j * 8 + 2 * t;
      if (c >= n_out) continue;     // n_out is even (a multiple of 16): c + 1 is inside too
      float v0 = acc[0][i][j][0], v1 = acc[0][i][j][1], v2 = acc[0][i][j][2], v3 = acc[0][i][j][3];
      if (MODE == 0) {
        v0 = v0 / (1.f + expf(-v0)) * acc[NMAT - 1][i][j][0];
        v1 = v1 / (1.f + expf(-v1)) * acc[NMAT - 1][i][j][1];
        v2 = v2 / (1.f + expf(-v2)) * acc[NMAT - 1][i][j][2];
        v3 = v3 / (1.f + expf(-v3)) * acc[NMAT - 1][i][j][3];
      }
      if (MODE == 3) {
        const float s0 = r0 < rows ? in_w[perm[p0 + r0]] : 0.f, s1 = r1 < rows ? in_w[perm[p0 + r1]] : 0.f;
        const float sc[4] = {s0, s0, s1, s1};
        float* v[4] = {&v0, &v1, &v2, &v3};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float gq = fminf(*v[q] * sc[q], limit);
          const float uq = fminf(fmaxf(acc[NMAT - 1][i][j][q] * sc[q], -limit), limit);
          *v[q] = gq / (1.f + expf(-alpha * gq)) * (uq + up_off);
        }
      }
      if (MODE == 2) {
        v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f);
        v0 *= v0; v1 *= v1; v2 *= v2; v3 *= v3;
      }
      if (r0 < rows) *reinterpret_cast<unsigned*>(out + o0 + c) = pack_bf16(v0, v1);
      if (r1 < rows) *reinterpret_cast<unsigned*>(out + o1 + c) = pack_bf16(v2, v3);
    }
  }
}

template <int MODE, int BM, int BN>
int gemm_launch(const void* a_in, const void* w, const int* offsets, const int* perm, const int* tile_expert, const int* tile_row0,
                const int* n_tiles, int top, int K, int n_out, void* out, int max_tiles, cudaStream_t st,
                const float* in_w = nullptr, float limit = 0.f, float alpha = 1.f, float up_off = 0.f) {
  static bool attr_set = false;   // set by the first (eager) launch, outside any stream capture
  constexpr size_t smem = sizeof(bf16) * (size_t)LDS * STAGES * (BM + ((MODE == 0 || MODE == 3) ? 2 * BN : BN));
  if (smem > 48 * 1024 && !attr_set) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<MODE, BM, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int n_tiles_n = (n_out + BN - 1) / BN;
  if (n_tiles_n > 65535) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(max_tiles, n_tiles_n);
  moe_grouped_kernel<MODE, BM, BN><<<grid, 128, smem, st>>>((const bf16*)a_in, (const bf16*)w, offsets, perm, tile_expert,
                                                          tile_row0, n_tiles, top, K, n_out, (bf16*)out, in_w, limit, alpha, up_off);
  return launch_status();
}

// rows per tile: 128 once an expert gets about a hundred rows on average (the weights are then re-read from L2 half as
// often), 64 below that (fewer rows of padding per expert)
inline int tile_rows_for(int n_assign, int E) {
  static int forced = -1;   // DRYFT_MOE_TILE_ROWS=64|128 pins the choice (measurements)
  if (forced < 0) {
    const char* v = getenv("DRYFT_MOE_TILE_ROWS");
    forced = v ? atoi(v) : 0;
  }
  if (forced == 64 || forced == 128) return forced;
  return n_assign / E >= 96 ? 128 : 64;
}
}  // namespace

DRYFT_API int dryft_moe_grouped_max_tiles(int n_assign, int E) {
  const int bm = tile_rows_for(n_assign, E);
  return (n_assign + bm - 1) / bm + E;
}

// ints the caller provides in `work`: offsets[E+1] | perm[n_assign] | tile_expert[max_tiles] | tile_row0[max_tiles] | n_tiles[1]
DRYFT_API long long dryft_moe_grouped_work_ints(int n_assign, int E) {
  return (long long)(E + 1) + n_assign + 2LL * dryft_moe_grouped_max_tiles(n_assign, E) + 1;
}

// y[n*top, C] = experts of idx[n, top] applied to h[n, W]; act [n*top, F] is scratch (sorted order)
// `gated`: 1 = w_gate_up is [E, 2F, W] and the activation is silu(gate) * up; 0 = it is [E, F, W] and the activation is max(., 0)^2;
// 2 = [E, 2F, W] with the clamped activation of MODE 3 (in_w [n*top]: each assignment's weight on the expert's input)
DRYFT_API int dryft_moe_grouped(const void* h, const void* w_gate_up, const void* w_down, const int* idx, int n_tokens, int top,
                                int E, int W, int F, void* act, void* y, int* work, int gated, const float* in_w, float limit,
                                float alpha, float up_off, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (top < 1 || E < 1 || W % 16 || F % 16 || W < 16 || F < 16 || gated < 0 || gated > 2 || (gated == 2 && !in_w)) return DRYFT_ERR_UNSUPPORTED;
  const long long n_assign_ll = (long long)n_tokens * top;
  if (n_assign_ll > (1LL << 30) || (size_t)E * 2 * sizeof(int) > 48 * 1024) return DRYFT_ERR_UNSUPPORTED;
  const int n_assign = (int)n_assign_ll;
  const int max_tiles = dryft_moe_grouped_max_tiles(n_assign, E);
  int* offsets = work;
  int* perm = offsets + E + 1;
  int* tile_expert = perm + n_assign;
  int* tile_row0 = tile_expert + max_tiles;
  int* n_tiles = tile_row0 + max_tiles;
  const int bm = tile_rows_for(n_assign, E);
  moe_sort_kernel<<<1, SORT_THREADS, sizeof(int) * 2 * E, st>>>(idx, n_assign, E, bm, offsets, perm, tile_expert, tile_row0, n_tiles);
  int rc = launch_status();
  if (rc) return rc;
  if (bm == 128) {
    rc = gated == 2 ? gemm_launch<3, 128, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st,
                                              in_w, limit, alpha, up_off)
         : gated    ? gemm_launch<0, 128, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st)
                    : gemm_launch<2, 128, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st);
    if (rc) return rc;
    return gemm_launch<1, 128, 128>(act, w_down, offsets, perm, tile_expert, tile_row0, n_tiles, top, F, W, y, max_tiles, st);
  }
  rc = gated == 2 ? gemm_launch<3, 64, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st,
                                           in_w, limit, alpha, up_off)
       : gated    ? gemm_launch<0, 64, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st)
                  : gemm_launch<2, 64, 64>(h, w_gate_up, offsets, perm, tile_expert, tile_row0, n_tiles, top, W, F, act, max_tiles, st);
  if (rc) return rc;
  return gemm_launch<1, 64, 128>(act, w_down, offsets, perm, tile_expert, tile_row0, n_tiles, top, F, W, y, max_tiles, st);
}
