// Prompt attention over a sliding window with pooled blocks and a sink (bfloat16): packed prompts of unequal lengths over
// the paged cache, flash style.  Compiled per head shape with -DDRYFT_QK_DIM, -DDRYFT_V_DIM, -DDRYFT_GROUP, -DDRYFT_PAGE (64).
//
// Grid (query tiles x query heads).  A tile is up to 64 consecutive query tokens of ONE sequence (tile_tok0 = first
// packed token, tile_rows = how many).  The block's 4 warps own 16 query rows each.  The block walks one list of key
// tiles of 64 rows: first the pages of POOLED rows (row b = the mean key and the mean value of positions bP .. bP+P-1)
// up to the last block any row of the tile sees, then the token pages from the first position the tile's first row sees
// to the tile's last position.  A tile is brought to shared memory with cp.async (two stages), so rows written by this
// very step and by earlier steps are read the same way -- a prompt may be fed in portions.  Q K^T and P V run on
// mma.sync.m16n8k16 (bf16 in, fp32 accumulate); scores, maxima, weights and sums are 32-bit, P is rounded to bfloat16 as
// the second product's operand.  Value rows that no row of the tile may see (positions behind the tile's last, blocks
// behind its last seen block) are filled with zeros on their way in: what a page's last holder left there is never
// multiplied.
// The query at position p sees the tokens j with 0 <= p - j < size and the blocks b with bP + P - 1 <= p - size
// (P = 0: no blocks).  The softmax's denominator also holds exp(sink_head): the running maximum starts at the sink and
// the running sum at one (no sink: -inf and zero).
//
// No block waits on another block; the only waits are cp.async.wait_group and __syncthreads.
#include "common.cuh"
#include <math.h>

#if !defined(DRYFT_QK_DIM) || !defined(DRYFT_V_DIM) || !defined(DRYFT_GROUP) || !defined(DRYFT_PAGE)
#error "compile with -DDRYFT_QK_DIM=.. -DDRYFT_V_DIM=.. -DDRYFT_GROUP=.. -DDRYFT_PAGE=.."
#endif

namespace {
constexpr int DQ = DRYFT_QK_DIM;
constexpr int DV = DRYFT_V_DIM;
constexpr int G = DRYFT_GROUP;
constexpr int KW = DQ;           // elements of a cached key row and of a query row
constexpr int BN = DRYFT_PAGE;   // keys per tile = one cache page
constexpr int BM = 64;           // query rows per block
constexpr int NWARP = 4;
constexpr int THREADS = NWARP * 32;
constexpr int KS = KW + 8;       // padded row strides (elements): conflict-free ldmatrix
constexpr int VS = DV + 8;
constexpr int KSTEPS = DQ / 16;  // k16 steps of Q K^T
constexpr int NT = BN / 8;       // n8 tiles of the scores
constexpr int DT = DV / 8;       // n8 tiles of the output
static_assert(DQ % 16 == 0 && DQ >= 16 && DQ <= 256, "key size 16..256 in steps of 16");
static_assert(DV % 16 == 0 && DV >= 16 && DV <= 256, "value size 16..256 in steps of 16");
static_assert(BN == 64, "the prefill kernel is written for 64-token pages");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {   // bytes < 16: the rest is zeros
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
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

constexpr size_t smem_bytes() { return sizeof(bf16) * ((size_t)KS * (BM + 2 * BN) + (size_t)VS * 2 * BN); }

// rows of V whose key position is >= v_end are zero-filled
__device__ __forceinline__ void load_page(bf16* ks, bf16* vs, const bf16* kp, const bf16* vp, int tid, int key0, int v_end) {
  constexpr int KCPR = KW / 8, VCPR = DV / 8;  // 16-byte chunks per row
  for (int i = tid; i < BN * KCPR; i += THREADS) {
    const int r = i / KCPR, c = i % KCPR;
    cp_async16(ks + r * KS + c * 8, kp + (size_t)r * KW + c * 8, 16);
  }
  for (int i = tid; i < BN * VCPR; i += THREADS) {
    const int r = i / VCPR, c = i % VCPR;
    cp_async16(vs + r * VS + c * 8, vp + (size_t)r * DV + c * 8, key0 + r < v_end ? 16 : 0);
  }
}

__global__ void __launch_bounds__(THREADS) pool_attn_prefill_kernel(
    const bf16* __restrict__ q,                                          // [N, nH, DQ]
    const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,  // [pages, nKV, BN, DQ], [pages, nKV, BN, DV]
    const int* __restrict__ page_table, int max_pages,
    const bf16* __restrict__ pk_pages, const bf16* __restrict__ pv_pages,  // pooled rows, the same layout (null when P == 0)
    const int* __restrict__ pool_table, int pool_max_pages,
    const float* __restrict__ sink,                                      // [nH] or null
    const int* __restrict__ tile_tok0, const int* __restrict__ tile_rows,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    bf16* __restrict__ out,                                              // [N, nH * DV]
    int nH, int nKV, float scale_log2, int size, int P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);   // [BM][KS]
  bf16* ks = qs + BM * KS;                        // [2][BN][KS]
  bf16* vs = ks + 2 * BN * KS;                    // [2][BN][VS]

  // heads run fastest: the host lists the tiles with the most keys first
  const int tile = blockIdx.x / nH, h = blockIdx.x % nH, kvh = h / G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tok0 = tile_tok0[tile], rows = tile_rows[tile];
  const int slot = tok_slot[tok0];
  if (slot < 0 || rows <= 0) return;  // padding tile (uniform for the block)
  const int pos0 = tok_pos[tok0];

  {
    constexpr int CPR = KW / 8;
    for (int i = tid; i < BM * CPR; i += THREADS) {
      const int r = i / CPR, c = i % CPR;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(tok0 + r) * nH + h) * KW + c * 8);
      *reinterpret_cast<uint4*>(qs + r * KS + c * 8) = v;
    }
  }

  const int last_pos = pos0 + rows - 1;
  auto blocks_seen = [&](int p) { return (P > 0 && p - size + 1 >= P) ? (p - size + 1) / P : 0; };
  const int nb_tile = blocks_seen(last_pos);              // pooled rows any row of the tile sees: 0 .. nb_tile - 1
  const int n_pool = (nb_tile + BN - 1) / BN;             // key tiles of pooled rows
  const int pg_first = max(0, pos0 - size + 1) / BN;      // the bound never decreases with the position
  const int pg_last = last_pos / BN;
  const int n_tiles = n_pool + (pg_last - pg_first + 1);
  const int* pt = page_table + (size_t)slot * max_pages;
  const int* ppt = pool_table + (size_t)slot * pool_max_pages;

  // key tile `it` of the list: pooled page `it`, or token page pg_first + (it - n_pool)
  auto load_tile = [&](int it, int stage) {
    bf16* kd = ks + stage * BN * KS;
    bf16* vd = vs + stage * BN * VS;
    if (it < n_pool) {
      const size_t pg = ((size_t)ppt[it] * nKV + kvh) * (size_t)BN;
      load_page(kd, vd, pk_pages + pg * KW, pv_pages + pg * DV, tid, it * BN, nb_tile);
    } else {
      const int page = pg_first + (it - n_pool);
      const size_t pg = ((size_t)pt[page] * nKV + kvh) * (size_t)BN;
      load_page(kd, vd, k_pages + pg * KW, v_pages + pg * DV, tid, page * BN, last_pos + 1);
    }
  };

  load_tile(0, 0);
  cp_async_commit();

  float o_acc[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[j][i] = 0.f;
  // rows g and g+8 of this warp, in log2 units; the sink opens the softmax: its weight is exp2(sink - max), once a row
  const float sink2 = sink != nullptr ? sink[h] * 1.4426950408889634f : -INFINITY;
  float m_run[2] = {sink2, sink2};
  const float l_init = (sink != nullptr && t == 0) ? 1.f : 0.f;   // this thread's share of the row sums
  float l_run[2] = {l_init, l_init};

  // positions of this thread's two rows (rows behind the tile's last are computed like the last and never stored)
  const int qrow0 = min(pos0 + warp * 16 + g, last_pos);
  const int qrow1 = min(pos0 + warp * 16 + g + 8, last_pos);
  const int lo0 = max(0, qrow0 - size + 1), lo1 = max(0, qrow1 - size + 1);
  const int nb0 = blocks_seen(qrow0), nb1 = blocks_seen(qrow1);

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_tiles) {
      load_tile(it + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kst = ks + stage * BN * KS;
    const bf16* vst = vs + stage * BN * VS;
    const bool pooled = it < n_pool;
    const int key0 = pooled ? it * BN : (pg_first + (it - n_pool)) * BN;   // first block, or first position, of the tile
    // what each of the two rows sees of this tile: indices in [vlo, vhi)
    const int vlo0 = pooled ? 0 : lo0, vhi0 = pooled ? nb0 : qrow0 + 1;
    const int vlo1 = pooled ? 0 : lo1, vhi1 = pooled ? nb1 : qrow1 + 1;

    // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      unsigned a0, a1, a2, a3;
      ldsm_x4(a0, a1, a2, a3, qs + (warp * 16 + (lane & 15)) * KS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, kst + (j * 8 + (lane & 7) + (lane >> 4) * 8) * KS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[j], a0, a1, a2, a3, b0, b1);
        mma16816(s[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- mask, online softmax (log2 domain) ----
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kp = key0 + j * 8 + 2 * t + (i & 1);
        const bool vis = (i < 2) ? (kp >= vlo0 && kp < vhi0) : (kp >= vlo1 && kp < vhi1);
        const float v = vis ? s[j][i] * scale_log2 : -INFINITY;
        s[j][i] = v;
        if (i < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
    const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0, mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = exp2f(m_run[0] - mu0), al1 = exp2f(m_run[1] - mu1);  // exp2(-inf) = 0
    m_run[0] = mn0;
    m_run[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      s[j][0] = exp2f(s[j][0] - mu0);
      s[j][1] = exp2f(s[j][1] - mu0);
      s[j][2] = exp2f(s[j][2] - mu1);
      s[j][3] = exp2f(s[j][3] - mu1);
      sum0 += s[j][0] + s[j][1];
      sum1 += s[j][2] + s[j][3];
    }
    l_run[0] = l_run[0] * al0 + sum0;
    l_run[1] = l_run[1] * al1 + sum1;
#pragma unroll
    for (int j = 0; j < DT; ++j) {
      o_acc[j][0] *= al0;
      o_acc[j][1] *= al0;
      o_acc[j][2] *= al1;
      o_acc[j][3] *= al1;
    }
    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < DT; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, vst + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + j * 8 + (lane >> 4) * 8);
        mma16816(o_acc[j], a0, a1, a2, a3, b0, b1);
        mma16816(o_acc[j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();  // both stages may be refilled only after every warp is done with this one
  }

  // ---- divide by the sum (the sink's share is in it), store ----
  float l0 = l_run[0], l1 = l_run[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float f0 = l0 > 0.f ? 1.f / l0 : 0.f, f1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < DT; ++j) {
    const int d = j * 8 + 2 * t;
    if (r0 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + r0) * nH + h) * DV + d) = pack_bf16(o_acc[j][0] * f0, o_acc[j][1] * f0);
    if (r1 < rows)
      *reinterpret_cast<unsigned*>(out + ((size_t)(tok0 + r1) * nH + h) * DV + d) = pack_bf16(o_acc[j][2] * f1, o_acc[j][3] * f1);
  }
}
}  // namespace

DRYFT_API int dryft_pool_attn_prefill_qk_dim() { return DQ; }
DRYFT_API int dryft_pool_attn_prefill_v_dim() { return DV; }

DRYFT_API int dryft_pool_attn_prefill(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
                                      int page_size, const void* pk_pages, const void* pv_pages, const int* pool_table,
                                      int pool_max_pages, const float* sink, const int* tile_tok0, const int* tile_rows,
                                      const int* tok_slot, const int* tok_pos, void* out, int n_tiles, int nH, int nKV, float scale,
                                      int size, int P, cudaStream_t st) {
  if (n_tiles <= 0) return 0;
  if (nH != nKV * G || nH > 65535 || page_size != BN || size < 1 || P < 0) return DRYFT_ERR_UNSUPPORTED;
  if (P > 0 && (pk_pages == nullptr || pv_pages == nullptr || pool_table == nullptr)) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = smem_bytes();
  if (smem > 227 * 1024) return DRYFT_ERR_UNSUPPORTED;
  static bool attr_set = false;  // set by the first (eager) launch, outside any stream capture
  if (smem > 48 * 1024 && !attr_set) {
    cudaError_t e = cudaFuncSetAttribute(pool_attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if ((long long)n_tiles * nH > 2147483647LL) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid((unsigned)(n_tiles * nH));
  pool_attn_prefill_kernel<<<grid, THREADS, smem, st>>>((const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, page_table,
                                                       max_pages, (const bf16*)pk_pages, (const bf16*)pv_pages, pool_table,
                                                       pool_max_pages, sink, tile_tok0, tile_rows, tok_slot, tok_pos, (bf16*)out, nH,
                                                       nKV, scale * 1.4426950408889634f, size, P);
  return launch_status();
}
