// Attention whose keys and values are low-rank latents: the cache holds, per token, one row
//     [ c (kv_rank entries, normalised) | k_rot (rot_dim entries, rotated) ]
// shared by all heads, and the per-head key and value matrices are folded into the query and the output:
//     score(i, j) = ( (W_uk,h^T q_plain,i) . c_j + q_rot,i . k_rot,j ) * scale          o_lat,i = sum_j p(i, j) c_j
// (the caller multiplies q_plain by W_uk,h^T before and o_lat by W_uv,h after, as matrix products).
//
// latent_prep        per token, from one projection row [.. dq (q_rank) .. dkv (kv_rank + rot_dim) ..]:
//                      cq = T( rmsnorm(dq) * w_q )                        -> the query up-projection's input
//                      c  = rmsnorm(dkv[:kv_rank]) * w_kv ; k_rot = rotate(dkv[kv_rank:]) at the token's position
//                      cache row (slot, position) <- T([c | k_rot])
// latent_attn_rows   one block per (query token, group of 16 heads, split of the keys), four heads a warp.  Keys
//                    position-window+1 .. position (all keys from 0 if window is 0) are staged 32 at a time in shared memory
//                    as floats (16-byte loads, several in flight per thread); a lane takes a key for the scores (softmax
//                    running maximum and sum in 32-bit) and a slice of the latent for the weighted sum.  A step of few
//                    tokens splits each token's keys over several blocks, joined by latent_combine.  The query's rotated part is rotated here.  Heads-major input and output:
//                    q_lat [H, N, kv_rank] (32-bit), q [N, H, q_stride] with the rotated part at q_rot_off,
//                    o_lat [H, N, kv_rank].
// head_gate          out[n, h, :] = T( o[h, n, :] * sigmoid(gate_logit[n, h]) )
//
// Rotation: pairs (2i, 2i+1) when `interleaved`, else (i, i + R/2); angle = position * inv_freq[i] (sincos_split below).
// Norms, angles, scores, softmax and the weighted sum are 32-bit whatever the cache type T.  Sizes are runtime arguments
// (kv_rank up to 512).  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int PREP_THREADS = 256;
constexpr int HW = 4;          // heads a warp of latent_attn_rows
constexpr int WPB = 4;         // warps a block
constexpr int HPB = HW * WPB;  // heads a block
constexpr int KT = 32;         // keys per staged tile

// sin and cos of  pos * (f_hi + f_lo)  for a rotary position: the product is formed in 32-bit, and what its rounding
// drops (recovered exactly with one fused multiply-add) plus the low half of the frequency are applied as a first-order
// turn, so the angle is as good as the frequency pair instead of losing one part in 2^24 of a large angle.  f_lo = 0 gives
// the plain 32-bit angle to within that correction.
__device__ __forceinline__ void sincos_split(float pos, float f_hi, float f_lo, float* sn, float* cs) {
  const float a = pos * f_hi;
  const float e = fmaf(pos, f_hi, -a) + pos * f_lo;
  float s, c;
  sincosf(a, &s, &c);
  *sn = fmaf(e, c, s);
  *cs = fmaf(-e, s, c);
}


__device__ __forceinline__ float rotated(const float* v, int d, int R, bool interleaved, float pos, const float* inv_freq,
                                         const float* inv_freq_lo) {
  // entry d (< R) of v after the rotation
  int j, partner;
  bool first;
  if (interleaved) { j = d >> 1; first = !(d & 1); partner = first ? d + 1 : d - 1; }
  else { const int half = R >> 1; first = d < half; j = first ? d : d - half; partner = first ? d + half : d - half; }
  float sn, cs;
  sincos_split(pos, inv_freq[j], inv_freq_lo ? inv_freq_lo[j] : 0.f, &sn, &cs);
  return first ? v[d] * cs - v[partner] * sn : v[d] * cs + v[partner] * sn;
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) latent_prep_kernel(
    const T* __restrict__ proj, int ld, int dq_off, int q_rank, const float* __restrict__ w_q, int dkv_off, int kv_rank,
    int rot, const float* __restrict__ w_kv, float eps, const float* __restrict__ inv_freq,
    const float* __restrict__ inv_freq_lo, int interleaved, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, T* __restrict__ cq, T* __restrict__ k_pages,
    const int* __restrict__ page_table, int max_pages, int page_size, T* __restrict__ c_out) {
  extern __shared__ __align__(16) float buf[];   // [rot]
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const int slot = tok_slot[n];
  const T* row = proj + (size_t)n * ld;
  if (q_rank > 0) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += PREP_THREADS) { const float v = to_f32<T>(row[dq_off + c]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += PREP_THREADS)
      cq[(size_t)n * q_rank + c] = from_f32<T>(to_f32<T>(row[dq_off + c]) * inv * w_q[c]);
  }
  if (slot < 0 || !k_pages) return;
  const int pos = tok_pos[n];
  const int page = page_table[(size_t)slot * max_pages + pos / page_size];
  T* dst = k_pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot);
  float ss = 0.f;
  for (int c = threadIdx.x; c < kv_rank; c += PREP_THREADS) { const float v = to_f32<T>(row[dkv_off + c]); ss = fmaf(v, v, ss); }
  for (int c = threadIdx.x; c < rot; c += PREP_THREADS) buf[c] = to_f32<T>(row[dkv_off + kv_rank + c]);
  ss = block_sum(ss, scratch);   // also orders buf
  const float inv = 1.f / sqrtf(ss / (float)kv_rank + eps);
  for (int c = threadIdx.x; c < kv_rank; c += PREP_THREADS) {
    const T v = from_f32<T>(to_f32<T>(row[dkv_off + c]) * inv * w_kv[c]);
    dst[c] = v;
    if (c_out) c_out[(size_t)n * kv_rank + c] = v;   // the latent as rows too, for a step that makes keys and values from it
  }
  for (int c = threadIdx.x; c < rot; c += PREP_THREADS)
    dst[kv_rank + c] = from_f32<T>(rotated(buf, c, rot, interleaved != 0, (float)pos, inv_freq, inv_freq_lo));
}

// Floats per staged key row: a multiple of four (16-byte reads) whose quarter is odd, so that the rows of a warp's 32
// keys fall on different banks.
__host__ __device__ __forceinline__ int tile_row(int Dk) {
  int d = (Dk + 3) & ~3;
  if (((d >> 2) & 1) == 0) d += 4;
  return d;
}

// 16 bytes of a cached row as floats (8 bfloat16 or 4 float)
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& raw, float* out) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y); out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& raw, float* out) {
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};

// One block per (query token, group of HPB heads, split of the visible keys); a warp takes HW heads, so that a key's
// staged row is read from shared memory once for all of them (16 bytes at a time where the row length allows): the loop is
// bound by shared-memory reads, and this quarters them.  With one split the result goes to o_lat; with several, each block
// leaves (max, sum, unnormalised weighted sum) in `part` and latent_combine joins them.
template <typename T, int NR>
__global__ void __launch_bounds__(WPB * 32) latent_attn_rows_kernel(
    const float* __restrict__ q_lat, const T* __restrict__ q, int q_stride, int q_rot_off, const T* __restrict__ k_pages,
    const int* __restrict__ page_table, int max_pages, int page_size, const int* __restrict__ tok_slot,
    const int* __restrict__ tok_pos, const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo,
    int interleaved, T* __restrict__ o_lat, float* __restrict__ part, int n_splits, int n_tokens, int H, int kv_rank, int rot,
    float scale, int window, const float* __restrict__ sink) {
  extern __shared__ __align__(16) float sm[];
  const int Dk = kv_rank + rot, Dq = (Dk + 3) & ~3, Dp = tile_row(Dk);
  float* tile = sm;                                  // [KT][Dp]
  float* qs_all = tile + (size_t)KT * Dp;            // [HPB][Dq]
  float* raw = qs_all + (size_t)HPB * Dq;            // [HPB][rot]
  const int n = blockIdx.x, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hd0 = blockIdx.y * HPB + warp * HW;      // this warp's first head
  const int slot = tok_slot[n];
  if (slot < 0) return;
  const int pos = tok_pos[n];
  const int lo_all = window > 0 ? max(0, pos - window + 1) : 0;
  // this split's share of the key tiles (whole tiles, in order)
  const int tiles_all = (pos - lo_all) / KT + 1;
  const int per_split = (tiles_all + n_splits - 1) / n_splits;
  const int lo = lo_all + split * per_split * KT;
  const int hi = min(pos, lo + per_split * KT - 1);   // last key of this split
  const int nh = max(0, min(HW, H - hd0));            // live heads of this warp
  float* qs = qs_all + (size_t)warp * HW * Dq;
  for (int i = 0; i < HW; ++i) {
    float* qi = qs + (size_t)i * Dq;
    if (i >= nh) {   // a head that does not exist: zeros, so that its sums stay finite
      for (int d = lane; d < Dq; d += 32) qi[d] = 0.f;
      continue;
    }
    const float* ql = q_lat + ((size_t)(hd0 + i) * n_tokens + n) * kv_rank;
    for (int d = lane; d < kv_rank; d += 32) qi[d] = ql[d] * scale;
    const T* qr = q + ((size_t)n * H + hd0 + i) * q_stride + q_rot_off;
    float* rw = raw + (size_t)(warp * HW + i) * rot;
    for (int d = lane; d < rot; d += 32) rw[d] = to_f32<T>(qr[d]);
    __syncwarp();
    for (int d = lane; d < rot; d += 32) qi[kv_rank + d] = rotated(rw, d, rot, interleaved != 0, (float)pos, inv_freq, inv_freq_lo) * scale;
    for (int d = Dk + lane; d < Dq; d += 32) qi[d] = 0.f;
  }
  float m[HW], l[HW], acc[HW][NR];
#pragma unroll
  for (int i = 0; i < HW; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[i][r] = 0.f;
  }
  const int* pt = page_table + (size_t)slot * max_pages;
  constexpr int VN = Vec16<T>::N;
  const bool vec_ok = (Dk % VN) == 0;     // rows start on 16-byte boundaries
  const bool quad_ok = (Dk & 3) == 0;     // 16-byte reads of the staged rows
  const int vpr = Dk / VN;
  for (int j0 = lo; j0 <= hi; j0 += KT) {
    const int cnt = min(KT, hi - j0 + 1);
    __syncthreads();   // the tile before is used up (and, the first time, qs is written)
    if (vec_ok) {
      // every thread asks for four 16-byte pieces before it unpacks the first: the loads' round trips overlap
      const int total = cnt * vpr;
      for (int base = threadIdx.x; base < total; base += 4 * WPB * 32) {
        uint4 v[4];
        int at[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = base + u * WPB * 32;
          at[u] = -1;
          if (idx < total) {
            const int kk = idx / vpr, c = idx - kk * vpr, j = j0 + kk;
            const T* src = k_pages + ((size_t)pt[j / page_size] * page_size + j % page_size) * Dk;
            v[u] = __ldg(reinterpret_cast<const uint4*>(src) + c);
            at[u] = kk * Dp + c * VN;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (at[u] >= 0) {
            float f[VN];
            Vec16<T>::unpack(v[u], f);
#pragma unroll
            for (int e = 0; e < VN; e += 4) *reinterpret_cast<float4*>(tile + at[u] + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
          }
        }
      }
    } else {
      for (int kk = warp; kk < cnt; kk += WPB) {
        const int j = j0 + kk;
        const T* src = k_pages + ((size_t)pt[j / page_size] * page_size + j % page_size) * Dk;
        for (int d = lane; d < Dk; d += 32) tile[kk * Dp + d] = to_f32<T>(src[d]);
      }
    }
    __syncthreads();
    if (nh == 0) continue;
    float s[HW];
#pragma unroll
    for (int i = 0; i < HW; ++i) s[i] = 0.f;
    if (lane < cnt) {
      const float* kr = tile + lane * Dp;
      if (quad_ok) {
        for (int d = 0; d < Dk; d += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
          for (int i = 0; i < HW; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + (size_t)i * Dq + d);
            s[i] = fmaf(q4.x, k4.x, fmaf(q4.y, k4.y, fmaf(q4.z, k4.z, fmaf(q4.w, k4.w, s[i]))));
          }
        }
      } else {
        for (int d = 0; d < Dk; ++d) {
          const float kv = kr[d];
#pragma unroll
          for (int i = 0; i < HW; ++i) s[i] = fmaf(qs[(size_t)i * Dq + d], kv, s[i]);
        }
      }
    }
    float p[HW];
#pragma unroll
    for (int i = 0; i < HW; ++i) {
      const float si = lane < cnt ? s[i] : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(si));
      p[i] = lane < cnt ? expf(si - m_new) : 0.f;
      const float corr = expf(m[i] - m_new);   // 0 the first time (m = -inf)
      l[i] = l[i] * corr + warp_sum(p[i]);
#pragma unroll
      for (int r = 0; r < NR; ++r) acc[i][r] *= corr;
      m[i] = m_new;
    }
    for (int kk = 0; kk < cnt; ++kk) {
      const float* kr = tile + kk * Dp;
      float cv[NR];
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int d = lane + 32 * r;
        cv[r] = d < kv_rank ? kr[d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < HW; ++i) {
        const float pk = __shfl_sync(0xffffffffu, p[i], kk);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[i][r] = fmaf(pk, cv[r], acc[i][r]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < HW; ++i) {
    if (i >= nh) break;
    const int hd = hd0 + i;
    if (n_splits > 1) {   // a split without keys leaves max = -inf, sum = 0
      float* dst = part + (((size_t)n * H + hd) * n_splits + split) * (kv_rank + 2);
      if (lane == 0) { dst[0] = m[i]; dst[1] = l[i]; }
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int d = lane + 32 * r;
        if (d < kv_rank) dst[2 + d] = acc[i][r];
      }
    } else {
      T* dst = o_lat + ((size_t)hd * n_tokens + n) * kv_rank;
      float li = l[i], keep = 1.f;
      if (sink != nullptr) {   // a number in the denominator without key or value: it is not scaled and counts once
        const float sk = sink[hd], m_all = fmaxf(m[i], sk);
        keep = expf(m[i] - m_all);
        li = li * keep + expf(sk - m_all);
      }
      const float inv = keep / li;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int d = lane + 32 * r;
        if (d < kv_rank) dst[d] = from_f32<T>(acc[i][r] * inv);
      }
    }
  }
}

// o_lat[h, n, :] from the splits' (max, sum, weighted sum): one block per (token, head).  The first warp turns the splits'
// maxima and sums into one weight per split (up to MAX_SPLITS of them); every thread then sums its latent entries.
constexpr int MAX_SPLITS = 64;

template <typename T>
__global__ void latent_combine_kernel(const float* __restrict__ part, const int* __restrict__ tok_slot, T* __restrict__ o_lat,
                                      int n_splits, int n_tokens, int H, int kv_rank, const float* __restrict__ sink) {
  __shared__ float w[MAX_SPLITS];
  const int n = blockIdx.x, hd = blockIdx.y;
  if (tok_slot[n] < 0) return;
  const size_t stride = (size_t)kv_rank + 2;
  const float* src = part + ((size_t)n * H + hd) * n_splits * stride;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float ms[MAX_SPLITS / 32], ls[MAX_SPLITS / 32];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < MAX_SPLITS / 32; ++u) {
      const int sidx = lane + 32 * u;
      ms[u] = sidx < n_splits ? src[sidx * stride] : -INFINITY;
      ls[u] = sidx < n_splits ? src[sidx * stride + 1] : 0.f;
      m = fmaxf(m, ms[u]);
    }
    m = warp_max(m);
    if (sink != nullptr) m = fmaxf(m, sink[hd]);
    float l = 0.f;
#pragma unroll
    for (int u = 0; u < MAX_SPLITS / 32; ++u) {
      ms[u] = ms[u] > -INFINITY ? expf(ms[u] - m) : 0.f;   // a split without keys weighs nothing
      l = fmaf(ls[u], ms[u], l);
    }
    l = warp_sum(l);
    if (sink != nullptr) l += expf(sink[hd] - m);           // the sink joins the denominator once, after the splits
#pragma unroll
    for (int u = 0; u < MAX_SPLITS / 32; ++u)
      if (lane + 32 * u < n_splits) w[lane + 32 * u] = ms[u] / l;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    float a = 0.f;
#pragma unroll 8
    for (int sidx = 0; sidx < n_splits; ++sidx) a = fmaf(src[sidx * stride + 2 + d], w[sidx], a);
    o_lat[((size_t)hd * n_tokens + n) * kv_rank + d] = from_f32<T>(a);
  }
}

template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_ld, T* __restrict__ out,
                                 int n_tokens, int H, int vdim) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * H * vdim) return;
  const int v = (int)(i % vdim);
  const int hd = (int)((i / vdim) % H);
  const size_t n = i / ((size_t)vdim * H);
  float val = o[((size_t)hd * n_tokens + n) * vdim + v];
  if (gate) {
    const float g = to_f32<T>(gate[n * gate_ld + hd]);
    val *= 1.f / (1.f + expf(-g));
  }
  out[i] = from_f32<T>(val);
}

// ---------------------------------------------------------------------------------------------------------------------
// A step in which every sequence starts at position 0 holds all its keys itself: the per-head keys and values are then made
// from the step's latents by one matrix product and handed, in pages of the step's own, to the library's tensor-core prompt
// attention (the ordinary kind: per-head keys [unrotated | rotated part] and values).
//
// latent_scratch_table   table[slot_b][p] = (pages of the sequences before b) + p   for the step's sequences
// latent_expand_store    per token: q_out[n, h] = [q_plain | rotate(q_rot)], key page row = [k_plain,h | rotate(k_rot)],
//                        value page row = [v_h | zeros]  (all of the head size `hd` >= the value size)
// head_gate_rows         out[n, h*V + v] = T( o[n, h, v] * sigmoid(gate_logit[n, h]) )   for o [n, H, hd]
__global__ void latent_scratch_table_kernel(const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int n_seqs,
                                            int* __restrict__ table, int max_pages, int page_size) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_seqs) return;
  const int slot = seq_slot[b];
  if (slot < 0) return;
  int base = 0;
  for (int bb = 0; bb < b; ++bb) base += (cu_q[bb + 1] - cu_q[bb] + page_size - 1) / page_size;
  const int np = (cu_q[b + 1] - cu_q[b] + page_size - 1) / page_size;
  for (int p = 0; p < np && p < max_pages; ++p) table[(size_t)slot * max_pages + p] = base + p;
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS) latent_expand_store_kernel(
    const T* __restrict__ q, const T* __restrict__ kv, int kv_ld, int v_off, const T* __restrict__ proj, int ld, int krot_off,
    const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, int interleaved,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, const int* __restrict__ table, int max_pages,
    int page_size, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages, int H, int dim, int rot, int vdim) {
  extern __shared__ __align__(16) float buf[];   // [rot] the shared key part, rotated; then [H][rot] raw query parts
  const int n = blockIdx.x;
  const int slot = tok_slot[n];
  if (slot < 0) return;
  const int pos = tok_pos[n], hd = dim + rot;
  float* krot = buf;
  float* qraw = buf + rot;
  for (int c = threadIdx.x; c < rot; c += PREP_THREADS) krot[c] = to_f32<T>(proj[(size_t)n * ld + krot_off + c]);
  for (int i = threadIdx.x; i < H * rot; i += PREP_THREADS)
    qraw[i] = to_f32<T>(q[((size_t)n * H + i / rot) * hd + dim + i % rot]);
  __syncthreads();
  const size_t page = (size_t)table[(size_t)slot * max_pages + pos / page_size];
  for (int i = threadIdx.x; i < H * hd; i += PREP_THREADS) {
    const int h = i / hd, d = i % hd;
    const size_t at = ((page * H + h) * page_size + pos % page_size) * hd + d;
    T qv, kvv;
    if (d < dim) {
      qv = q[((size_t)n * H + h) * hd + d];
      kvv = kv[(size_t)n * kv_ld + h * dim + d];
    } else {
      qv = from_f32<T>(rotated(qraw + h * rot, d - dim, rot, interleaved != 0, (float)pos, inv_freq, inv_freq_lo));
      kvv = from_f32<T>(rotated(krot, d - dim, rot, interleaved != 0, (float)pos, inv_freq, inv_freq_lo));
    }
    q_out[((size_t)n * H + h) * hd + d] = qv;
    k_pages[at] = kvv;
    v_pages[at] = d < vdim ? kv[(size_t)n * kv_ld + v_off + h * vdim + d] : from_f32<T>(0.f);
  }
}

template <typename T>
__global__ void head_gate_rows_kernel(const T* __restrict__ o, int hd, const T* __restrict__ gate, int gate_ld,
                                      T* __restrict__ out, int n_tokens, int H, int vdim) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * H * vdim) return;
  const int v = (int)(i % vdim);
  const int h = (int)((i / vdim) % H);
  const size_t n = i / ((size_t)vdim * H);
  float val = to_f32<T>(o[(n * H + h) * hd + v]);
  if (gate) val *= 1.f / (1.f + expf(-to_f32<T>(gate[n * gate_ld + h])));
  out[i] = from_f32<T>(val);
}

// The per-head key and value matrices folded into the query and the output, for steps of few tokens and for the 32-bit
// path (sums in a fixed order, so a row's result does not depend on its company):
//   latent_fold_q     q_lat[h, n, r] = sum_d q[n, h, d] * w_k[h, d, r]                      (32-bit result)
//   latent_unfold_o   out[n, h*V + v] = T( sigmoid(gate[n, h]) * sum_r o_lat[h, n, r] * w_v[h, r, v] )
// One block per (token, head); a thread per output entry reads along the matrices' rows.
template <typename T>
__global__ void latent_fold_q_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ w, float* __restrict__ q_lat,
                                     int n_tokens, int H, int dim, int kv_rank) {
  extern __shared__ __align__(16) float vin[];
  const int n = blockIdx.x, h = blockIdx.y;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) vin[d] = to_f32<T>(q[((size_t)n * H + h) * q_stride + d]);
  __syncthreads();
  const T* wh = w + (size_t)h * dim * kv_rank;
  for (int r = threadIdx.x; r < kv_rank; r += blockDim.x) {
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < dim; ++d) acc = fmaf(vin[d], to_f32<T>(wh[(size_t)d * kv_rank + r]), acc);
    q_lat[((size_t)h * n_tokens + n) * kv_rank + r] = acc;
  }
}

template <typename T>
__global__ void latent_unfold_o_kernel(const T* __restrict__ o_lat, const T* __restrict__ w, const T* __restrict__ gate,
                                       int gate_ld, T* __restrict__ out, int n_tokens, int H, int kv_rank, int vdim) {
  extern __shared__ __align__(16) float vin[];
  const int n = blockIdx.x, h = blockIdx.y;
  for (int r = threadIdx.x; r < kv_rank; r += blockDim.x) vin[r] = to_f32<T>(o_lat[((size_t)h * n_tokens + n) * kv_rank + r]);
  __syncthreads();
  const float g = gate ? 1.f / (1.f + expf(-to_f32<T>(gate[(size_t)n * gate_ld + h]))) : 1.f;
  const T* wh = w + (size_t)h * kv_rank * vdim;
  for (int v = threadIdx.x; v < vdim; v += blockDim.x) {
    float acc = 0.f;
#pragma unroll 8
    for (int r = 0; r < kv_rank; ++r) acc = fmaf(vin[r], to_f32<T>(wh[(size_t)r * vdim + v]), acc);
    out[((size_t)n * H + h) * vdim + v] = from_f32<T>(acc * g);
  }
}

template <typename K> int opt_in(K kernel, size_t bytes) {
  if (bytes > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

template <typename T, int NR>
int launch_rows(const float* q_lat, const void* q, int q_stride, int q_rot_off, const void* k_pages, const int* page_table,
                int max_pages, int page_size, const int* tok_slot, const int* tok_pos, const float* inv_freq,
                const float* inv_freq_lo, int interleaved, void* o_lat, float* part, int n_splits, int n_tokens, int H, int kv_rank,
                int rot, float scale, int window, const float* sink, cudaStream_t st) {
  const int Dk = kv_rank + rot;
  const size_t smem = sizeof(float) * ((size_t)KT * tile_row(Dk) + (size_t)HPB * ((Dk + 3) & ~3) + (size_t)HPB * rot);
  int rc = opt_in(latent_attn_rows_kernel<T, NR>, smem);
  if (rc) return rc;
  dim3 grid(n_tokens, (H + HPB - 1) / HPB, n_splits);
  latent_attn_rows_kernel<T, NR><<<grid, WPB * 32, smem, st>>>(q_lat, (const T*)q, q_stride, q_rot_off, (const T*)k_pages, page_table,
                                                               max_pages, page_size, tok_slot, tok_pos, inv_freq, inv_freq_lo,
                                                               interleaved, (T*)o_lat, part, n_splits, n_tokens, H, kv_rank, rot, scale,
                                                               window, sink);
  int e = launch_status();
  if (e || n_splits <= 1) return e;
  latent_combine_kernel<T><<<dim3(n_tokens, H), 128, 0, st>>>(part, tok_slot, (T*)o_lat, n_splits, n_tokens, H, kv_rank, sink);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_latent_prep(int is_bf16, const void* proj, int ld, int dq_off, int q_rank, const float* w_q, int dkv_off,
                                int kv_rank, int rot, const float* w_kv, float eps, const float* inv_freq,
                                const float* inv_freq_lo, int interleaved, const int* tok_slot, const int* tok_pos, void* cq,
                                void* k_pages, const int* page_table, int max_pages, int page_size, void* c_out, int n,
                                cudaStream_t st) {
  if (n <= 0) return 0;
  if (kv_rank <= 0 || rot < 0 || (rot & 1)) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * (size_t)(rot > 0 ? rot : 1);
  if (smem > 48 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16)
    latent_prep_kernel<bf><<<n, PREP_THREADS, smem, st>>>((const bf*)proj, ld, dq_off, q_rank, w_q, dkv_off, kv_rank, rot, w_kv, eps,
                                                          inv_freq, inv_freq_lo, interleaved, tok_slot, tok_pos, (bf*)cq, (bf*)k_pages, page_table,
                                                          max_pages, page_size, (bf*)c_out);
  else
    latent_prep_kernel<float><<<n, PREP_THREADS, smem, st>>>((const float*)proj, ld, dq_off, q_rank, w_q, dkv_off, kv_rank, rot, w_kv,
                                                             eps, inv_freq, inv_freq_lo, interleaved, tok_slot, tok_pos, (float*)cq, (float*)k_pages,
                                                             page_table, max_pages, page_size, (float*)c_out);
  return launch_status();
}

DRYFT_API int dryft_latent_attn_rows(int is_bf16, const float* q_lat, const void* q, int q_stride, int q_rot_off,
                                     const void* k_pages, const int* page_table, int max_pages, int page_size,
                                     const int* tok_slot, const int* tok_pos, const float* inv_freq, const float* inv_freq_lo,
                                     int interleaved, void* o_lat, float* part, int n_splits, int n_tokens, int H, int kv_rank,
                                     int rot, float scale, int window, const float* sink, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (kv_rank <= 0 || kv_rank > 512 || rot < 0 || (rot & 1) || H <= 0 || (H + HPB - 1) / HPB > 65535) return DRYFT_ERR_UNSUPPORTED;
  if (n_splits < 1 || n_splits > MAX_SPLITS || (n_splits > 1 && !part)) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int nr = (kv_rank + 31) / 32;
#define DRYFT_LATENT_ROWS(NR)                                                                                                      \
  return is_bf16 ? launch_rows<bf, NR>(q_lat, q, q_stride, q_rot_off, k_pages, page_table, max_pages, page_size, tok_slot, tok_pos,  \
                                       inv_freq, inv_freq_lo, interleaved, o_lat, part, n_splits, n_tokens, H, kv_rank, rot, scale, window, sink, st) \
                 : launch_rows<float, NR>(q_lat, q, q_stride, q_rot_off, k_pages, page_table, max_pages, page_size, tok_slot,      \
                                          tok_pos, inv_freq, inv_freq_lo, interleaved, o_lat, part, n_splits, n_tokens, H, kv_rank, rot, scale, \
                                          window, sink, st)
  if (nr <= 1) { DRYFT_LATENT_ROWS(1); }
  if (nr <= 2) { DRYFT_LATENT_ROWS(2); }
  if (nr <= 4) { DRYFT_LATENT_ROWS(4); }
  if (nr <= 8) { DRYFT_LATENT_ROWS(8); }
  DRYFT_LATENT_ROWS(16);
#undef DRYFT_LATENT_ROWS
}

DRYFT_API int dryft_latent_fold_q(int is_bf16, const void* q, int q_stride, const void* w, float* q_lat, int n_tokens, int H, int dim,
                                  int kv_rank, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || dim <= 0 || kv_rank <= 0 || dim > 12000) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int threads = kv_rank >= 256 ? 256 : (kv_rank >= 128 ? 128 : 64);
  const size_t smem = sizeof(float) * (size_t)dim;
  dim3 grid(n_tokens, H);
  if (is_bf16) latent_fold_q_kernel<bf><<<grid, threads, smem, st>>>((const bf*)q, q_stride, (const bf*)w, q_lat, n_tokens, H, dim, kv_rank);
  else latent_fold_q_kernel<float><<<grid, threads, smem, st>>>((const float*)q, q_stride, (const float*)w, q_lat, n_tokens, H, dim, kv_rank);
  return launch_status();
}

DRYFT_API int dryft_latent_unfold_o(int is_bf16, const void* o_lat, const void* w, const void* gate, int gate_ld, void* out, int n_tokens,
                                    int H, int kv_rank, int vdim, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || H > 65535 || vdim <= 0 || kv_rank <= 0 || kv_rank > 12000) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const int threads = vdim >= 256 ? 256 : (vdim >= 128 ? 128 : 64);
  const size_t smem = sizeof(float) * (size_t)kv_rank;
  dim3 grid(n_tokens, H);
  if (is_bf16)
    latent_unfold_o_kernel<bf><<<grid, threads, smem, st>>>((const bf*)o_lat, (const bf*)w, (const bf*)gate, gate_ld, (bf*)out, n_tokens, H,
                                                            kv_rank, vdim);
  else
    latent_unfold_o_kernel<float><<<grid, threads, smem, st>>>((const float*)o_lat, (const float*)w, (const float*)gate, gate_ld, (float*)out,
                                                               n_tokens, H, kv_rank, vdim);
  return launch_status();
}

DRYFT_API int dryft_latent_scratch_table(const int* cu_q, const int* seq_slot, int n_seqs, int* table, int max_pages, int page_size,
                                         cudaStream_t st) {
  if (n_seqs <= 0) return 0;
  latent_scratch_table_kernel<<<(n_seqs + 127) / 128, 128, 0, st>>>(cu_q, seq_slot, n_seqs, table, max_pages, page_size);
  return launch_status();
}

DRYFT_API int dryft_latent_expand_store(int is_bf16, const void* q, const void* kv, int kv_ld, int v_off, const void* proj, int ld,
                                        int krot_off, const float* inv_freq, const float* inv_freq_lo, int interleaved,
                                        const int* tok_slot, const int* tok_pos, const int* table, int max_pages, int page_size,
                                        void* q_out, void* k_pages, void* v_pages, int n, int H, int dim, int rot, int vdim,
                                        cudaStream_t st) {
  if (n <= 0) return 0;
  if (H <= 0 || dim <= 0 || rot < 0 || (rot & 1) || vdim > dim + rot) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  const size_t smem = sizeof(float) * ((size_t)rot * (H + 1) + 1);
  if (smem > 48 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16)
    latent_expand_store_kernel<bf><<<n, PREP_THREADS, smem, st>>>((const bf*)q, (const bf*)kv, kv_ld, v_off, (const bf*)proj, ld, krot_off,
                                                                  inv_freq, inv_freq_lo, interleaved, tok_slot, tok_pos, table, max_pages,
                                                                  page_size, (bf*)q_out, (bf*)k_pages, (bf*)v_pages, H, dim, rot, vdim);
  else
    latent_expand_store_kernel<float><<<n, PREP_THREADS, smem, st>>>((const float*)q, (const float*)kv, kv_ld, v_off, (const float*)proj,
                                                                     ld, krot_off, inv_freq, inv_freq_lo, interleaved, tok_slot, tok_pos,
                                                                     table, max_pages, page_size, (float*)q_out, (float*)k_pages,
                                                                     (float*)v_pages, H, dim, rot, vdim);
  return launch_status();
}

DRYFT_API int dryft_head_gate_rows(int is_bf16, const void* o, int hd, const void* gate, int gate_ld, void* out, int n_tokens, int H,
                                   int vdim, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const size_t total = (size_t)n_tokens * H * vdim;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (is_bf16) head_gate_rows_kernel<bf><<<blocks, 256, 0, st>>>((const bf*)o, hd, (const bf*)gate, gate_ld, (bf*)out, n_tokens, H, vdim);
  else head_gate_rows_kernel<float><<<blocks, 256, 0, st>>>((const float*)o, hd, (const float*)gate, gate_ld, (float*)out, n_tokens, H, vdim);
  return launch_status();
}

DRYFT_API int dryft_head_gate(int is_bf16, const float* o, const void* gate, int gate_ld, void* out, int n_tokens, int H, int vdim,
                              cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  typedef __nv_bfloat16 bf;
  const size_t total = (size_t)n_tokens * H * vdim;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (is_bf16) head_gate_kernel<bf><<<blocks, 256, 0, st>>>(o, (const bf*)gate, gate_ld, (bf*)out, n_tokens, H, vdim);
  else head_gate_kernel<float><<<blocks, 256, 0, st>>>(o, (const float*)gate, gate_ld, (float*)out, n_tokens, H, vdim);
  return launch_status();
}
