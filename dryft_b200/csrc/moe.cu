// Mixture of experts: the router's choice and the experts evaluated assignment by assignment.
//
//   moe_route     scores s = softmax(logits) over all E experts (32-bit), or (bit 1 of `renorm` set) s_e = sigmoid(logit_e).  Expert e belongs to group e / (E / n_groups)
//                 (contiguous, equally sized); a group is ranked by the maximum score among its members, and selection
//                 is restricted to the `keep` highest-ranked groups
//                 (n_groups = keep = 1: no groups).  The `top` allowed experts with the largest scores are chosen;
//                 their weights are the scores themselves, or the scores divided by their sum (`renorm`: the softmax
//                 over the chosen logits only).  `bias` (optional, [E]) is added to the logits first.
//                 Ties go to the lower index.  One warp per token.  moe_route_rows is the same for few tokens with the
//                 router's product inside (one block per token, one launch instead of two).
//   moe_rows      an assignment a = (token, k) multiplies its token's activation row by its expert's matrices, every
//                 weight row read once per assignment (a matrix-vector product per warp row): the form for few
//                 tokens (decode) and for the 32-bit path.
//                   mode 0:  act[a, f] = silu(Wg_e[f] . h[token]) * (Wu_e[f] . h[token])      (W_gu [E, 2F, K]: gate rows, then up rows)
//                   mode 1:  y[a, c]   = Wd_e[c] . act[a]                                    (W_d [E, C, F])
//                   mode 2:  act[a, f] = max(Wu_e[f] . h[token], 0)^2                         (W_u [E, F, K]: experts without a gate)
//                   mode 3:  the assignment's weight s = in_w[a] scales the expert's INPUT, and the activation is clamped:
//                            g = min(s * Wg_e[f] . h, limit), u = clamp(s * Wu_e[f] . h, -limit, limit),
//                            act[a, f] = g * sigmoid(alpha * g) * (u + up_off)
//                 32-bit accumulation in a fixed order, one rounding to T at the end.
//   moe_combine   out[n] = sum_k wts[n, k] * y[n*top + k]   (32-bit sum, rounded once) for callers that do not fold the
//                 weighted sum into a kernel of their own.
// No block waits on another block.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// One warp's choice for one token: z holds the E logits (global or shared memory), s and gs are the warp's scratch
// ([E] scores, [n_groups] group scores) in shared memory.
__device__ __forceinline__ void route_one(const float* z, const float* __restrict__ bias, float* s, float* gs, int lane, int n, int E,
                                          int n_groups, int keep, int top, int renorm, int* __restrict__ idx_out,
                                          float* __restrict__ w_out) {
  const bool sigmoid_scores = renorm >= 2;      // bit 1 of `renorm`: every expert's score is the sigmoid of its own logit
  renorm &= 1;
  if (sigmoid_scores) {
    for (int e = lane; e < E; e += 32) s[e] = 1.f / (1.f + expf(-(z[e] + (bias != nullptr ? bias[e] : 0.f))));
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e] + (bias != nullptr ? bias[e] : 0.f));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(z[e] + (bias != nullptr ? bias[e] : 0.f) - mx);
      s[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  }
  __syncwarp();
  if (n_groups > 1) {
    const int gsz = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float m = -1.f;
      for (int j = 0; j < gsz; ++j) m = fmaxf(m, s[g * gsz + j]);
      gs[g] = m;
    }
    __syncwarp();
    // take the `keep` best groups away one by one (marking them -2); what is left at the end is shut out
    for (int r = 0; r < keep; ++r) {
      float bv = -1.5f;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (gs[g] > bv) { bv = gs[g]; bi = g; }
      warp_argmax(bv, bi);
      if (lane == 0 && bi < n_groups) gs[bi] = -2.f;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / gsz] != -2.f) s[e] = -1.f;
    __syncwarp();
  }
  float wsum = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -2.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > bv) { bv = s[e]; bi = e; }
    warp_argmax(bv, bi);
    if (bi >= E) { bi = 0; bv = 0.f; }   // nothing comparable left (a NaN row): a defined choice of weight zero
    if (bv < 0.f) bv = 0.f;              // fewer allowed experts than `top`
    if (lane == 0) {
      idx_out[(size_t)n * top + r] = bi;
      w_out[(size_t)n * top + r] = bv;
      s[bi] = -2.f;
    }
    wsum += bv;
    __syncwarp();
  }
  if (renorm && lane == 0 && wsum > 0.f)
    for (int r = 0; r < top; ++r) w_out[(size_t)n * top + r] /= wsum;
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, int n_tokens, int E, int n_groups, int keep, int top, int renorm,
    int* __restrict__ idx_out, float* __restrict__ w_out) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * ROUTE_WARPS + warp;
  if (n >= n_tokens) return;
  float* s = sm + (size_t)warp * (E + n_groups);
  route_one(logits + (size_t)n * E, bias, s, s + E, lane, n, E, n_groups, keep, top, renorm, idx_out, w_out);
}

// Few tokens (decode): the router's product and its choice in one launch.  One block per token: the token's row is staged
// in shared memory, every warp takes experts in turn (z_e = W_router[e] . h, 32-bit accumulation), warp 0 then chooses.
constexpr int ROUTE_ROW_THREADS = 1024;   // 32 warps: one or two experts a warp keeps the block one or two trips to memory long
template <typename T>
__global__ void __launch_bounds__(ROUTE_ROW_THREADS) moe_route_rows_kernel(
    const T* __restrict__ h, const T* __restrict__ w_router, const float* __restrict__ bias, int K, int E, int n_groups, int keep, int top,
    int renorm, int* __restrict__ idx_out, float* __restrict__ w_out) {
  extern __shared__ __align__(16) unsigned char smraw[];
  T* xs = reinterpret_cast<T*>(smraw);                  // the token's row
  float* z = reinterpret_cast<float*>(smraw + (sizeof(T) * (size_t)K + 15) / 16 * 16);   // [E] logits, [E] scores, [n_groups]
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = threadIdx.x; c < K; c += ROUTE_ROW_THREADS) xs[c] = h[(size_t)n * K + c];
  __syncthreads();
  for (int e = warp; e < E; e += ROUTE_ROW_THREADS / 32) {
    const T* wr = w_router + (size_t)e * K;
    float d = 0.f;
    constexpr int V = 16 / sizeof(T);
    if (K % V == 0) {
#pragma unroll 4
      for (int c = lane * V; c < K; c += 32 * V) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wr + c), xv = *reinterpret_cast<const uint4*>(xs + c);
        const T* we = reinterpret_cast<const T*>(&wv);
        const T* xe = reinterpret_cast<const T*>(&xv);
#pragma unroll
        for (int t = 0; t < V; ++t) d = fmaf(to_f32<T>(we[t]), to_f32<T>(xe[t]), d);
      }
    } else {
      for (int c = lane; c < K; c += 32) d = fmaf(to_f32<T>(wr[c]), to_f32<T>(xs[c]), d);
    }
    d = warp_sum(d);
    if (lane == 0) z[e] = d;
  }
  __syncthreads();
  if (warp == 0) route_one(z, bias, z + E, z + 2 * E, lane, n, E, n_groups, keep, top, renorm, idx_out, w_out);
}

constexpr int ROWS_THREADS = 128;
constexpr int ROWS_PER_BLOCK = 8;    // output features a block computes (2 per warp): many small blocks keep enough loads in flight

template <typename T>
__global__ void __launch_bounds__(ROWS_THREADS) moe_rows_kernel(
    const T* __restrict__ a_in, int a_div,              // activation row of assignment a: a_in[(a / a_div) * K]
    const T* __restrict__ w, const int* __restrict__ idx, int E, int rows_per_expert, int K, int n_out, int mode,
    T* __restrict__ out, const float* __restrict__ in_w, float limit, float alpha, float up_off) {
  extern __shared__ __align__(16) unsigned char smraw[];
  T* xs = reinterpret_cast<T*>(smraw);
  const int a = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int e = idx[a];
  e = min(max(e, 0), E - 1);
  const T* x = a_in + (size_t)(a / a_div) * K;
  for (int c = threadIdx.x; c < K; c += ROWS_THREADS) xs[c] = x[c];
  __syncthreads();
  const T* we = w + (size_t)e * rows_per_expert * K;
  const int o0 = blockIdx.y * ROWS_PER_BLOCK;
  constexpr int V = 16 / sizeof(T);
  const bool vec = (K % V) == 0;
  const int o_end = min(o0 + ROWS_PER_BLOCK, n_out);
  const bool two_mats = mode == 0 || mode == 3;
  const float in_s = mode == 3 ? in_w[a] : 1.f;
  // a warp takes two output features at a time: all their weight vectors are requested before any is used
  for (int o = o0 + 2 * warp; o < o_end; o += 2 * (ROWS_THREADS / 32)) {
    const bool two = o + 1 < o_end;
    float d[2][2] = {{0.f, 0.f}, {0.f, 0.f}};    // [feature][gate | up]
    const T* r[2][2];
#pragma unroll
    for (int f = 0; f < 2; ++f) {
      r[f][0] = we + (size_t)(o + (two ? f : 0)) * K;
      r[f][1] = we + (size_t)(n_out + o + (two ? f : 0)) * K;   // mode 0: the matching up row
    }
    if (vec) {
#pragma unroll 2
      for (int c = lane * V; c < K; c += 32 * V) {
        uint4 wv[2][2];
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          wv[f][0] = *reinterpret_cast<const uint4*>(r[f][0] + c);
          if (two_mats) wv[f][1] = *reinterpret_cast<const uint4*>(r[f][1] + c);
        }
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + c);
        const T* xe = reinterpret_cast<const T*>(&xv);
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          const T* e0 = reinterpret_cast<const T*>(&wv[f][0]);
#pragma unroll
          for (int t = 0; t < V; ++t) d[f][0] = fmaf(to_f32<T>(e0[t]), to_f32<T>(xe[t]), d[f][0]);
          if (two_mats) {
            const T* e1 = reinterpret_cast<const T*>(&wv[f][1]);
#pragma unroll
            for (int t = 0; t < V; ++t) d[f][1] = fmaf(to_f32<T>(e1[t]), to_f32<T>(xe[t]), d[f][1]);
          }
        }
      }
    } else {
      for (int c = lane; c < K; c += 32) {
        const float xv = to_f32<T>(xs[c]);
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          d[f][0] = fmaf(to_f32<T>(r[f][0][c]), xv, d[f][0]);
          if (two_mats) d[f][1] = fmaf(to_f32<T>(r[f][1][c]), xv, d[f][1]);
        }
      }
    }
#pragma unroll
    for (int f = 0; f < 2; ++f) {
      float v = warp_sum(d[f][0]);
      if (mode == 0) v = v / (1.f + expf(-v)) * warp_sum(d[f][1]);
      if (mode == 3) {
        const float g = fminf(v * in_s, limit), u = fminf(fmaxf(warp_sum(d[f][1]) * in_s, -limit), limit);
        v = g / (1.f + expf(-alpha * g)) * (u + up_off);
      }
      if (mode == 2) { v = fmaxf(v, 0.f); v *= v; }
      if (lane == 0 && (f == 0 || two)) out[(size_t)a * n_out + o + f] = from_f32<T>(v);
    }
  }
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ wts, int top, int width, T* __restrict__ out) {
  const int n = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < top; ++k) v = fmaf(wts[(size_t)n * top + k], to_f32<T>(y[((size_t)n * top + k) * width + c]), v);
    out[(size_t)n * width + c] = from_f32<T>(v);
  }
}

template <typename T>
int rows_launch(const void* a_in, int a_div, const void* w, const int* idx, int E, int K, int n_out, int mode, void* out,
                int n_assign, const float* in_w, float limit, float alpha, float up_off, cudaStream_t st) {
  if (n_assign <= 0) return 0;
  if (E < 1 || K < 1 || n_out < 1 || a_div < 1 || mode < 0 || mode > 3 || (mode == 3 && !in_w)) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = (sizeof(T) * (size_t)K + 15) / 16 * 16;
  if (smem > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int tiles = (n_out + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  if (tiles > 65535) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(n_assign, tiles);
  moe_rows_kernel<T><<<grid, ROWS_THREADS, smem, st>>>((const T*)a_in, a_div, (const T*)w, idx, E, (mode == 0 || mode == 3) ? 2 * n_out : n_out, K,
                                                      n_out, mode, (T*)out, in_w, limit, alpha, up_off);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_moe_route(const float* logits, const float* bias, int n_tokens, int E, int n_groups, int keep, int top, int renorm,
                              int* idx_out, float* w_out, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (E < 1 || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * (size_t)ROUTE_WARPS * (E + n_groups);
  if (smem > 48 * 1024) return DRYFT_ERR_UNSUPPORTED;
  moe_route_kernel<<<(n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, smem, st>>>(logits, bias, n_tokens, E, n_groups, keep,
                                                                                               top, renorm, idx_out, w_out);
  return launch_status();
}

DRYFT_API int dryft_moe_rows(int is_bf16, const void* a_in, int a_div, const void* w, const int* idx, int E, int K, int n_out,
                             int mode, void* out, int n_assign, const float* in_w, float limit, float alpha, float up_off,
                             cudaStream_t st) {
  return is_bf16 ? rows_launch<__nv_bfloat16>(a_in, a_div, w, idx, E, K, n_out, mode, out, n_assign, in_w, limit, alpha, up_off, st)
                 : rows_launch<float>(a_in, a_div, w, idx, E, K, n_out, mode, out, n_assign, in_w, limit, alpha, up_off, st);
}

DRYFT_API int dryft_moe_combine(int is_bf16, const void* y, const float* wts, int top, int width, void* out, int n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (is_bf16)
    moe_combine_kernel<__nv_bfloat16><<<n, 256, 0, st>>>((const __nv_bfloat16*)y, wts, top, width, (__nv_bfloat16*)out);
  else
    moe_combine_kernel<float><<<n, 256, 0, st>>>((const float*)y, wts, top, width, (float*)out);
  return launch_status();
}

DRYFT_API int dryft_moe_route_rows(int is_bf16, const void* h, const void* w_router, const float* bias, int n_tokens, int K, int E, int n_groups,
                                   int keep, int top, int renorm, int* idx_out, float* w_out, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (E < 1 || top < 1 || top > E || n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups || K < 1) return DRYFT_ERR_UNSUPPORTED;
  const size_t smem = sizeof(float) * (size_t)(2 * E + n_groups) + ((is_bf16 ? 2 : 4) * (size_t)K + 15) / 16 * 16;
  if (smem > 48 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16)
    moe_route_rows_kernel<__nv_bfloat16><<<n_tokens, ROUTE_ROW_THREADS, smem, st>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)w_router,
                                                                                    bias, K, E, n_groups, keep, top, renorm, idx_out, w_out);
  else
    moe_route_rows_kernel<float><<<n_tokens, ROUTE_ROW_THREADS, smem, st>>>((const float*)h, (const float*)w_router, bias, K, E, n_groups, keep,
                                                                            top, renorm, idx_out, w_out);
  return launch_status();
}
