// Row-wise operations around a 32-bit residual stream whose norm comes AFTER the sum, and activations that
// normalise over a token's whole feed-forward vector.  Every kernel is one block per row (or per row and part),
// arithmetic in 32-bit, one rounding to T on the way out.
//
//   gated_postnorm    v = alpha * x + sigmoid(gl + gb) * (sum_k wts[k] y_k  [+ sigmoid(sgl) * ys]) ;
//                     x <- v / sqrt(mean(v^2) + eps) * w ;  h <- T(x)
//                     y: the sublayer's output [n, W], or `top` rows per token with their weights (a routed
//                     feed-forward: the weighted sum is formed here); ys / sgl: an always-on expert's output and its
//                     per-token gate logit (none: the expert counts fully); gl: the residual gate's logits (a product's output, row stride gl_ld),
//                     gb its bias.
//   polynorm          out = a N(z) + b N(z^2) + c N(z^3) + e, N(u) = u / sqrt(mean(u^2) + eps) over the row
//   relu2             out = max(z, 0)^2
//   gated_group_norm  v = y * z * sigmoid(z); each of `parts` equal parts of the row divided by its own root mean
//                     square, times w
// No block waits on another block.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int ROW_THREADS = 256;

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) gated_postnorm_kernel(
    const T* __restrict__ y, const float* __restrict__ wts, int top, const T* __restrict__ ys, const T* __restrict__ sgl,
    int sgl_ld, const T* __restrict__ gl, int gl_ld, const float* __restrict__ gb, const float* __restrict__ w, float alpha,
    float eps, float* __restrict__ x32, T* __restrict__ h, int W) {
  extern __shared__ float row[];     // [W] the row before the norm
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const float sg = ys == nullptr ? 0.f : (sgl != nullptr ? sigmoidf_(to_f32<T>(sgl[(size_t)n * sgl_ld])) : 1.f);
  float ss = 0.f;
#pragma unroll 4
  for (int c = threadIdx.x; c < W; c += ROW_THREADS) {   // unrolled: the loads of four columns are in flight together
    float acc;
    if (top > 0) {
      acc = 0.f;
      for (int k = 0; k < top; ++k) acc = fmaf(wts[(size_t)n * top + k], to_f32<T>(y[((size_t)n * top + k) * W + c]), acc);
    } else {
      acc = to_f32<T>(y[(size_t)n * W + c]);
    }
    if (ys != nullptr) acc = fmaf(sg, to_f32<T>(ys[(size_t)n * W + c]), acc);
    const float g = gl != nullptr ? sigmoidf_(to_f32<T>(gl[(size_t)n * gl_ld + c]) + (gb != nullptr ? gb[c] : 0.f)) : 1.f;
    const float v = fmaf(alpha, x32[(size_t)n * W + c], g * acc);
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float tot = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(tot / (float)W + eps);
#pragma unroll 4
  for (int c = threadIdx.x; c < W; c += ROW_THREADS) {
    const float o = row[c] * r * w[c];
    x32[(size_t)n * W + c] = o;
    if (h != nullptr) h[(size_t)n * W + c] = from_f32<T>(o);
  }
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) polynorm_kernel(const T* __restrict__ z, int ldz, const float* __restrict__ coef,
                                                               float eps, T* __restrict__ out, int F) {
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const T* zr = z + (size_t)n * ldz;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int c = threadIdx.x; c < F; c += ROW_THREADS) {
    const float v = to_f32<T>(zr[c]), v2 = v * v;
    s2 += v2;
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v2 * v2, v2, s6);
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float r1 = coef[0] / sqrtf(s2 / (float)F + eps), r2 = coef[1] / sqrtf(s4 / (float)F + eps),
              r3 = coef[2] / sqrtf(s6 / (float)F + eps), e = coef[3];
  for (int c = threadIdx.x; c < F; c += ROW_THREADS) {
    const float v = to_f32<T>(zr[c]), v2 = v * v;
    out[(size_t)n * F + c] = from_f32<T>(fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))));
  }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ z, int ldz, T* __restrict__ out, int n, int F) {
  const long long total = (long long)n * F;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / F), c = (int)(i % F);
    const float v = fmaxf(to_f32<T>(z[(size_t)r * ldz + c]), 0.f);
    out[i] = from_f32<T>(v * v);
  }
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS) gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z,
                                                                       int ldz, const float* __restrict__ w, int part, float eps,
                                                                       T* __restrict__ out, int inner) {
  __shared__ float scratch[33];
  const int n = blockIdx.x, c0 = blockIdx.y * part;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += ROW_THREADS) {
    const float zz = z[(size_t)n * ldz + c0 + c];
    const float v = y[(size_t)n * inner + c0 + c] * (zz * sigmoidf_(zz));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float r = 1.f / sqrtf(ss / (float)part + eps);
  for (int c = threadIdx.x; c < part; c += ROW_THREADS) {
    const float zz = z[(size_t)n * ldz + c0 + c];
    const float v = y[(size_t)n * inner + c0 + c] * (zz * sigmoidf_(zz));
    out[(size_t)n * inner + c0 + c] = from_f32<T>(v * r * w[c0 + c]);
  }
}

template <typename T>
int postnorm_launch(const void* y, const float* wts, int top, const void* ys, const void* sgl, int sgl_ld, const void* gl, int gl_ld,
                    const float* gb, const float* w, float alpha, float eps, float* x32, void* h, int n, int W, cudaStream_t st) {
  const size_t smem = sizeof(float) * (size_t)W;
  if (smem > 200 * 1024) return DRYFT_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gated_postnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  gated_postnorm_kernel<T><<<n, ROW_THREADS, smem, st>>>((const T*)y, wts, top, (const T*)ys, (const T*)sgl, sgl_ld, (const T*)gl,
                                                        gl_ld, gb, w, alpha, eps, x32, (T*)h, W);
  return launch_status();
}
}  // namespace

DRYFT_API int dryft_gated_postnorm(int is_bf16, const void* y, const float* wts, int top, const void* ys, const void* sgl, int sgl_ld,
                                   const void* gl, int gl_ld, const float* gb, const float* w, float alpha, float eps, float* x32,
                                   void* h, int n, int W, cudaStream_t st) {
  if (n <= 0) return 0;
  if (W < 1 || top < 0 || (top > 0 && wts == nullptr)) return DRYFT_ERR_UNSUPPORTED;
  return is_bf16 ? postnorm_launch<__nv_bfloat16>(y, wts, top, ys, sgl, sgl_ld, gl, gl_ld, gb, w, alpha, eps, x32, h, n, W, st)
                 : postnorm_launch<float>(y, wts, top, ys, sgl, sgl_ld, gl, gl_ld, gb, w, alpha, eps, x32, h, n, W, st);
}

DRYFT_API int dryft_polynorm(int is_bf16, const void* z, int ldz, const float* coef, float eps, void* out, int n, int F,
                             cudaStream_t st) {
  if (n <= 0) return 0;
  if (F < 1 || ldz < F) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16)
    polynorm_kernel<__nv_bfloat16><<<n, ROW_THREADS, 0, st>>>((const __nv_bfloat16*)z, ldz, coef, eps, (__nv_bfloat16*)out, F);
  else
    polynorm_kernel<float><<<n, ROW_THREADS, 0, st>>>((const float*)z, ldz, coef, eps, (float*)out, F);
  return launch_status();
}

DRYFT_API int dryft_relu2(int is_bf16, const void* z, int ldz, void* out, int n, int F, cudaStream_t st) {
  if (n <= 0) return 0;
  if (F < 1 || ldz < F) return DRYFT_ERR_UNSUPPORTED;
  const long long total = (long long)n * F;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (is_bf16)
    relu2_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)z, ldz, (__nv_bfloat16*)out, n, F);
  else
    relu2_kernel<float><<<blocks, 256, 0, st>>>((const float*)z, ldz, (float*)out, n, F);
  return launch_status();
}

DRYFT_API int dryft_gated_group_norm(int is_bf16, const float* y, const float* z, int ldz, const float* w, int parts, float eps,
                                     void* out, int n, int inner, cudaStream_t st) {
  if (n <= 0) return 0;
  if (parts < 1 || inner < 1 || inner % parts || parts > 65535) return DRYFT_ERR_UNSUPPORTED;
  dim3 grid(n, parts);
  if (is_bf16)
    gated_group_norm_kernel<__nv_bfloat16><<<grid, ROW_THREADS, 0, st>>>(y, z, ldz, w, inner / parts, eps, (__nv_bfloat16*)out, inner);
  else
    gated_group_norm_kernel<float><<<grid, ROW_THREADS, 0, st>>>(y, z, ldz, w, inner / parts, eps, (float*)out, inner);
  return launch_status();
}
