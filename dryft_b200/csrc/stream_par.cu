// Kernels around a 32-bit residual stream whose layers add several results at once (a mixer and a feed-forward that read
// the same normed input, two mixers side by side), and around a stretch of layers that is entered through a product over
// the stream joined with an earlier copy of it.  T is the activation type; every sum and norm is 32-bit.
//
//   stream_sum    x32[n] += s0 * y0[n] + s1 * y1[n] + s2 * y2[n] + sr * sum_k yr[n * top + k] + vec        (every term optional)
//                 and, when a norm weight is given, h[n] = T( x32[n] / sqrt(mean(x32[n]^2) + eps) * w ): the sum of a layer
//                 and the norm of the next in one launch.  `src` (optional, 32-bit) replaces x32 as the sum's start
//                 (x32[n] = src[n] + ...).
//   pack_pair     out[n] = T([a32[n] | b32[n]]): two 32-bit rows side by side as one operand row of a product
//   softcap       z <- cap * tanh(z / cap) over 32-bit logits, in place
//
// One block per row; widths are runtime arguments of any size.  Rows whose slot is -1 (padding) are computed like any
// other: they read and write only their own row.  No block waits on another.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS) stream_sum_kernel(
    float* __restrict__ x32, const float* __restrict__ src, const T* __restrict__ y0, float s0, const T* __restrict__ y1, float s1,
    const T* __restrict__ y2, float s2, const T* __restrict__ yr, int top, float sr, const float* __restrict__ vec,
    const float* __restrict__ norm_w, float eps, T* __restrict__ h, int width) {
  __shared__ float scratch[33];
  const size_t n = blockIdx.x;
  float* x = x32 + n * width;
  const float* xs = src != nullptr ? src + n * width : x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v = xs[c];
    float add = 0.f;
    if (y0 != nullptr) add = fmaf(s0, to_f32<T>(y0[n * width + c]), add);
    if (y1 != nullptr) add = fmaf(s1, to_f32<T>(y1[n * width + c]), add);
    if (y2 != nullptr) add = fmaf(s2, to_f32<T>(y2[n * width + c]), add);
    if (yr != nullptr) {
      float r = 0.f;
      for (int k = 0; k < top; ++k) r += to_f32<T>(yr[(n * top + k) * width + c]);   // in the order of the choices
      add = fmaf(sr, r, add);
    }
    if (vec != nullptr) add += vec[c];
    v += add;
    x[c] = v;
    ss = fmaf(v, v, ss);
  }
  if (norm_w == nullptr) return;
  ss = block_sum(ss, scratch);
  const float rinv = 1.f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) h[n * width + c] = from_f32<T>(x[c] * rinv * norm_w[c]);   // the thread's own writes
}

template <typename T>
__global__ void __launch_bounds__(THREADS) pack_pair_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                           T* __restrict__ out, int width) {
  const size_t n = blockIdx.x;
  for (int c = threadIdx.x; c < 2 * width; c += THREADS)
    out[n * 2 * width + c] = from_f32<T>(c < width ? a[n * width + c] : b[n * width + (c - width)]);
}

__global__ void softcap_kernel(float* __restrict__ z, size_t count, float cap) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) z[i] = cap * tanhf(z[i] / cap);
}
}  // namespace

DRYFT_API int dryft_stream_sum(int is_bf16, float* x32, const float* src, const void* y0, float s0, const void* y1, float s1,
                               const void* y2, float s2, const void* yr, int top, float sr, const float* vec, const float* norm_w,
                               float eps, void* h, int n, int width, cudaStream_t st) {
  if (n <= 0) return 0;
  if (width <= 0 || (yr != nullptr && top < 1) || (norm_w != nullptr && h == nullptr)) return DRYFT_ERR_UNSUPPORTED;
  typedef __nv_bfloat16 bf;
  if (is_bf16)
    stream_sum_kernel<bf><<<n, THREADS, 0, st>>>(x32, src, (const bf*)y0, s0, (const bf*)y1, s1, (const bf*)y2, s2, (const bf*)yr, top, sr,
                                                 vec, norm_w, eps, (bf*)h, width);
  else
    stream_sum_kernel<float><<<n, THREADS, 0, st>>>(x32, src, (const float*)y0, s0, (const float*)y1, s1, (const float*)y2, s2,
                                                    (const float*)yr, top, sr, vec, norm_w, eps, (float*)h, width);
  return launch_status();
}

DRYFT_API int dryft_pack_pair(int is_bf16, const float* a, const float* b, void* out, int n, int width, cudaStream_t st) {
  if (n <= 0) return 0;
  if (width <= 0) return DRYFT_ERR_UNSUPPORTED;
  if (is_bf16) pack_pair_kernel<__nv_bfloat16><<<n, THREADS, 0, st>>>(a, b, (__nv_bfloat16*)out, width);
  else pack_pair_kernel<float><<<n, THREADS, 0, st>>>(a, b, (float*)out, width);
  return launch_status();
}

DRYFT_API int dryft_softcap(float* z, long long count, float cap, cudaStream_t st) {
  if (count <= 0) return 0;
  if (!(cap > 0.f)) return DRYFT_ERR_UNSUPPORTED;
  softcap_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>(z, (size_t)count, cap);
  return launch_status();
}
