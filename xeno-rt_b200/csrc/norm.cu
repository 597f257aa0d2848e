// RMSNorm over rows of the 32-bit residual stream: y = (x * rsqrt(mean(x^2) + eps)) * w.
// Restates crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43 and the reference's PTX rmsnorm_kernel
// (crates/xrt-cuda/src/lib.rs:41-224: one block a row, a tree reduction, then the scaling).
// Statistics are 32-bit; the output is 32-bit or bfloat16.  With `rows` the kernel gathers:
// output row r is the norm of input row rows[r] (used for the rows whose logits are wanted).
//
// A decode step normalises a handful of rows, so the kernel's time is load latency, not
// bandwidth: a row is read once with 16-byte loads that are all issued before the first is used
// (up to eight a thread, kept in registers for the scaling pass), one block a row.
#include "common.cuh"

namespace xrt {

constexpr int NORM_THREADS = 256;

template <typename TW> struct Vec4Of;
template <> struct Vec4Of<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct Vec4Of<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
};
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// width is a multiple of 4 and at most CHUNKS * NORM_THREADS * 4
template <typename TW, typename TO, int CHUNKS>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                   const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  // the weight does not depend on the step: it is on its way while the kernel before this one finishes
  float wv[CHUNKS][4];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<TW>::load(w + c, wv[i]);
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float v[CHUNKS][4];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) Vec4Of<float>::load(xr + c, v[i]);
    else v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc = fmaf(v[i][j], v[i][j], acc);
  const float total = block_sum(acc, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (size_t)r * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (threadIdx.x + i * NORM_THREADS) * 4;
    if (c < width) {
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = (v[i][j] * inv) * wv[i][j];
      store4(dst + c, y);
    }
  }
}

// any width
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                               const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + (size_t)src * width;
  float acc = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = xr[c];
    acc = fmaf(v, v, acc);
  }
  const float total = block_sum(acc, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  TO* dst = out + (size_t)r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    dst[c] = from_float<TO>((xr[c] * inv) * to_float(w[c]));
}

}  // namespace xrt


XRT_EXPORT int xrt_rmsnorm(void* out, const float* x, const void* weight, const int* rows, int n_rows,
                           int width, float eps, int weight_dtype, int out_dtype, cudaStream_t stream) {
  if (n_rows < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  const bool vec = width % 4 == 0 && width <= 8 * xrt::NORM_THREADS * 4 && (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  const int chunks = (width / 4 + xrt::NORM_THREADS - 1) / xrt::NORM_THREADS;
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      if (vec && chunks <= 1)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 1>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 2)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 2>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec && chunks <= 4)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 4>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else if (vec)
        xrt::launch_kernel(xrt::rmsnorm_vec_kernel<TW, TO, 8>, dim3(n_rows), dim3(xrt::NORM_THREADS), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
      else
        xrt::launch_kernel(xrt::rmsnorm_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, (TO*)out, x, (const TW*)weight, rows, width, eps);
    });
  });
  return xrt::launch_status();
}
