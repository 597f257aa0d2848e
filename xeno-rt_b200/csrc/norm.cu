// RMSNorm over rows of the 32-bit residual stream: y = (x * rsqrt(mean(x^2) + eps)) * w.
// Restates crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43 and the reference's PTX rmsnorm_kernel
// (crates/xrt-cuda/src/lib.rs:41-224: one block a row, a tree reduction, then the scaling).
// Statistics are 32-bit; the output is 32-bit or bfloat16.  With `rows` the kernel gathers:
// output row r is the norm of input row rows[r] (used for the rows whose logits are wanted).
#include "common.cuh"

namespace xrt {

template <typename TW, typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const TW* __restrict__ w,
                               const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[33];
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
  const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  XRT_DISPATCH_DTYPE(weight_dtype, TW, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      xrt::rmsnorm_kernel<TW, TO><<<n_rows, threads, 0, stream>>>((TO*)out, x, (const TW*)weight, rows,
                                                                 width, eps);
    });
  });
  return xrt::launch_status();
}
