// SwiGLU on the fused gate/up product: out[t, f] = silu(gu[t, f]) * gu[t, F + f],
// silu(g) = g / (1 + exp(-g)).  Restates crates/xrt-kernels/src/cpu/silu.rs:1-3, 22-24; the
// reference's PTX silu_kernel (crates/xrt-cuda/src/lib.rs:596-635) has no gate product.
#include "common.cuh"

namespace xrt {

template <typename TI, typename TO>
__global__ void swiglu_kernel(TO* __restrict__ out, const TI* __restrict__ gate_up, int n_tokens, int width) {
  const size_t total = (size_t)n_tokens * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / width, f = i - t * width;
    const float g = to_float(gate_up[t * 2 * width + f]);
    const float u = to_float(gate_up[t * 2 * width + width + f]);
    out[i] = from_float<TO>((g / (1.0f + expf(-g))) * u);
  }
}

}  // namespace xrt

XRT_EXPORT int xrt_swiglu(void* out, const void* gate_up, int n_tokens, int width, int in_dtype,
                          int out_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || width <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const size_t total = (size_t)n_tokens * width;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  XRT_DISPATCH_DTYPE(in_dtype, TI, {
    XRT_DISPATCH_DTYPE(out_dtype, TO, {
      xrt::swiglu_kernel<TI, TO><<<blocks, 256, 0, stream>>>((TO*)out, (const TI*)gate_up, n_tokens, width);
    });
  });
  return xrt::launch_status();
}
