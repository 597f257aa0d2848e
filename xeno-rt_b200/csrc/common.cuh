// Shared helpers of the sm_100a kernels: dtype codes, conversions, status codes, reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

// dtype codes, the same integers as DType.code on the Python side
#define XRT_F32 0
#define XRT_BF16 1

// Tokens in one block of the cache; the attention kernels tile keys by it.
#define XRT_BLOCK_TOKENS 64

// Status codes returned by every launcher.  0 = launched; negative = the arguments were refused
// before any launch; positive = a cudaError_t reported by the launch.
#define XRT_OK 0
#define XRT_ERR_ARGUMENT -1
#define XRT_ERR_UNSUPPORTED -2

#define XRT_EXPORT extern "C" __attribute__((visibility("default")))

namespace xrt {

// Kernel variants a caller may force (tuning.cu holds the one instance; xrt_set_tuning sets it).
struct Tuning {
  bool pdl = true;                  // launch with programmatic dependent launch
  int decode_attention = 0;         // 0 auto, 1 heads as rows, 2 cp.async copies, 3 no clusters
  int gemm_tile_rows = 0;           // 0 auto, 128 or 256: the prefill product's tile
  bool decode_gemm_clusters = true; // the decode product's splits meet through a cluster's shared memory
  int decode_cluster_pairs = 128;    // decode attention merges its splits as clusters up to so many (token, kv head) pairs
};
const Tuning& tuning();

// A norm that is finished by the product after it.  A product that adds into the residual stream can
// prepare the RMSNorm that follows (crates/xrt-kernels/src/cpu/rmsnorm.rs:26-43), so that no norm kernel
// has to run between two products: beside the new residual it writes residual * norm weight in bfloat16
// (the next product's operand) and, for every row, partial sums of squares of the new residual (NormEmit:
// `squares` is [parts, rows]; what a part covers is the emitting kernel's business).  The next product
// multiplies row m of its result by 1 / sqrt(sum of the row's parts / width + eps) (RowScale), since
// W . ((x * inv) * w) = inv * (W . (x * w)).  The statistics are 32-bit sums over the 32-bit residual,
// added in a fixed order.
struct NormEmit {
  __nv_bfloat16* scaled = nullptr;  // [M, ld] bfloat16: new residual * weight
  const void* weight = nullptr;     // [N] norm weight, 32-bit or bfloat16
  float* squares = nullptr;         // [parts, M]
  int ld = 0;
  int weight_dtype = XRT_F32;
};
struct RowScale {
  const float* squares = nullptr;   // [parts, M], or null: the input is what it is
  int parts = 0;
  int width = 1;
  float eps = 0.f;
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block with a fixed order: lanes by butterfly, then warps in index order.
// `scratch` holds at least 33 floats of shared memory.  Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < n_warps; ++w) total += scratch[w];
    scratch[32] = total;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch.  A kernel launched with `pdl` may begin while the kernel before it
// in the stream is still running: what it does before pdl_wait() (prefetching weights, set-up)
// overlaps the predecessor's tail and hides its own launch latency; pdl_wait() returns once the
// predecessor has completed and its writes are visible.  Every kernel of the decode step calls
// pdl_trigger() first (its successor may be launched) and pdl_wait() before it touches anything a
// predecessor wrote or reads anything it will overwrite.  Tuning::pdl = false turns the launch
// attribute off (the instructions are then no-ops).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() { return tuning().pdl; }

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  const bool pdl = pdl_enabled();
  config.attrs = pdl ? attribute : nullptr;
  config.numAttrs = pdl ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

// The same launch with a range of global memory that the kernel reads once (a weight): its lines
// are marked as streaming in the L2 (an access-policy window of the launch), so they are the first to
// leave and what the step reads again stays.  For kernels whose copies cannot carry a cache hint
// themselves.  The window is cut to what the device allows.
template <typename... KArgs, typename... Args>
inline void launch_kernel_streaming(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    const void* read_once, size_t read_once_bytes, Args... args) {
  static int max_window = -1;
  if (max_window < 0) {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&value, cudaDevAttrMaxAccessPolicyWindowSize, device) != cudaSuccess)
      value = 0;
    cudaGetLastError();
    max_window = value;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  int n = 0;
  if (pdl_enabled()) {
    attribute[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (max_window > 0 && read_once != nullptr && read_once_bytes > 0) {
    attribute[n].id = cudaLaunchAttributeAccessPolicyWindow;
    attribute[n].val.accessPolicyWindow.base_ptr = const_cast<void*>(read_once);
    attribute[n].val.accessPolicyWindow.num_bytes = read_once_bytes < (size_t)max_window ? read_once_bytes : (size_t)max_window;
    attribute[n].val.accessPolicyWindow.hitRatio = 1.0f;
    attribute[n].val.accessPolicyWindow.hitProp = cudaAccessPropertyStreaming;
    attribute[n].val.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    ++n;
  }
  config.attrs = n ? attribute : nullptr;
  config.numAttrs = n;
  cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

inline int launch_status() {
  cudaError_t err = cudaPeekAtLastError();
  return err == cudaSuccess ? XRT_OK : (int)err;
}

}  // namespace xrt

// Dispatch on a dtype code: runs BODY with `T` bound to float or __nv_bfloat16.
#define XRT_DISPATCH_DTYPE(code, T, ...)            \
  do {                                              \
    if ((code) == XRT_F32) {                        \
      using T = float;                              \
      __VA_ARGS__                                   \
    } else if ((code) == XRT_BF16) {                \
      using T = __nv_bfloat16;                      \
      __VA_ARGS__                                   \
    } else {                                        \
      return XRT_ERR_UNSUPPORTED;                   \
    }                                               \
  } while (0)
