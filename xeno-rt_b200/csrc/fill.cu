// Seeded normal fill of a tensor on the device, element for element the generator of
// weights/random_init.py:
//   bits(i) = splitmix64(key + (i + 1) * 0x9E3779B97F4A7C15)
//   u1 = ((bits >> 32) + 1) / 2^32,  u2 = (bits & 0xFFFFFFFF) / 2^32
//   value(i) = mean + std * sqrt(-2 ln u1) * cos(2 pi u2)        (float64, then rounded)
// The reference draws test weights from a linear congruential generator on the host
// (tests/common/mod.rs:719-731); this kernel exists so that models of tens of gigabytes can be
// drawn where they live.
#include "common.cuh"

namespace xrt {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t count, uint64_t key, double mean, double std) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t bits = splitmix64(key + (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull);
    const double u1 = ((double)(bits >> 32) + 1.0) / 4294967296.0;
    const double u2 = (double)(bits & 0xFFFFFFFFull) / 4294967296.0;
    const double z = sqrt(-2.0 * log(u1)) * cos(2.0 * 3.14159265358979323846 * u2);
    out[i] = from_float<T>((float)(mean + std * z));
  }
}

}  // namespace xrt

XRT_EXPORT int xrt_fill_normal(void* out, long long count, unsigned long long key, double mean, double std,
                               int dtype, cudaStream_t stream) {
  if (count < 0) return XRT_ERR_ARGUMENT;
  if (count == 0) return XRT_OK;
  const long long want = (count + 255) / 256;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  XRT_DISPATCH_DTYPE(dtype, T, {
    xrt::fill_normal_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, (size_t)count, (uint64_t)key, mean, std);
  });
  return xrt::launch_status();
}
