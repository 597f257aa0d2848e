// Embedding gather: rows of the table to the 32-bit residual stream.
// Restates crates/xrt-cuda/src/lib.rs:815-882 (embedding_kernel) of the reference, which writes
// zeros for an id outside the table while its host wrapper refuses such ids (1217-1225); here the
// kernel writes zeros and raises an error flag that the host reads.
#include "common.cuh"

namespace xrt {

template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab,
                                 int* __restrict__ error_flag) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = ok ? to_float(row[c]) : 0.f;
}

// 16 bytes of the table a thread and step (hidden a multiple of 8 for bfloat16, of 4 for float32)
template <typename TW>
__global__ void embedding_vec_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                     const int* __restrict__ ids, int hidden, int vocab,
                                     int* __restrict__ error_flag) {
  constexpr int PER = 16 / (int)sizeof(TW);
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
#pragma unroll 4
  for (int c = threadIdx.x * PER; c < hidden; c += blockDim.x * PER) {
    const uint4 raw = ok ? *reinterpret_cast<const uint4*>(row + c) : make_uint4(0u, 0u, 0u, 0u);
    const TW* vals = reinterpret_cast<const TW*>(&raw);
    float f[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) f[j] = ok ? to_float(vals[j]) : 0.f;
#pragma unroll
    for (int j = 0; j < PER; j += 4) *reinterpret_cast<float4*>(dst + c + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
  }
}

}  // namespace xrt

XRT_EXPORT int xrt_embedding(float* out, const void* table, const int* ids, int n_tokens, int hidden,
                             int vocab, int table_dtype, int* error_flag, cudaStream_t stream) {
  if (n_tokens < 0 || hidden <= 0 || vocab <= 0) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const bool vec = hidden % 8 == 0 && (((uintptr_t)out | (uintptr_t)table) & 15) == 0;
  XRT_DISPATCH_DTYPE(table_dtype, TW, {
    if (vec)
      xrt::launch_kernel(xrt::embedding_vec_kernel<TW>, dim3(n_tokens), dim3(128), 0, stream, out, (const TW*)table, ids, hidden, vocab, error_flag);
    else
      xrt::launch_kernel(xrt::embedding_kernel<TW>, dim3(n_tokens), dim3(256), 0, stream, out, (const TW*)table, ids, hidden, vocab, error_flag);
  });
  return xrt::launch_status();
}
