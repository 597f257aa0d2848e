// Y[M, N] = X[M, K] . W[N, K]^T on CUDA cores with 32-bit fused multiply-adds: the matrix product
// of the true 32-bit path (no tensor cores, no reduced-precision mode), and the product that takes
// any size and any dtype mix when a tensor-core kernel refuses a shape.
//
// W is row-major [out, in] as the reference stores every matrix (crates/xrt-models/src/llama.rs:447-486),
// so both operands are contiguous along K.  The reference's own CUDA matmul_kernel
// (crates/xrt-cuda/src/lib.rs:636-772) takes B untransposed with 16x16 tiles and one fma a step;
// this one computes a 4x4 patch a thread from 64x64x16 shared-memory tiles.
// Every output element is summed over k = 0 .. K-1 in order by one thread, so a row's result does
// not depend on how many other rows the call carries.
#include "common.cuh"

namespace xrt {

constexpr int RG_BM = 64, RG_BN = 64, RG_BK = 16;

// epilogue: 0 = store, 1 = add into the 32-bit output (the residual stream)
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_reference_kernel(TO* __restrict__ out, const TX* __restrict__ x, const TW* __restrict__ w, int M, int N,
                      int K, int ldx, int ldo, int epilogue) {
  __shared__ float xs[RG_BK][RG_BM + 4];
  __shared__ float ws[RG_BK][RG_BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * RG_BM, n0 = blockIdx.x * RG_BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += RG_BK) {
    // each thread loads 4 elements of each tile: row = (tid*4 + i) / 16, k = (tid*4 + i) % 16
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid * 4 + i, r = e / RG_BK, kk = e % RG_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      xs[kk][r] = (gm < M && gk < K) ? to_float(x[(size_t)gm * ldx + gk]) : 0.f;
      ws[kk][r] = (gn < N && gk < K) ? to_float(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < RG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[kk][tm + i]; b[i] = ws[kk][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      TO* dst = out + (size_t)gm * ldo + gn;
      if (epilogue == 1) *dst = from_float<TO>(to_float(*dst) + acc[i][j]);
      else *dst = from_float<TO>(acc[i][j]);
    }
  }
}

}  // namespace xrt

// x: [M, K] with row stride ldx; w: [N, K] contiguous; out: [M, N] with row stride ldo.
XRT_EXPORT int xrt_gemm_reference(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                  int x_dtype, int w_dtype, int out_dtype, int epilogue, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || epilogue < 0 || epilogue > 1) return XRT_ERR_ARGUMENT;
  if (epilogue == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (M == 0) return XRT_OK;
  dim3 grid((N + xrt::RG_BN - 1) / xrt::RG_BN, (M + xrt::RG_BM - 1) / xrt::RG_BM);
  if (grid.y > 65535) return XRT_ERR_UNSUPPORTED;
  XRT_DISPATCH_DTYPE(x_dtype, TX, {
    XRT_DISPATCH_DTYPE(w_dtype, TW, {
      XRT_DISPATCH_DTYPE(out_dtype, TO, {
        xrt::gemm_reference_kernel<TX, TW, TO><<<grid, 256, 0, stream>>>(
            (TO*)out, (const TX*)x, (const TW*)w, M, N, K, ldx, ldo, epilogue);
      });
    });
  });
  return xrt::launch_status();
}
