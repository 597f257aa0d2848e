// Y[M, N] = X[M, K] . W[N, K]^T for few rows (decode steps): the weight is streamed from HBM once,
// bfloat16 operands, 32-bit accumulation on the tensor cores (mma.sync m16n8k16).
//
// The reference streams each weight row once per token through a row-parallel dot product
// (crates/xrt-kernels/src/cpu/matmul.rs:100-192, and 194-320 for several tokens sharing one pass
// over the weight); this is the same idea for a GPU whose time for this product is the time to read W.
//
// One thread block (8 warps) owns 8 weight rows.  The warps split K: warp w takes the 32-wide
// k blocks w, w+8, w+16, ...; inside a block lane (g = lane / 4, t = lane % 4) reads the 16 bytes
// W[row g][k0 + 8t .. k0 + 8t + 8) and the matching 16 bytes of up to two X rows.  A dot product
// does not care in which order k is visited as long as both operands agree, so the four 32-bit
// words of such a load are fed to two MMAs as the fragment slots (2t, 2t+1), (2t+8, 2t+9): every
// load is 16 bytes wide and no shuffle or shared-memory staging is needed.  The batch rows are the
// MMA's M (16 a tile), the 8 weight rows its N.  The eight warps' partial sums meet in shared
// memory and are added in warp order, so the result does not depend on the number of rows M.
// Epilogues: store (32-bit or bfloat16), add into the 32-bit residual stream, or SwiGLU
// (the block owns 8 gate rows and the 8 matching up rows, four warps each).
#include "common.cuh"

namespace xrt {

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 8;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: store, 1: add into float out, 2: SwiGLU of (W rows, W rows + up_offset)
template <int M_TILES, int MODE, typename TO>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(TO* __restrict__ out, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   int M, int N, int K, int ldx, int ldo, long long up_offset) {
  __shared__ float partial[SK_WARPS][M_TILES][16][SK_ROWS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * SK_ROWS;
  const int k_ways = MODE == 2 ? SK_WARPS / 2 : SK_WARPS;        // warps that split K
  const int k_lane = MODE == 2 ? (warp & 3) : warp;
  const int w_row = min(row0 + g, N - 1);                          // clamped; masked at the store
  const __nv_bfloat16* wp = w + (size_t)w_row * K + (MODE == 2 && warp >= 4 ? up_offset : 0);

  float acc[M_TILES][4];
#pragma unroll
  for (int mt = 0; mt < M_TILES; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

  // rows at or beyond M are clamped to the last row: their results are never stored, and a row of
  // the MMA depends on its own operand row only
  const __nv_bfloat16* xlo[M_TILES];
  const __nv_bfloat16* xhi[M_TILES];
#pragma unroll
  for (int mt = 0; mt < M_TILES; ++mt) {
    xlo[mt] = x + (size_t)min(mt * 16 + g, M - 1) * ldx;
    xhi[mt] = x + (size_t)min(mt * 16 + g + 8, M - 1) * ldx;
  }
  const int n_full = K / 32;
#pragma unroll 4
  for (int b = k_lane; b < n_full; b += k_ways) {
    const int k0 = b * 32 + t * 8;
    const uint4 wv = ldg_stream(wp + k0);
#pragma unroll
    for (int mt = 0; mt < M_TILES; ++mt) {
      const uint4 xa = *reinterpret_cast<const uint4*>(xlo[mt] + k0);
      const uint4 xb = *reinterpret_cast<const uint4*>(xhi[mt] + k0);
      mma_bf16_16816(acc[mt], xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
      mma_bf16_16816(acc[mt], xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
    }
  }
  // the last, partial block of 32 (K is a multiple of 8: a 16-byte piece is wholly inside or outside)
  if ((K & 31) != 0 && (n_full % k_ways) == k_lane) {  // uniform over the warp
    const int k0 = n_full * 32 + t * 8;
    const bool inside = k0 < K;  // differs between lanes: only the loads are conditional, every
    //                              lane runs the MMAs (a lane outside contributes zeros)
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4 wv = inside ? ldg_stream(wp + k0) : zero;
#pragma unroll
    for (int mt = 0; mt < M_TILES; ++mt) {
      const uint4 xa = inside ? *reinterpret_cast<const uint4*>(xlo[mt] + k0) : zero;
      const uint4 xb = inside ? *reinterpret_cast<const uint4*>(xhi[mt] + k0) : zero;
      mma_bf16_16816(acc[mt], xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
      mma_bf16_16816(acc[mt], xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
    }
  }

  // c0, c1: (m = g, n = 2t, 2t+1); c2, c3: (m = g + 8, same n)
#pragma unroll
  for (int mt = 0; mt < M_TILES; ++mt) {
    partial[warp][mt][g][2 * t] = acc[mt][0];
    partial[warp][mt][g][2 * t + 1] = acc[mt][1];
    partial[warp][mt][g + 8][2 * t] = acc[mt][2];
    partial[warp][mt][g + 8][2 * t + 1] = acc[mt][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < M_TILES * 16 * SK_ROWS; e += blockDim.x) {
    const int n = e % SK_ROWS, m = e / SK_ROWS;
    const int mt = m / 16, mr = m % 16;
    const int row = row0 + n;
    if (m >= M || row >= N) continue;
    TO* dst = out + (size_t)m * ldo + row;
    if (MODE == 2) {
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int ww = 0; ww < 4; ++ww) { gate += partial[ww][mt][mr][n]; up += partial[ww + 4][mt][mr][n]; }
      *dst = from_float<TO>((gate / (1.0f + expf(-gate))) * up);
    } else {
      float sum = 0.f;
#pragma unroll
      for (int ww = 0; ww < SK_WARPS; ++ww) sum += partial[ww][mt][mr][n];
      if (MODE == 1) *dst = from_float<TO>(to_float(*dst) + sum);
      else *dst = from_float<TO>(sum);
    }
  }
}

template <int M_TILES>
int launch_skinny(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo, int out_dtype,
                  int mode, long long up_offset, cudaStream_t stream) {
  const int blocks = (N + SK_ROWS - 1) / SK_ROWS;
  const auto* xp = (const __nv_bfloat16*)x;
  const auto* wp = (const __nv_bfloat16*)w;
  if (mode == 1) {
    gemm_skinny_kernel<M_TILES, 1, float><<<blocks, SK_WARPS * 32, 0, stream>>>((float*)out, xp, wp, M, N, K, ldx, ldo, 0);
  } else if (mode == 2) {
    if (out_dtype == XRT_BF16)
      gemm_skinny_kernel<M_TILES, 2, __nv_bfloat16><<<blocks, SK_WARPS * 32, 0, stream>>>((__nv_bfloat16*)out, xp, wp, M, N, K, ldx, ldo, up_offset);
    else
      gemm_skinny_kernel<M_TILES, 2, float><<<blocks, SK_WARPS * 32, 0, stream>>>((float*)out, xp, wp, M, N, K, ldx, ldo, up_offset);
  } else {
    if (out_dtype == XRT_BF16)
      gemm_skinny_kernel<M_TILES, 0, __nv_bfloat16><<<blocks, SK_WARPS * 32, 0, stream>>>((__nv_bfloat16*)out, xp, wp, M, N, K, ldx, ldo, 0);
    else
      gemm_skinny_kernel<M_TILES, 0, float><<<blocks, SK_WARPS * 32, 0, stream>>>((float*)out, xp, wp, M, N, K, ldx, ldo, 0);
  }
  return launch_status();
}

}  // namespace xrt

// x: bfloat16 [M, K] with row stride ldx (a multiple of 8); w: bfloat16 [N, K] contiguous, K a
// multiple of 8; out: [M, N] with row stride ldo.  mode 0 stores, 1 adds into a float32 out,
// 2 computes silu(x . W[n]) * (x . W[n + up_rows]) for n < N (w then has N + up_rows... rows, the
// "up" half starting up_rows rows after the "gate" half).  M is at most 64.
XRT_EXPORT int xrt_gemm_skinny(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                               int out_dtype, int mode, int up_rows, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || mode < 0 || mode > 2) return XRT_ERR_ARGUMENT;
  if (mode == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (out_dtype != XRT_F32 && out_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (K % 8 != 0 || ldx % 8 != 0 || M > 64) return XRT_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return XRT_ERR_UNSUPPORTED;
  if (M == 0) return XRT_OK;
  const long long up_offset = (long long)up_rows * K;
  if (M <= 16) return xrt::launch_skinny<1>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, stream);
  if (M <= 32) return xrt::launch_skinny<2>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, stream);
  return xrt::launch_skinny<4>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, stream);
}
