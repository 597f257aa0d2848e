// Y[M, N] = X[M, K] . W[N, K]^T for many rows (prompts), bfloat16 operands and 32-bit accumulation
// on the fifth-generation tensor cores: tcgen05.mma issued by one thread, operands staged in shared
// memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), accumulators in tensor memory (TMEM),
// read back with tcgen05.ld for the epilogue.
//
// W is row-major [out, in] as the reference stores every matrix (crates/xrt-models/src/llama.rs:447-486),
// so both operands are K-major and no transposition is needed.  The reference's own CUDA matmul_kernel
// (crates/xrt-cuda/src/lib.rs:636-772) is a 16x16-tile scalar kernel; this is its Blackwell counterpart.
//
// A persistent block (one a multiprocessor) walks output tiles of 128 x 256.  Six warps:
//   warp 0     producer: for each 64-wide slab of K, one TMA load of the X tile (128 x 64) and two of
//              the W tile (2 x 128 x 64) into the next free stage of a four-stage ring; the loads
//              complete on the stage's "full" mbarrier.  Tiles that reach beyond M, N or K are
//              zero-filled by TMA, so any M and N and any K that is a multiple of 8 work.
//   warp 1     allocates 512 TMEM columns (two accumulators of 128 lanes x 256 columns) and issues the
//              MMAs: four tcgen05.mma (128 x 256 x 16) a stage, then tcgen05.commit to the stage's
//              "empty" mbarrier; after the last slab, tcgen05.commit to the accumulator's "full" mbarrier.
//   warps 2-5  epilogue: each warp reads its 32 TMEM lanes (rows) with tcgen05.ld, 32 columns at a
//              time, and stores, adds into the 32-bit residual stream, or applies SwiGLU (the W
//              tile is then 128 gate rows and the 128 matching up rows), while the MMA warp already
//              fills the other accumulator.
// Every output element is the sum over K in one fixed order, whatever M is.
// Every wait on an mbarrier is bounded.  A wait that runs out raises the error flag and an abort
// flag in shared memory; all roles leave their loops, the block frees its TMEM and returns.
#include "tcgen05.cuh"

namespace xrt {

using namespace sm100;

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_UMMA_K = 16;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;        // 16 KB: 128 rows of X, one slab of K
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;        // 32 KB
// MT = 1: tiles of 128 x 256, four stages, two accumulators (the epilogue of a tile overlaps the MMAs
// of the next).  MT = 2: tiles of 256 x 256 (two MMAs a slab share the W tile: a third fewer operand
// bytes per flop, which is what bounds this kernel), three stages, one accumulator of all 512 TMEM
// columns and eight epilogue warps to drain it.
template <int MT> struct TcShape {
  static constexpr int STAGES = MT == 1 ? 4 : 3;
  static constexpr int STAGE_BYTES = MT * TC_A_BYTES + TC_BN * TC_BK * 2;
  static constexpr int ACC_SETS = MT == 1 ? 2 : 1;
  static constexpr int EPI_WARPS = 4 * MT;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int STAGING_BYTES = EPI_WARPS * 32 * 33 * 4;    // a 32 x 32 patch (padded) an epilogue warp
  static constexpr int SMEM = STAGES * STAGE_BYTES + STAGING_BYTES + 256 + 1024;  // + barriers + alignment slack
};
constexpr int TC_TMEM_COLS = 512;

// Four consecutive outputs of one row: 16 bytes of float32 (stored, or added into the residual
// stream) or 8 bytes of bfloat16.
template <int MODE>
__device__ __forceinline__ void store_quad(float* dst, float a, float b, float c, float d) {
  float4* p = reinterpret_cast<float4*>(dst);
  if (MODE == 1) {
    const float4 old = *p;
    *p = make_float4(old.x + a, old.y + b, old.z + c, old.w + d);
  } else {
    *p = make_float4(a, b, c, d);
  }
}
template <int MODE>
__device__ __forceinline__ void store_quad(__nv_bfloat16* dst, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

// MODE 0: store, 1: add into float out, 2: SwiGLU.  n_tiles_n counts tiles of 256 output columns
// (SwiGLU: of 128, each computed from 128 gate rows and 128 up rows of W).
template <int MODE, int MT, typename TO>
__global__ void __launch_bounds__(TcShape<MT>::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    TO* __restrict__ out, int M, int N, int K, int ldo, int up_rows, int* __restrict__ error_flag,
                    const NormEmit emit, const RowScale scale) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int TC_STAGES = TcShape<MT>::STAGES, ACC_SETS = TcShape<MT>::ACC_SETS;
  constexpr int STAGE_A = MT * TC_A_BYTES;
  unsigned char* a_stages = smem;
  unsigned char* b_stages = smem + TC_STAGES * STAGE_A;
  float* staging = reinterpret_cast<float*>(smem + TC_STAGES * TcShape<MT>::STAGE_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_STAGES * TcShape<MT>::STAGE_BYTES + TcShape<MT>::STAGING_BYTES);
  uint64_t* full = bars;                       // [TC_STAGES]
  uint64_t* empty = bars + TC_STAGES;          // [TC_STAGES]
  uint64_t* acc_full = bars + 2 * TC_STAGES;   // [ACC_SETS] (room for two)
  uint64_t* acc_empty = acc_full + 2;          // [ACC_SETS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int N_PER_TILE = MODE == 2 ? TC_BN / 2 : TC_BN;  // output columns a tile
  const int tiles_m = (M + MT * TC_BM - 1) / (MT * TC_BM);
  const int tiles_n = (N + N_PER_TILE - 1) / N_PER_TILE;
  const int n_tiles = tiles_m * tiles_n;
  const int k_iters = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 32 * TcShape<MT>::EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % TC_STAGES;
          ok = mbar_wait(smem_u32(&empty[s]), ((it / TC_STAGES) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full[s]);
          mbar_arrive_expect_tx(bar, STAGE_A + TC_B_BYTES);
#pragma unroll
          for (int h = 0; h < MT; ++h)
            tma_load_2d(smem_u32(a_stages + s * STAGE_A + h * TC_A_BYTES), &map_x, kb * TC_BK,
                           (m_blk * MT + h) * TC_BM, bar);
          const int w_row0 = n_blk * N_PER_TILE;
          const int w_row1 = MODE == 2 ? up_rows + w_row0 : w_row0 + 128;
          tma_load_2d(smem_u32(b_stages + s * TC_B_BYTES), &map_w, kb * TC_BK, w_row0, bar);
          tma_load_2d(smem_u32(b_stages + s * TC_B_BYTES + TC_B_BYTES / 2), &map_w, kb * TC_BK, w_row1, bar);
        }
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 3); }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(TC_BM, TC_BN);
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tile_i) {
        const int a = tile_i % ACC_SETS;
        ok = mbar_wait(smem_u32(&acc_empty[a]), ((tile_i / ACC_SETS) & 1) ^ 1, abort_flag);
        if (!ok) break;
        fence_after();
        const uint32_t tmem_d = tmem_base + a * MT * TC_BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % TC_STAGES;
          ok = mbar_wait(smem_u32(&full[s]), (it / TC_STAGES) & 1, abort_flag);
          if (!ok) break;
          fence_after();
          const uint64_t desc_b = desc_k_major(smem_u32(b_stages + s * TC_B_BYTES));
#pragma unroll
          for (int h = 0; h < MT; ++h) {
            const uint64_t desc_a = desc_k_major(smem_u32(a_stages + s * STAGE_A + h * TC_A_BYTES));
#pragma unroll
            for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)  // 32 bytes further along K inside the swizzle atom
              mma_f16(tmem_d + h * TC_BN, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0);
          }
          commit(smem_u32(&empty[s]));
        }
        if (ok) commit(smem_u32(&acc_full[a]));
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 3); }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32 * quarter ..
    const int half = (warp - 2) / 4;  // which 128 rows of the tile (always 0 for tiles of 128 rows)
    int tile_i = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tile_i) {
      const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
      const int a = tile_i % ACC_SETS;
      const int row0 = (m_blk * MT + half) * TC_BM + quarter * 32;  // the warp's first row
      // a pending norm of the input (RowScale): this lane's row's 1 / rms, from the parts the product before
      // this one left, added in part order while the tile's products still run
      float row_inv = 1.f;
      if (MODE != 1 && scale.squares != nullptr) {
        float sum = 0.f;
        if (row0 + lane < M)
          for (int p = 0; p < scale.parts; ++p) sum += __ldcg(scale.squares + (size_t)p * M + row0 + lane);
        row_inv = 1.0f / sqrtf(sum / (float)scale.width + scale.eps);
      }
      ok = mbar_wait(smem_u32(&acc_full[a]), (tile_i / ACC_SETS) & 1, abort_flag);
      if (!ok) break;
      fence_after();
      const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (a * MT + half) * TC_BN;
      const int col0 = n_blk * N_PER_TILE;
      // A thread holds one ROW of the accumulator; written as it is, every store instruction of the
      // warp would touch 32 lines.  The warp turns each 32 x 32 patch around in shared memory and
      // writes it with 16 bytes a lane, four whole 128-byte row pieces an instruction.
      float* patch = staging + (warp - 2) * 32 * 33;
      const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
      float squares[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // of rows it * 4 + sub_row, this lane's columns
#pragma unroll 1
      for (int c = 0; c < N_PER_TILE; c += 32) {
        uint32_t v[32];
        tmem_ld32(v, tmem_row + c);
        if (MODE == 2) {
          uint32_t u[32];
          tmem_ld32(u, tmem_row + TC_BN / 2 + c);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(v[j]) * row_inv;
            v[j] = __float_as_uint((g / (1.0f + expf(-g))) * (__uint_as_float(u[j]) * row_inv));
          }
        } else {
          tmem_wait_ld();
          if (MODE == 0 && scale.squares != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * row_inv);
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) patch[lane * 33 + j] = __uint_as_float(v[j]);
        __syncwarp();
        // the residual values first, all eight loads in flight (a load may not pass a store that
        // could alias it, so a read-modify-write a row piece at a time would wait for each in turn)
        float4 old[8];
        if (MODE == 1) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = row0 + it * 4 + sub_row, col = col0 + c + sub_col;
            const float* src = reinterpret_cast<const float*>(out) + (size_t)row * ldo + col;
            const bool whole = row < M && col + 3 < N && (((uintptr_t)src) & 15) == 0;
            old[it] = whole ? *reinterpret_cast<const float4*>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int pr = it * 4 + sub_row;  // row of the patch
          const int row = row0 + pr, col = col0 + c + sub_col;
          const float* src = patch + pr * 33 + sub_col;
          if (row < M) {
            TO* dst = out + (size_t)row * ldo + col;
            if (col + 3 < N && (((uintptr_t)dst) & (4 * sizeof(TO) - 1)) == 0) {
              if (MODE == 1) {
                const float4 sum = make_float4(old[it].x + src[0], old[it].y + src[1], old[it].z + src[2], old[it].w + src[3]);
                store_quad<0>(dst, sum.x, sum.y, sum.z, sum.w);
                if (emit.scaled != nullptr) {  // the launcher made sure that N is a multiple of 4 and the buffers aligned
                  float w4[4];
                  if (emit.weight_dtype == XRT_BF16) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(emit.weight) + col);
                    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                    w4[0] = __low2float(lo); w4[1] = __high2float(lo); w4[2] = __low2float(hi); w4[3] = __high2float(hi);
                  } else {
                    const float4 raw = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(emit.weight) + col);
                    w4[0] = raw.x; w4[1] = raw.y; w4[2] = raw.z; w4[3] = raw.w;
                  }
                  store_quad<0>(emit.scaled + (size_t)row * emit.ld + col, sum.x * w4[0], sum.y * w4[1], sum.z * w4[2], sum.w * w4[3]);
                  squares[it] = fmaf(sum.x, sum.x, squares[it]);
                  squares[it] = fmaf(sum.y, sum.y, squares[it]);
                  squares[it] = fmaf(sum.z, sum.z, squares[it]);
                  squares[it] = fmaf(sum.w, sum.w, squares[it]);
                }
              } else
                store_quad<0>(dst, src[0], src[1], src[2], src[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (col + e < N) {
                  if (MODE == 1) dst[e] = from_float<TO>(to_float(dst[e]) + src[e]);
                  else dst[e] = from_float<TO>(src[e]);
                }
            }
          }
        }
        __syncwarp();
      }
      if (MODE == 1 && emit.squares != nullptr) {
        // a row's columns of this tile sit in eight neighbouring lanes: summed in a fixed order, one part a tile of columns
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          float sum = squares[it];
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          const int row = row0 + it * 4 + sub_row;
          if ((lane & 7) == 0 && row < M) emit.squares[(size_t)n_blk * M + row] = sum;
        }
      }
      fence_before();
      mbar_arrive(smem_u32(&acc_empty[a]));
    }
    if (!ok && lane == 0) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 3); }
  }

  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS));
  }
}

// A map over a row-major bfloat16 matrix [rows, cols] with row stride ld, boxes of 128 rows x 64 columns.
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  return sm100::make_map_bf16_2d(map, base, rows, cols, ld, 128);
}

template <int MODE, int MT, typename TO>
int launch_tcgen05_tiled(void* out, const CUtensorMap& map_x, const CUtensorMap& map_w, int M, int N, int K, int ldo,
                         int up_rows, int* error_flag, int sm_count, const NormEmit& emit, const RowScale& scale,
                         cudaStream_t stream) {
  auto kernel = gemm_tcgen05_kernel<MODE, MT, TO>;
  static bool allowed = false;
  if (!allowed) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcShape<MT>::SMEM);
    if (err != cudaSuccess) return (int)err;
    allowed = true;
  }
  constexpr int n_per_tile = MODE == 2 ? TC_BN / 2 : TC_BN;
  const int tiles = ((M + MT * TC_BM - 1) / (MT * TC_BM)) * ((N + n_per_tile - 1) / n_per_tile);
  const int blocks = tiles < sm_count ? tiles : sm_count;
  // (no programmatic dependent launch: see attention_prefill_tcgen05.cu's launcher)
  kernel<<<blocks, TcShape<MT>::THREADS, TcShape<MT>::SMEM, stream>>>(map_x, map_w, (TO*)out, M, N, K, ldo, up_rows,
                                                                      error_flag, emit, scale);
  return launch_status();
}

// Tiles of 256 rows for products of few tiles, when they keep the multiprocessors about as busy as
// tiles of 128 rows would (the larger tile moves a third fewer operand bytes per flop and drains its
// accumulator with twice the warps; with many tiles the overlap of the small tile's two accumulators wins).
// Tuning::gemm_tile_rows = 128 or 256 forces one, for comparison.
template <int MODE, typename TO>
int launch_tcgen05(void* out, const CUtensorMap& map_x, const CUtensorMap& map_w, int M, int N, int K, int ldo,
                   int up_rows, int* error_flag, int sm_count, const NormEmit& emit, const RowScale& scale,
                   cudaStream_t stream) {
  constexpr int n_per_tile = MODE == 2 ? TC_BN / 2 : TC_BN;
  const long long tiles_n = (N + n_per_tile - 1) / n_per_tile;
  auto busy = [&](long long tiles) { return (double)tiles / (double)(((tiles + sm_count - 1) / sm_count) * sm_count); };
  const long long small_tiles = ((M + 127) / 128) * tiles_n;
  const double small = busy(small_tiles), large = 1.25 * busy(((M + 255) / 256) * tiles_n);
  const int forced = tuning().gemm_tile_rows;
  // measured at 2,048 and 8,192 rows: the large tile wins where the small one leaves under two rounds of work
  const bool use_large = forced == 256 || (forced != 128 && M > 128 && small_tiles <= 2 * sm_count && large > small);
  if (use_large)
    return launch_tcgen05_tiled<MODE, 2, TO>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, emit, scale, stream);
  return launch_tcgen05_tiled<MODE, 1, TO>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, emit, scale, stream);
}

}  // namespace xrt

// How many parts of a row's sum of squares a product that prepares the following norm leaves: one a tile
// of 256 output columns.
XRT_EXPORT int xrt_gemm_tcgen05_norm_parts(int N) { return N <= 0 ? XRT_ERR_ARGUMENT : (N + xrt::TC_BN - 1) / xrt::TC_BN; }

// x: bfloat16 [M, K] with row stride ldx; w: bfloat16 [rows, K] contiguous; K and ldx multiples of 8,
// both bases 16-byte aligned.  out: [M, N] with row stride ldo.  mode 0 stores, 1 adds into a float32
// out, 2 computes silu(x . W[n]) * (x . W[n + up_rows]) for n < N (W then has up_rows + N rows).
// error_flag (may be null) is set to 3 if a bounded wait inside the kernel ran out.
// A norm that the next product finishes (common.cuh, NormEmit and RowScale).  With mode 1 and `scaled`
// not null (bfloat16 [M, ld_scaled], N a multiple of 4, 16-byte aligned like norm_weight [N] in norm_dtype and
// out) the product also writes (new out) * norm_weight there and the rows' sums of squares, one part a
// tile of 256 columns, into squares = float32 [xrt_gemm_tcgen05_norm_parts(N), M].  With mode 0 or 2 and
// in_squares not null (float32 [in_parts, M]) x is such a prepared input: row m of the result is
// multiplied by 1 / sqrt(sum of the row's parts / K + eps).
XRT_EXPORT int xrt_gemm_tcgen05_normed(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                       int w_rows, int out_dtype, int mode, int up_rows, int* error_flag, void* scaled,
                                       int ld_scaled, const void* norm_weight, int norm_dtype, float* squares,
                                       const float* in_squares, int in_parts, float eps, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || mode < 0 || mode > 2) return XRT_ERR_ARGUMENT;
  if (mode == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (mode == 2 ? w_rows < up_rows + N : w_rows < N) return XRT_ERR_ARGUMENT;
  if (out_dtype != XRT_F32 && out_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (K % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return XRT_ERR_UNSUPPORTED;
  xrt::NormEmit emit;
  xrt::RowScale scale;
  if (scaled != nullptr) {
    if (mode != 1 || norm_weight == nullptr || squares == nullptr || ld_scaled < N) return XRT_ERR_ARGUMENT;
    if (N % 4 != 0 || ldo % 4 != 0 || ld_scaled % 4 != 0 || (norm_dtype != XRT_F32 && norm_dtype != XRT_BF16) ||
        (((uintptr_t)scaled | (uintptr_t)norm_weight | (uintptr_t)out) & 15) != 0)
      return XRT_ERR_UNSUPPORTED;
    emit.scaled = (__nv_bfloat16*)scaled; emit.weight = norm_weight; emit.squares = squares;
    emit.ld = ld_scaled; emit.weight_dtype = norm_dtype;
  }
  if (in_squares != nullptr) {
    if (mode == 1 || in_parts <= 0) return XRT_ERR_ARGUMENT;
    scale.squares = in_squares; scale.parts = in_parts; scale.width = K; scale.eps = eps;
  }
  if (M == 0) return XRT_OK;
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0)
      return XRT_ERR_UNSUPPORTED;
  }
  CUtensorMap map_x, map_w;
  if (!xrt::make_map(&map_x, x, M, K, ldx) || !xrt::make_map(&map_w, w, w_rows, K, K)) return XRT_ERR_UNSUPPORTED;
  if (mode == 1)
    return xrt::launch_tcgen05<1, float>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, emit, scale, stream);
  if (mode == 2) {
    if (out_dtype == XRT_BF16)
      return xrt::launch_tcgen05<2, __nv_bfloat16>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, emit, scale, stream);
    return xrt::launch_tcgen05<2, float>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, emit, scale, stream);
  }
  if (out_dtype == XRT_BF16)
    return xrt::launch_tcgen05<0, __nv_bfloat16>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, emit, scale, stream);
  return xrt::launch_tcgen05<0, float>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, emit, scale, stream);
}

// The same without a norm on either side.
XRT_EXPORT int xrt_gemm_tcgen05(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                int w_rows, int out_dtype, int mode, int up_rows, int* error_flag,
                                cudaStream_t stream) {
  return xrt_gemm_tcgen05_normed(out, x, w, M, N, K, ldx, ldo, w_rows, out_dtype, mode, up_rows, error_flag, nullptr, 0,
                                 nullptr, XRT_F32, nullptr, nullptr, 0, 0.f, stream);
}
