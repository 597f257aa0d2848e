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
#include <cuda.h>

#include "common.cuh"

namespace xrt {

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
constexpr long long TC_SPIN_LIMIT = 1ll << 24;

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase of the given parity.  False if it ran out or another role aborted.
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (long long spin = 0; spin < TC_SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 1023) == 1023 && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void tc_tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, groups of
// eight rows 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((addr & 0x3FFFF) >> 4);          // start address, bits [0, 14)
  desc |= (uint64_t)1 << 16;                          // leading byte offset (unused with swizzle), bits [16, 30)
  desc |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset, bits [32, 46)
  desc |= (uint64_t)1 << 46;                          // version, bits [46, 48)
  desc |= (uint64_t)2 << 61;                          // layout type SWIZZLE_128B, bits [61, 64)
  return desc;
}
// Instruction descriptor of kind::f16: bfloat16 A and B, float32 D, both K-major, M x N.
__host__ __device__ constexpr uint32_t tc_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
               " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld32(uint32_t (&r)[32], uint32_t addr) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(addr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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
                    TO* __restrict__ out, int M, int N, int K, int ldo, int up_rows, int* __restrict__ error_flag) {
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
    for (int s = 0; s < TC_STAGES; ++s) { tc_mbar_init(tc_smem(&full[s]), 1); tc_mbar_init(tc_smem(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { tc_mbar_init(tc_smem(&acc_full[a]), 1); tc_mbar_init(tc_smem(&acc_empty[a]), 32 * TcShape<MT>::EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)), "r"(TC_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
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
          ok = tc_mbar_wait(tc_smem(&empty[s]), ((it / TC_STAGES) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t bar = tc_smem(&full[s]);
          tc_mbar_expect_tx(bar, STAGE_A + TC_B_BYTES);
#pragma unroll
          for (int h = 0; h < MT; ++h)
            tc_tma_load_2d(tc_smem(a_stages + s * STAGE_A + h * TC_A_BYTES), &map_x, kb * TC_BK,
                           (m_blk * MT + h) * TC_BM, bar);
          const int w_row0 = n_blk * N_PER_TILE;
          const int w_row1 = MODE == 2 ? up_rows + w_row0 : w_row0 + 128;
          tc_tma_load_2d(tc_smem(b_stages + s * TC_B_BYTES), &map_w, kb * TC_BK, w_row0, bar);
          tc_tma_load_2d(tc_smem(b_stages + s * TC_B_BYTES + TC_B_BYTES / 2), &map_w, kb * TC_BK, w_row1, bar);
        }
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 3); }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instr_desc(TC_BM, TC_BN);
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tile_i) {
        const int a = tile_i % ACC_SETS;
        ok = tc_mbar_wait(tc_smem(&acc_empty[a]), ((tile_i / ACC_SETS) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + a * MT * TC_BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % TC_STAGES;
          ok = tc_mbar_wait(tc_smem(&full[s]), (it / TC_STAGES) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t desc_b = tc_smem_desc(tc_smem(b_stages + s * TC_B_BYTES));
#pragma unroll
          for (int h = 0; h < MT; ++h) {
            const uint64_t desc_a = tc_smem_desc(tc_smem(a_stages + s * STAGE_A + h * TC_A_BYTES));
#pragma unroll
            for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)  // 32 bytes further along K inside the swizzle atom
              tc_mma(tmem_d + h * TC_BN, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(tc_smem(&empty[s]));
        }
        if (ok) tc_commit(tc_smem(&acc_full[a]));
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
      ok = tc_mbar_wait(tc_smem(&acc_full[a]), (tile_i / ACC_SETS) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int row0 = (m_blk * MT + half) * TC_BM + quarter * 32;  // the warp's first row
      const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (a * MT + half) * TC_BN;
      const int col0 = n_blk * N_PER_TILE;
      // A thread holds one ROW of the accumulator; written as it is, every store instruction of the
      // warp would touch 32 lines.  The warp turns each 32 x 32 patch around in shared memory and
      // writes it with 16 bytes a lane, four whole 128-byte row pieces an instruction.
      float* patch = staging + (warp - 2) * 32 * 33;
      const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
#pragma unroll 1
      for (int c = 0; c < N_PER_TILE; c += 32) {
        uint32_t v[32];
        tc_ld32(v, tmem_row + c);
        if (MODE == 2) {
          uint32_t u[32];
          tc_ld32(u, tmem_row + TC_BN / 2 + c);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(v[j]);
            v[j] = __float_as_uint((g / (1.0f + expf(-g))) * __uint_as_float(u[j]));
          }
        } else {
          tc_wait_ld();
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
              if (MODE == 1)
                store_quad<0>(dst, old[it].x + src[0], old[it].y + src[1], old[it].z + src[2], old[it].w + src[3]);
              else
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
      tc_fence_before();
      tc_mbar_arrive(tc_smem(&acc_empty[a]));
    }
    if (!ok && lane == 0) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 3); }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// A map over a row-major bfloat16 matrix [rows, cols] with row stride ld, boxes of 128 rows x 64 columns.
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
  EncodeTiledFn encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, 128u};
  const cuuint32_t elem[2] = {1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE, int MT, typename TO>
int launch_tcgen05_tiled(void* out, const CUtensorMap& map_x, const CUtensorMap& map_w, int M, int N, int K, int ldo,
                         int up_rows, int* error_flag, int sm_count, cudaStream_t stream) {
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
  kernel<<<blocks, TcShape<MT>::THREADS, TcShape<MT>::SMEM, stream>>>(map_x, map_w, (TO*)out, M, N, K, ldo, up_rows,
                                                                      error_flag);
  return launch_status();
}

// Tiles of 256 rows for products of few tiles, when they keep the multiprocessors about as busy as
// tiles of 128 rows would (the larger tile moves a third fewer operand bytes per flop and drains its
// accumulator with twice the warps; with many tiles the overlap of the small tile's two accumulators wins).
// Tuning::gemm_tile_rows = 128 or 256 forces one, for comparison.
template <int MODE, typename TO>
int launch_tcgen05(void* out, const CUtensorMap& map_x, const CUtensorMap& map_w, int M, int N, int K, int ldo,
                   int up_rows, int* error_flag, int sm_count, cudaStream_t stream) {
  constexpr int n_per_tile = MODE == 2 ? TC_BN / 2 : TC_BN;
  const long long tiles_n = (N + n_per_tile - 1) / n_per_tile;
  auto busy = [&](long long tiles) { return (double)tiles / (double)(((tiles + sm_count - 1) / sm_count) * sm_count); };
  const long long small_tiles = ((M + 127) / 128) * tiles_n;
  const double small = busy(small_tiles), large = 1.25 * busy(((M + 255) / 256) * tiles_n);
  const int forced = tuning().gemm_tile_rows;
  // measured at 2,048 and 8,192 rows: the large tile wins where the small one leaves under two rounds of work
  const bool use_large = forced == 256 || (forced != 128 && M > 128 && small_tiles <= 2 * sm_count && large > small);
  if (use_large)
    return launch_tcgen05_tiled<MODE, 2, TO>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, stream);
  return launch_tcgen05_tiled<MODE, 1, TO>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, stream);
}

}  // namespace xrt

// x: bfloat16 [M, K] with row stride ldx; w: bfloat16 [rows, K] contiguous; K and ldx multiples of 8,
// both bases 16-byte aligned.  out: [M, N] with row stride ldo.  mode 0 stores, 1 adds into a float32
// out, 2 computes silu(x . W[n]) * (x . W[n + up_rows]) for n < N (W then has up_rows + N rows).
// error_flag (may be null) is set to 3 if a bounded wait inside the kernel ran out.
XRT_EXPORT int xrt_gemm_tcgen05(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                int w_rows, int out_dtype, int mode, int up_rows, int* error_flag,
                                cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || mode < 0 || mode > 2) return XRT_ERR_ARGUMENT;
  if (mode == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (mode == 2 ? w_rows < up_rows + N : w_rows < N) return XRT_ERR_ARGUMENT;
  if (out_dtype != XRT_F32 && out_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (K % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return XRT_ERR_UNSUPPORTED;
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
  if (mode == 1) return xrt::launch_tcgen05<1, float>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, stream);
  if (mode == 2) {
    if (out_dtype == XRT_BF16)
      return xrt::launch_tcgen05<2, __nv_bfloat16>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, stream);
    return xrt::launch_tcgen05<2, float>(out, map_x, map_w, M, N, K, ldo, up_rows, error_flag, sm_count, stream);
  }
  if (out_dtype == XRT_BF16)
    return xrt::launch_tcgen05<0, __nv_bfloat16>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, stream);
  return xrt::launch_tcgen05<0, float>(out, map_x, map_w, M, N, K, ldo, 0, error_flag, sm_count, stream);
}
