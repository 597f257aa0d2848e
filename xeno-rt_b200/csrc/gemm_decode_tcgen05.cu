// Y[M, N] = X[M, K] . W[N, K]^T for few rows (decode steps) on the fifth-generation tensor cores,
// with the operands swapped: the WEIGHT rows are the MMA's 128 lanes (M of tcgen05.mma), the batch
// rows its N (16 .. 128), so that a step of a handful of sequences still fills the tensor core's
// rows, and the product's time is the time to stream W from HBM.
//
// The reference streams each weight row once per token (crates/xrt-kernels/src/cpu/matmul.rs:100-192,
// 194-320).  Here the weight is streamed by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a deep
// ring of shared-memory stages: no registers are held by bytes in flight, and a persistent block
// per multiprocessor never drains its pipeline between work items.
//
// Work items are (tile of 128 weight rows, split of K).  K is split so that the items fill the
// multiprocessors evenly even when N is small; every split writes its 128 x NB partial sums to
// scratch memory, and the block that finishes a tile's last split (found with one atomic counter a
// tile, no block ever waits for another) adds the partials IN SPLIT ORDER and applies the epilogue:
// the result does not depend on which block came last, nor on the number of rows M.
// Epilogues: store (32-bit or bfloat16), add into the 32-bit residual stream, SwiGLU (an item then
// streams 128 gate rows and the 128 matching up rows into two accumulators).
//
// Where all items of a launch run at once (tiles x splits is no more than the multiprocessors), the
// splits of a tile are the blocks of one thread-block cluster instead, if the device holds so many
// clusters of that size at once: each block sends its partial sums for a share of the tile's rows to the
// block that finishes them (remote stores into shared memory that the ring never uses), the cluster
// meets once, and every block adds and finishes its rows locally, again in split order: no scratch in
// global memory, no fence, no counter.  Such a finish can also prepare the RMSNorm that follows a
// product that adds into the residual stream (NormEmit), and every epilogue can finish a norm that the
// product before prepared (RowScale).
//
// The weight is read once a step: its TMA loads carry an evict-first policy for the L2, so that what the
// step reads again (activations, the residual, partial sums, code) stays there.  How many splits a product
// gets, and whether they meet as a cluster, is decided from measured costs (choose_splits).
//
// Six warps: warp 0 issues TMA loads, warp 1 owns TMEM and issues the MMAs, warps 2-5 read the
// accumulators (tcgen05.ld, one TMEM lane quarter each) while the MMA warp fills the other
// accumulator.  Every mbarrier wait is bounded; a wait that runs out raises the error flag and an
// abort flag, all roles leave their loops, TMEM is freed and the block returns.
#include "tcgen05.cuh"

namespace xrt {

using namespace sm100;

constexpr int DG_ROWS = 128, DG_BK = 64, DG_UMMA_K = 16;
constexpr int DG_W_BYTES = DG_ROWS * DG_BK * 2;  // 16 KB: one slab of one group of weight rows
constexpr int DG_THREADS = 192;
constexpr int DG_MAX_SPLITS = 8;

// The two halves of a cluster meeting, thread by thread: a block may store into another block's shared
// memory only once that block runs, which the first meeting (arrive at the start, wait before the first
// store) makes sure of without holding anybody up.
__device__ __forceinline__ void dg_cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void dg_cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ void dg_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Weight rows of a tile that one block of a cluster finishes: ceil(128 / splits), rounded up to a
// multiple of 4 so that a thread can take four rows at once; the last block has the remainder.
__host__ __device__ inline int dg_rows_per_block(int splits) { return ((DG_ROWS + splits - 1) / splits + 3) & ~3; }

// x * sigmoid(x) for a result of type TO.  A bfloat16 result keeps 8 bits: the fast exponential and
// division (2 ulp of 32-bit each) change none of them, and are a tenth of the instructions, which is
// what an epilogue that runs once a block pays for (its code comes cold from the L2).
template <typename TO> __device__ __forceinline__ float silu_for(float x) { return x / (1.0f + expf(-x)); }
template <> __device__ __forceinline__ float silu_for<__nv_bfloat16>(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

__device__ __forceinline__ void store_four(float* dst, const float (&v)[4]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_four(__nv_bfloat16* dst, const float (&v)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

struct DecodeGemmShape {
  int M, N, K, ldo;
  int nb;            // batch rows padded to a multiple of 16: the MMA's N
  int tiles;         // tiles of 128 weight rows
  int splits;        // splits of K
  int k_per_split;   // 64-wide slabs a split
  int up_rows;       // SwiGLU: the up rows start this many rows after the gate rows
  int stages;        // ring depth
  int tmem_cols;     // power of two >= 2 accumulators
  int clustered;     // the splits of a tile are one cluster; one item a block
};

// MODE 0: store, 1: add into float out, 2: SwiGLU.
template <int MODE, typename TO>
__global__ void __launch_bounds__(DG_THREADS, 1)
gemm_decode_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           TO* __restrict__ out, float* __restrict__ partial, int* __restrict__ counters,
                           const DecodeGemmShape shape, int* __restrict__ error_flag, const RowScale scale,
                           const NormEmit emit) {
  constexpr int GROUPS = MODE == 2 ? 2 : 1;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int x_bytes = shape.nb * DG_BK * 2;
  const int stage_bytes = GROUPS * DG_W_BYTES + ((x_bytes + 1023) & ~1023);
  const int stages = shape.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + stages;
  uint64_t* acc_full = bars + 2 * stages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;
  float* row_inv = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes + 512);  // [nb] when the input's norm is pending
  float* recv = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes + 1024);    // the cluster's sums for this block's rows

  pdl_trigger();
  if (shape.clustered) dg_cluster_arrive();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = shape.tiles * shape.splits;
  const int k_iters_total = (shape.K + DG_BK - 1) / DG_BK;
  const int acc_cols = GROUPS * shape.nb;  // TMEM columns of one accumulator set

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(smem_u32(&full[s]), 2); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&acc_full[a]), 1); mbar_init(smem_u32(&acc_empty[a]), 128); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(shape.tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> (tile, split); consecutive items are the splits of one tile
  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      // The walk over this block's slabs: items in turn, and inside an item the slabs of its split of K.
      // Blocks that work at the same time start their walk over K at different slabs (a rotation that
      // depends on the tile only, so the order of the sum is fixed per output element): otherwise every
      // block asks the L2 for the same few lines of X at the same moment.
      struct Walk {
        int item, i, span, kb0, rotate, tile;
        __device__ void enter(const DecodeGemmShape& sh, int k_total) {
          tile = item / sh.splits;
          kb0 = (item % sh.splits) * sh.k_per_split;
          span = max(0, min(k_total, kb0 + sh.k_per_split) - kb0);
          rotate = span > 0 ? (tile * 5) % span : 0;
          i = 0;
        }
        __device__ bool settle(const DecodeGemmShape& sh, int k_total, int n_items, int stride) {
          while (item < n_items) {  // skips items without slabs (a split beyond K)
            if (i < span) return true;
            item += stride;
            if (item < n_items) enter(sh, k_total);
          }
          return false;
        }
        __device__ int kb() const { return kb0 + (i + rotate) % span; }
      };
      Walk walk;
      walk.item = blockIdx.x;
      if (walk.item < n_items) walk.enter(shape, k_iters_total);
      const uint32_t w_bytes = GROUPS * DG_W_BYTES;
      // a weight is read once a step: its lines leave the L2 first, and what the step reads again
      // (activations, the residual, the partial sums, the kernels' code) stays (measured at the
      // 8B shape, context 4096: 4 to 7 percent of a step of 17 to 64 sequences)
      const uint64_t once = policy_evict_first();
      auto load_w = [&](const Walk& at, int s) {
        const uint32_t bar = smem_u32(&full[s]);
        unsigned char* stage = smem + (size_t)s * stage_bytes;
        mbar_arrive_expect_tx(bar, w_bytes);
        tma_load_2d(smem_u32(stage), &map_w, at.kb() * DG_BK, at.tile * DG_ROWS, bar, once);
        if (MODE == 2) tma_load_2d(smem_u32(stage + DG_W_BYTES), &map_w, at.kb() * DG_BK, shape.up_rows + at.tile * DG_ROWS, bar, once);
      };
      auto load_x = [&](const Walk& at, int s) {
        const uint32_t bar = smem_u32(&full[s]);
        mbar_arrive_expect_tx(bar, x_bytes);
        tma_load_2d(smem_u32(smem + (size_t)s * stage_bytes + GROUPS * DG_W_BYTES), &map_x, at.kb() * DG_BK, 0, bar);
      };
      // The weights do not depend on the step: the whole ring is filled with them while the kernel
      // before this one finishes.  X does: its loads follow once that kernel has completed.  A stage's
      // barrier takes two arrivals (weights asked for, X asked for) and the bytes of both.
      Walk ahead = walk;
      int filled = 0;
      while (filled < stages && ahead.settle(shape, k_iters_total, n_items, gridDim.x)) {
        load_w(ahead, filled);
        ++ahead.i;
        ++filled;
      }
      pdl_wait();
      int it = 0;
      bool ok = true;
      while (it < filled && walk.settle(shape, k_iters_total, n_items, gridDim.x)) {
        load_x(walk, it);
        ++walk.i;
        ++it;
      }
      while (ok && walk.settle(shape, k_iters_total, n_items, gridDim.x)) {
        const int s = it % stages;
        ok = mbar_wait(smem_u32(&empty[s]), ((it / stages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        load_w(walk, s);
        load_x(walk, s);
        ++walk.i;
        ++it;
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 4); }
    }
    if (shape.clustered) dg_cluster_wait();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc(DG_ROWS, shape.nb);
      int it = 0, item_i = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_i) {
        const int split = item % shape.splits;
        const int kb0 = split * shape.k_per_split;
        const int kb1 = min(k_iters_total, kb0 + shape.k_per_split);
        const int a = item_i & 1;
        ok = mbar_wait(smem_u32(&acc_empty[a]), ((item_i >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        fence_after();
        const uint32_t tmem_d = tmem_base + a * acc_cols;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {  // the slabs arrive in the producer's rotated order
          const int s = it % stages;
          ok = mbar_wait(smem_u32(&full[s]), (it / stages) & 1, abort_flag);
          if (!ok) break;
          fence_after();
          unsigned char* stage = smem + (size_t)s * stage_bytes;
          const uint64_t desc_x = desc_k_major(smem_u32(stage + GROUPS * DG_W_BYTES));
#pragma unroll
          for (int gr = 0; gr < GROUPS; ++gr) {
            const uint64_t desc_w = desc_k_major(smem_u32(stage + gr * DG_W_BYTES));
#pragma unroll
            for (int k = 0; k < DG_BK / DG_UMMA_K; ++k)
              mma_f16(tmem_d + gr * shape.nb, desc_w + 2 * k, desc_x + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          commit(smem_u32(&empty[s]));
        }
        if (ok) commit(smem_u32(&acc_full[a]));
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 4); }
    }
    if (shape.clustered) dg_cluster_wait();
  } else {
    // ---------------------------------------------------------------- epilogue
    if (shape.clustered) dg_cluster_wait();  // every block of the cluster runs: its shared memory may be written
    pdl_wait();  // the output (and the residual it adds into) belongs to the step
    if (scale.squares != nullptr) {
      // 1 / rms of every batch row from the parts the product before this one left: sixteen lanes a row
      // take every sixteenth part each and meet in a fixed order
      const int tid = threadIdx.x - 64, sub = tid & 15;
      for (int m = tid >> 4; m < shape.nb; m += 8) {
        float sum = 0.f;
        if (m < shape.M)
          for (int p = sub; p < scale.parts; p += 16) sum += __ldcg(scale.squares + (size_t)p * shape.M + m);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (sub == 0) row_inv[m] = m < shape.M ? 1.0f / sqrtf(sum / (float)scale.width + scale.eps) : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const bool scaled = scale.squares != nullptr;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;  // weight row inside the tile = TMEM lane
    int item_i = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++item_i) {
      const int tile = item / shape.splits, split = item % shape.splits;
      const int kb0 = split * shape.k_per_split;
      const bool has_k = kb0 < k_iters_total;  // a split beyond K (uneven division) contributes zeros
      const int a = item_i & 1;
      const int n = tile * DG_ROWS + r;  // output column = weight row
      const uint32_t tmem_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + a * acc_cols;
      if (has_k) {
        ok = mbar_wait(smem_u32(&acc_full[a]), (item_i >> 1) & 1, abort_flag);
        if (!ok) break;
        fence_after();
      }
      if (shape.splits == 1) {
        // one split: straight to the output
        for (int c = 0; c < shape.nb; c += 16) {
          uint32_t v[16], u[16];
          tmem_ld16(v, tmem_row + c);
          if (MODE == 2) tmem_ld16(u, tmem_row + shape.nb + c);
          tmem_wait_ld();
          if (n < shape.N) {
            // the residual values first, all sixteen loads in flight (a load may not pass a store that
            // could alias it: read-modify-write one value at a time would wait for each in turn)
            float old[16];
            if (MODE == 1) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                old[j] = c + j < shape.M ? __ldcg(reinterpret_cast<const float*>(out) + (size_t)(c + j) * shape.ldo + n) : 0.f;
            }
            // sixteen values worked out side by side (rows beyond M too: their stores are left out), so
            // that one element's exponential and division do not wait for the one before it
            float val[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float inv = scaled ? row_inv[c + j] : 1.f;
              val[j] = __uint_as_float(v[j]) * inv;
              if (MODE == 2) val[j] = silu_for<TO>(val[j]) * (__uint_as_float(u[j]) * inv);
              if (MODE == 1) val[j] += old[j];
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < shape.M) out[(size_t)(c + j) * shape.ldo + n] = from_float<TO>(val[j]);
          }
        }
      } else if (shape.clustered) {
        // This split's sums go to the blocks of the cluster that finish them: block d of the cluster owns
        // rows d * per .. of the tile, and keeps one slot a split, [slot][accumulator column][row], in a
        // part of its shared memory that its own ring never uses.  Remote stores, no reply awaited.
        const int per = dg_rows_per_block(shape.splits);
        const int owner = r / per, local = r - owner * per;
        uint32_t remote;
        asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(recv)), "r"(owner));
        remote += (uint32_t)((split * acc_cols * per + local) * 4);
        for (int c = 0; c < acc_cols; c += 16) {
          uint32_t v[16];
          if (has_k) { tmem_ld16(v, tmem_row + c); tmem_wait_ld(); }
#pragma unroll
          for (int j = 0; j < 16; ++j)
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)((c + j) * per * 4)),
                         "f"(has_k ? __uint_as_float(v[j]) : 0.f) : "memory");
        }
      } else {
        // partial[(tile * splits + split)][group][weight row][NB]: a thread owns its row's NB floats
        float* mine = partial + ((size_t)item * GROUPS) * DG_ROWS * shape.nb;
        for (int c = 0; c < acc_cols; c += 16) {
          uint32_t v[16];
          if (has_k) { tmem_ld16(v, tmem_row + c); tmem_wait_ld(); }
          const int gr = c / shape.nb, col = c - gr * shape.nb;
          float4* dst4 = reinterpret_cast<float4*>(mine + ((size_t)gr * DG_ROWS + r) * shape.nb + col);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst4[j] = has_k ? make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                          __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      if (has_k) {
        fence_before();
        mbar_arrive(smem_u32(&acc_empty[a]));
      }
      if (shape.splits > 1 && !shape.clustered) {
        // the block that brings a tile's last split adds the partials in split order
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (threadIdx.x == 64) {
          const int before = atomicAdd(&counters[tile], 1);
          *last_flag = before == shape.splits - 1;
          if (before == shape.splits - 1) counters[tile] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          const float* first = partial + ((size_t)tile * shape.splits * GROUPS) * DG_ROWS * shape.nb;
          const size_t split_stride = (size_t)GROUPS * DG_ROWS * shape.nb;
          if (n < shape.N) {
            // sixteen batch rows at a time, every split's partial loaded (16 bytes a load) before the
            // first is added: the loads are in flight together, the additions stay in split order
            for (int m0 = 0; m0 < shape.M; m0 += 16) {
              float sums[GROUPS][16];
#pragma unroll
              for (int gr = 0; gr < GROUPS; ++gr) {
                float4 part[DG_MAX_SPLITS][4];
                const float* row = first + ((size_t)gr * DG_ROWS + r) * shape.nb + m0;
#pragma unroll
                for (int s = 0; s < DG_MAX_SPLITS; ++s)
#pragma unroll
                  for (int q = 0; q < 4; ++q)
                    part[s][q] = s < shape.splits ? __ldcg(reinterpret_cast<const float4*>(row + s * split_stride) + q)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                  for (int s = 0; s < DG_MAX_SPLITS; ++s) {
                    t.x += part[s][q].x; t.y += part[s][q].y; t.z += part[s][q].z; t.w += part[s][q].w;
                  }
                  sums[gr][4 * q] = t.x; sums[gr][4 * q + 1] = t.y; sums[gr][4 * q + 2] = t.z; sums[gr][4 * q + 3] = t.w;
                }
              }
              float old[16];
              if (MODE == 1) {  // all sixteen residual loads in flight before the first store
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  old[j] = m0 + j < shape.M ? __ldcg(reinterpret_cast<const float*>(out) + (size_t)(m0 + j) * shape.ldo + n) : 0.f;
              }
              float val[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float inv = scaled ? row_inv[m0 + j] : 1.f;
                val[j] = sums[0][j] * inv;
                if (MODE == 2) val[j] = silu_for<TO>(val[j]) * (sums[GROUPS - 1][j] * inv);
                if (MODE == 1) val[j] += old[j];
              }
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (m0 + j < shape.M) out[(size_t)(m0 + j) * shape.ldo + n] = from_float<TO>(val[j]);
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // last_flag is rewritten for the next item
      }
    }
    if (!ok && lane == 0) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 4); }
  }

  if (shape.clustered) {
    // Every thread of every block of the cluster comes here, also after a wait that ran out (all waits
    // are bounded).  After the meeting every split's sums for this block's rows lie in its own shared
    // memory; it adds them in split order and finishes its rows: consecutive threads take consecutive
    // weight rows (consecutive output addresses) of one batch row.  Nothing touches another block's
    // memory after the meeting, so a block may leave when it is done.
    dg_cluster_sync();
    if (warp >= 2 && !*abort_flag) {
      uint32_t rank;
      asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
      const int tile = blockIdx.x / shape.splits;
      const int per = dg_rows_per_block(shape.splits);
      const int row_lo = (int)rank * per;
      const int rows_here = max(0, min(per, DG_ROWS - row_lo));
      const int slot_floats = acc_cols * per;
      const int n_lo = tile * DG_ROWS + row_lo;
      // Four weight rows a thread where the output allows it (16 bytes of shared memory a split, one
      // load and one store of four outputs): the four warps have little else to hide latency behind,
      // so the loop's cost is its instruction count.  per, row_lo and rows_here are multiples of 4.
      const bool by_four = shape.N % 4 == 0 && shape.ldo % 4 == 0 && ((uintptr_t)out & (sizeof(TO) * 4 - 1)) == 0;
      if (by_four) {
        // after the meeting nothing is left in flight into this block's ring: room for the shares of
        // the sums of squares, [batch row][four weight rows]
        float* square_parts = reinterpret_cast<float*>(smem);
        const int quads = rows_here / 4;
        const int total = quads * shape.M;
        constexpr int UNROLL = 1;
#pragma unroll 1
        for (int base = threadIdx.x - 64; base < total; base += 128 * UNROLL) {
          float4 old[UNROLL], sums[UNROLL][GROUPS];
          int m_of[UNROLL], n_of[UNROLL];
          bool live[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const int idx = base + u * 128;
            const int m = idx / quads, local = (idx - m * quads) * 4;
            m_of[u] = m;
            n_of[u] = n_lo + local;
            live[u] = idx < total && n_of[u] < shape.N;
            old[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (MODE == 1 && live[u])
              old[u] = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(out) + (size_t)m * shape.ldo + n_of[u]));
#pragma unroll
            for (int gr = 0; gr < GROUPS; ++gr) {
              float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
              if (live[u]) {
                const float* mine = recv + (size_t)(gr * shape.nb + m) * per + local;
                for (int sp = 0; sp < shape.splits; ++sp) {
                  const float4 part = *reinterpret_cast<const float4*>(mine + (size_t)sp * slot_floats);
                  t.x += part.x; t.y += part.y; t.z += part.z; t.w += part.w;
                }
              }
              sums[u][gr] = t;
            }
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            if (!live[u]) continue;
            const float inv = scale.squares != nullptr ? row_inv[m_of[u]] : 1.f;
            float val[4] = {sums[u][0].x * inv, sums[u][0].y * inv, sums[u][0].z * inv, sums[u][0].w * inv};
            if (MODE == 2) {
              const float4 up = sums[u][GROUPS - 1];
              const float ups[4] = {up.x * inv, up.y * inv, up.z * inv, up.w * inv};
#pragma unroll
              for (int j = 0; j < 4; ++j) val[j] = silu_for<TO>(val[j]) * ups[j];
            }
            if (MODE == 1) { val[0] += old[u].x; val[1] += old[u].y; val[2] += old[u].z; val[3] += old[u].w; }
            store_four(out + (size_t)m_of[u] * shape.ldo + n_of[u], val);
            if (MODE == 1 && emit.scaled != nullptr) {
              // the norm that follows: new residual * its weight for the next product, and this thread's
              // share of the row's sum of squares, to be added in a fixed order below
              float w4[4];
              if (emit.weight_dtype == XRT_BF16) {
                const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(emit.weight) + n_of[u]);
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                w4[0] = lo.x; w4[1] = lo.y; w4[2] = hi.x; w4[3] = hi.y;
              } else {
                const float4 raw = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(emit.weight) + n_of[u]);
                w4[0] = raw.x; w4[1] = raw.y; w4[2] = raw.z; w4[3] = raw.w;
              }
              const float scaled4[4] = {val[0] * w4[0], val[1] * w4[1], val[2] * w4[2], val[3] * w4[3]};
              store_four(emit.scaled + (size_t)m_of[u] * emit.ld + n_of[u], scaled4);
              square_parts[base + u * 128] = (val[0] * val[0] + val[1] * val[1]) + (val[2] * val[2] + val[3] * val[3]);
            }
          }
          if (MODE == 1 && emit.scaled != nullptr) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
              if (!live[u] && base + u * 128 < total) square_parts[base + u * 128] = 0.f;  // rows beyond N
          }
        }
        if (MODE == 1 && emit.squares != nullptr) {
          // part (this block) of every batch row's sum of squares: its threads' shares in row order
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int m = threadIdx.x - 64; m < shape.M; m += 128) {
            float sum = 0.f;
            for (int q = 0; q < quads; ++q) sum += square_parts[m * quads + q];
            emit.squares[(size_t)blockIdx.x * shape.M + m] = sum;
          }
        }
      } else {
        const int total = rows_here * shape.M;
        for (int idx = threadIdx.x - 64; idx < total; idx += 128) {
          const int m = idx / rows_here, local = idx - m * rows_here;
          const int n = n_lo + local;
          if (n >= shape.N) continue;
          const float inv = scale.squares != nullptr ? row_inv[m] : 1.f;
          float sums[GROUPS];
#pragma unroll
          for (int gr = 0; gr < GROUPS; ++gr) {
            const float* mine = recv + (size_t)(gr * shape.nb + m) * per + local;
            float t = 0.f;
            for (int sp = 0; sp < shape.splits; ++sp) t += mine[(size_t)sp * slot_floats];
            sums[gr] = t;
          }
          float val = sums[0] * inv;
          if (MODE == 2) val = (val / (1.0f + expf(-val))) * (sums[GROUPS - 1] * inv);
          TO* dst = out + (size_t)m * shape.ldo + n;
          if (MODE == 1) *dst = from_float<TO>(*reinterpret_cast<const float*>(dst) + val);
          else *dst = from_float<TO>(val);
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(shape.tmem_cols));
  }
}

static bool dg_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  return sm100::make_map_bf16_2d(map, base, rows, cols, ld, box_rows);
}

// The kernel's limit of dynamic shared memory only ever grows (setting it anew would lower it): one
// record for each instance of the kernel.
template <int MODE, typename TO>
cudaError_t allow_shared_memory(int smem) {
  static int allowed = 0;
  if (smem <= allowed) return cudaSuccess;
  const cudaError_t err = cudaFuncSetAttribute(gemm_decode_tcgen05_kernel<MODE, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err == cudaSuccess) allowed = smem;
  return err;
}

// How many clusters of 2 .. 8 blocks of this kernel (one block a multiprocessor) the device runs at
// the same time: asked of the current device once; where there is none (host arithmetic only), or
// it has another number of multiprocessors than asked about, nine tenths of them, which is what a
// B200 answers within one cluster (148: 45 clusters of 3, 33 of 4, 26 of 5, 22 of 6).
struct ClusterLimits { int sms; int held[9]; };
static ClusterLimits ask_cluster_limits() {
  ClusterLimits asked = {};
  int device = 0, count = 0;
  if (cudaGetDevice(&device) == cudaSuccess &&
      cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess) {
    auto kernel = gemm_decode_tcgen05_kernel<0, __nv_bfloat16>;
    const int smem = 200 * 1024;
    bool ok = allow_shared_memory<0, __nv_bfloat16>(smem) == cudaSuccess;
    for (int size = 2; ok && size <= 8; ++size) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(size, 1, 1);
      probe.blockDim = dim3(DG_THREADS);
      probe.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      probe.attrs = attr;
      probe.numAttrs = 1;
      int clusters = 0;
      ok = cudaOccupancyMaxActiveClusters(&clusters, kernel, &probe) == cudaSuccess;
      asked.held[size] = clusters;
    }
    if (ok) asked.sms = count;
  }
  cudaGetLastError();  // no device, or a refusal: an answer, not an error of a stream
  return asked;
}
static ClusterLimits cluster_limits(int sms) {
  static const ClusterLimits asked = ask_cluster_limits();  // once, whichever thread comes first
  if (sms == asked.sms) return asked;
  ClusterLimits estimate = {};
  estimate.sms = sms;
  for (int size = 2; size <= 8; ++size) estimate.held[size] = sms * 9 / 10 / size;
  return estimate;
}

// Tuning::decode_gemm_clusters = false keeps the scratch-and-counter reduction everywhere, for comparison.
inline bool decode_gemm_clusters_wanted() { return tuning().decode_gemm_clusters; }

// Splits of K: more splits fill the multiprocessors more evenly when the tiles are few, but every
// split has its price.  Where all items run at once and the device holds a tile's splits as one
// cluster, they meet through shared memory: a ramp, a meeting and a short finish, measured about
// the time of 350 KB of weights an item.  Else every split writes and the last reads a 128 x NB
// partial tile, with a fence, a counter, and one block that finishes all of a tile's rows: the time of
// 450 KB an item at NB = 16, growing with NB (12 microseconds at 64 rows).  The choice minimises
// (weight bytes + that) / (share of the block rounds that do work).  It depends on N, K and the
// padded batch NB (16, 32, ... 128), so a row's sum has the same order for every batch of the same
// NB; between NB classes it may differ by rounding.  At least 4 slabs a split.
static int choose_splits(int tiles, int k_iters, int sms, int groups, int nb) {
  int best = 1;
  double best_cost = 0.0;
  const double weight_bytes = (double)groups * DG_ROWS * k_iters * DG_BK * 2;
  const ClusterLimits limits = cluster_limits(sms);
  const bool clusters = decode_gemm_clusters_wanted();
  for (int s = 1; s <= DG_MAX_SPLITS; ++s) {
    const int per = (k_iters + s - 1) / s;
    if (s > 1 && per < 4) break;
    if ((s - 1) * per >= k_iters) continue;  // the last split would be empty
    const long long items = (long long)tiles * s;
    const long long rounds = (items + sms - 1) / sms;
    const double busy = (double)items / (double)(rounds * sms);
    double split_bytes = 0.0;
    if (s > 1 && s <= 8 && clusters && items <= sms && tiles <= limits.held[s])
      split_bytes = s * 350.0 * 1024;
    else if (s > 1)
      split_bytes = 2.0 * s * groups * nb * DG_ROWS * 4 + s * 450.0 * 1024 * (0.75 + nb / 64.0);
    const double cost = (weight_bytes + split_bytes) / busy;
    if (s == 1 || cost < best_cost * 0.98) { best_cost = cost; best = s; }
  }
  return best;
}


// Whether the splits of a tile run as one cluster: all clusters of the launch must find room at the
// same time (asked once for each cluster size and shared-memory size).
template <int MODE, typename TO>
bool decode_gemm_as_clusters(const DecodeGemmShape& shape, int smem, int sm_count) {
  auto kernel = gemm_decode_tcgen05_kernel<MODE, TO>;
  const int items = shape.tiles * shape.splits;
  if (!(shape.splits > 1 && shape.splits <= 8 && items <= sm_count && decode_gemm_clusters_wanted())) return false;
  if (allow_shared_memory<MODE, TO>(smem) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  static int held[9] = {}, held_smem[9] = {};  // clusters at once by cluster size: 0 unknown, -1 none
  if (held[shape.splits] == 0 || held_smem[shape.splits] != smem) {
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(shape.splits, 1, 1);
    probe.blockDim = dim3(DG_THREADS);
    probe.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = shape.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    probe.attrs = attr;
    probe.numAttrs = 1;
    int clusters = 0;
    const bool asked = cudaOccupancyMaxActiveClusters(&clusters, kernel, &probe) == cudaSuccess;
    cudaGetLastError();  // a refusal here is an answer, not an error of the stream
    held[shape.splits] = (asked && clusters >= 1) ? clusters : -1;
    held_smem[shape.splits] = smem;
  }
  return held[shape.splits] >= shape.tiles;
}

template <int MODE, typename TO>
int launch_decode_gemm(void* out, float* partial, int* counters, const CUtensorMap& map_w, const CUtensorMap& map_x,
                       DecodeGemmShape shape, int smem, int blocks, int sm_count, int* error_flag, const RowScale& scale,
                       const NormEmit& emit, cudaStream_t stream) {
  auto kernel = gemm_decode_tcgen05_kernel<MODE, TO>;
  const cudaError_t err = allow_shared_memory<MODE, TO>(smem);
  if (err != cudaSuccess) return (int)err;
  const int items = shape.tiles * shape.splits;
  shape.clustered = decode_gemm_as_clusters<MODE, TO>(shape, smem, sm_count) ? 1 : 0;
  if (emit.scaled != nullptr && !shape.clustered) return XRT_ERR_UNSUPPORTED;  // only the clusters' finish prepares a norm
  if (!shape.clustered) {
    launch_kernel(kernel, dim3(blocks), dim3(DG_THREADS), (size_t)smem, stream, map_w, map_x, (TO*)out, partial, counters,
                  shape, error_flag, scale, emit);
    return launch_status();
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(items);
  config.blockDim = dim3(DG_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n_attrs = 0;
  if (pdl_enabled()) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
  attrs[n_attrs].val.clusterDim.x = shape.splits; attrs[n_attrs].val.clusterDim.y = 1; attrs[n_attrs].val.clusterDim.z = 1;
  ++n_attrs;
  config.attrs = attrs;
  config.numAttrs = n_attrs;
  cudaLaunchKernelEx(&config, kernel, map_w, map_x, (TO*)out, partial, counters, shape, error_flag, scale, emit);
  return launch_status();
}

}  // namespace xrt

// How much scratch a call needs: floats of `partial` (0 when K is not split).  The same
// arithmetic as the launcher's, for the caller that allocates.
XRT_EXPORT long long xrt_gemm_decode_tcgen05_scratch(int M, int N, int K, int mode, int sm_count) {
  const int tiles = (N + xrt::DG_ROWS - 1) / xrt::DG_ROWS;
  const int k_iters = (K + xrt::DG_BK - 1) / xrt::DG_BK;
  const int splits = xrt::choose_splits(tiles, k_iters, sm_count, mode == 2 ? 2 : 1, (M + 15) / 16 * 16);
  if (splits == 1) return 0;
  const int nb = (M + 15) / 16 * 16;
  return (long long)tiles * splits * (mode == 2 ? 2 : 1) * nb * xrt::DG_ROWS;
}

// What the launcher would do with this product: plan[0] = tiles of 128 weight rows, plan[1] = splits of K,
// plan[2] = 1 if the splits of a tile would meet as a cluster (by the device's limits where there is a
// device, by their estimate else), 0 if through scratch and the merging block or if K is not split.
// The caller that has another kernel for few rows uses it to decide between the two.
XRT_EXPORT int xrt_gemm_decode_tcgen05_plan(int M, int N, int K, int mode, int sm_count, int* plan) {
  if (M <= 0 || N <= 0 || K <= 0 || sm_count <= 0 || plan == nullptr) return XRT_ERR_ARGUMENT;
  const int tiles = (N + xrt::DG_ROWS - 1) / xrt::DG_ROWS;
  const int k_iters = (K + xrt::DG_BK - 1) / xrt::DG_BK;
  const int splits = xrt::choose_splits(tiles, k_iters, sm_count, mode == 2 ? 2 : 1, (M + 15) / 16 * 16);
  plan[0] = tiles;
  plan[1] = splits;
  plan[2] = splits > 1 && splits <= 8 && xrt::decode_gemm_clusters_wanted() && (long long)tiles * splits <= sm_count &&
                    tiles <= xrt::cluster_limits(sm_count).held[splits]
                ? 1 : 0;
  return XRT_OK;
}

namespace xrt {

// Sizes of a launch from the sizes of the product (host arithmetic): the shape the kernel gets, its
// dynamic shared memory and its blocks when the splits are not clusters.
static int plan_decode_gemm(int M, int N, int K, int ldo, int mode, int up_rows, int sm_count, DecodeGemmShape* shape_out,
                            int* smem_out, int* blocks_out) {
  DecodeGemmShape shape;
  shape.M = M; shape.N = N; shape.K = K; shape.ldo = ldo;
  shape.nb = (M + 15) / 16 * 16;
  shape.tiles = (N + DG_ROWS - 1) / DG_ROWS;
  const int k_iters = (K + DG_BK - 1) / DG_BK;
  shape.splits = choose_splits(shape.tiles, k_iters, sm_count, mode == 2 ? 2 : 1, shape.nb);
  shape.k_per_split = (k_iters + shape.splits - 1) / shape.splits;
  shape.up_rows = up_rows;
  const int groups = mode == 2 ? 2 : 1;
  const int x_bytes = shape.nb * DG_BK * 2;
  const int stage_bytes = groups * DG_W_BYTES + ((x_bytes + 1023) & ~1023);
  // where K is split, a block also keeps the cluster's sums for its share of a tile's rows:
  // splits x accumulator columns x rows a block finishes, floats
  const int per = shape.splits > 1 ? dg_rows_per_block(shape.splits) : 0;
  const int recv_bytes = shape.splits * groups * shape.nb * per * 4;
  const int budget = 200 * 1024 - 512 - recv_bytes;
  shape.stages = budget / stage_bytes;
  if (shape.stages > 12) shape.stages = 12;
  if (shape.stages < 2) return XRT_ERR_UNSUPPORTED;
  int cols = 32;
  while (cols < 2 * groups * shape.nb) cols *= 2;
  if (cols > 512) return XRT_ERR_UNSUPPORTED;
  shape.tmem_cols = cols;
  shape.clustered = 0;
  *smem_out = shape.stages * stage_bytes + 1024 + recv_bytes + 1024;
  const int items = shape.tiles * shape.splits;
  *blocks_out = items < sm_count ? items : sm_count;
  *shape_out = shape;
  return XRT_OK;
}

static int decode_gemm(void* out, const void* x, const void* w, float* partial, int* counters, int M, int N, int K, int ldx,
                       int ldo, int w_rows, int out_dtype, int mode, int up_rows, int sm_count, int* error_flag,
                       const RowScale& scale, const NormEmit& emit, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || mode < 0 || mode > 2 || sm_count <= 0) return XRT_ERR_ARGUMENT;
  if (mode == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (mode == 2 ? w_rows < up_rows + N : w_rows < N) return XRT_ERR_ARGUMENT;
  if (out_dtype != XRT_F32 && out_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (K % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || M > 128) return XRT_ERR_UNSUPPORTED;
  if (M == 0) return XRT_OK;
  DecodeGemmShape shape;
  int smem = 0, blocks = 0;
  const int planned = plan_decode_gemm(M, N, K, ldo, mode, up_rows, sm_count, &shape, &smem, &blocks);
  if (planned != XRT_OK) return planned;
  if (shape.splits > 1 && (partial == nullptr || counters == nullptr)) return XRT_ERR_ARGUMENT;
  CUtensorMap map_w, map_x;
  if (!dg_make_map(&map_w, w, w_rows, K, K, DG_ROWS) || !dg_make_map(&map_x, x, M, K, ldx, shape.nb))
    return XRT_ERR_UNSUPPORTED;
  if (mode == 1)
    return launch_decode_gemm<1, float>(out, partial, counters, map_w, map_x, shape, smem, blocks, sm_count, error_flag, scale, emit, stream);
  if (mode == 2) {
    if (out_dtype == XRT_BF16)
      return launch_decode_gemm<2, __nv_bfloat16>(out, partial, counters, map_w, map_x, shape, smem, blocks, sm_count, error_flag, scale, emit, stream);
    return launch_decode_gemm<2, float>(out, partial, counters, map_w, map_x, shape, smem, blocks, sm_count, error_flag, scale, emit, stream);
  }
  if (out_dtype == XRT_BF16)
    return launch_decode_gemm<0, __nv_bfloat16>(out, partial, counters, map_w, map_x, shape, smem, blocks, sm_count, error_flag, scale, emit, stream);
  return launch_decode_gemm<0, float>(out, partial, counters, map_w, map_x, shape, smem, blocks, sm_count, error_flag, scale, emit, stream);
}

}  // namespace xrt

// x: bfloat16 [M, K] with row stride ldx, M <= 128; w: bfloat16 [w_rows, K] contiguous; K and ldx
// multiples of 8, bases 16-byte aligned.  out: [M, N] with row stride ldo.  Modes as for
// xrt_gemm_stream.  partial: float32 scratch of xrt_gemm_decode_tcgen05_scratch floats (may be null
// when that is 0); counters: int32 [at least ceil(N / 128)], zero before the first call (the
// kernel leaves them zero).  error_flag (may be null) is set to 4 if a bounded wait ran out.
// squares not null: the input's RMSNorm was prepared by the product before it (xrt_gemm_stream_norm):
// x is the residual times the norm weight, squares = float32 [square_parts, M] its partial sums of
// squares, and every batch row's result is multiplied by 1 / sqrt(sum of its parts / K + eps).
XRT_EXPORT int xrt_gemm_decode_tcgen05_normed(void* out, const void* x, const void* w, float* partial, int* counters,
                                              int M, int N, int K, int ldx, int ldo, int w_rows, int out_dtype, int mode,
                                              int up_rows, int sm_count, int* error_flag, const float* squares,
                                              int square_parts, float eps, cudaStream_t stream) {
  if (squares != nullptr && (square_parts <= 0 || mode == 1)) return XRT_ERR_ARGUMENT;
  xrt::RowScale scale;
  scale.squares = squares; scale.parts = square_parts; scale.width = K; scale.eps = eps;
  return xrt::decode_gemm(out, x, w, partial, counters, M, N, K, ldx, ldo, w_rows, out_dtype, mode, up_rows, sm_count,
                          error_flag, scale, xrt::NormEmit(), stream);
}

// How many partial sums of squares a row xrt_gemm_decode_tcgen05_norm leaves (one a block: tiles x
// splits), or 0 when this product cannot prepare a norm on the current device: only the finish of
// splits that run as clusters does.
XRT_EXPORT int xrt_gemm_decode_tcgen05_norm_parts(int M, int N, int K, int sm_count) {
  if (M <= 0 || M > 128 || N <= 0 || K <= 0 || sm_count <= 0 || N % 4 != 0) return 0;
  xrt::DecodeGemmShape shape;
  int smem = 0, blocks = 0;
  if (xrt::plan_decode_gemm(M, N, K, N, 1, 0, sm_count, &shape, &smem, &blocks) != XRT_OK) return 0;
  return xrt::decode_gemm_as_clusters<1, float>(shape, smem, sm_count) ? shape.tiles * shape.splits : 0;
}

// out (float32 [M, N]) += x . w^T, and the RMSNorm that follows prepared on the way, as
// xrt_gemm_stream_norm does: scaled (bfloat16 [M, ld_scaled]) = new out * norm_weight ([N], float32 or
// bfloat16 by norm_dtype), squares (float32 [xrt_gemm_decode_tcgen05_norm_parts, M]) = the rows' partial
// sums of squares.  N, ldo and ld_scaled multiples of 4; out and norm_weight 16-byte aligned, scaled 8.
// XRT_ERR_UNSUPPORTED where xrt_gemm_decode_tcgen05_norm_parts is 0.
XRT_EXPORT int xrt_gemm_decode_tcgen05_norm(void* out, const void* x, const void* w, float* partial, int* counters, int M,
                                            int N, int K, int ldx, int ldo, int w_rows, int sm_count, int* error_flag,
                                            void* scaled, int ld_scaled, const void* norm_weight, int norm_dtype,
                                            float* squares, cudaStream_t stream) {
  if (scaled == nullptr || norm_weight == nullptr || squares == nullptr || ld_scaled < N) return XRT_ERR_ARGUMENT;
  if (norm_dtype != XRT_F32 && norm_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (N % 4 != 0 || ldo % 4 != 0 || ld_scaled % 4 != 0 || ((uintptr_t)out & 15) || ((uintptr_t)norm_weight & 15) ||
      ((uintptr_t)scaled & 7))
    return XRT_ERR_UNSUPPORTED;
  xrt::NormEmit emit;
  emit.scaled = (__nv_bfloat16*)scaled; emit.weight = norm_weight; emit.squares = squares;
  emit.ld = ld_scaled; emit.weight_dtype = norm_dtype;
  return xrt::decode_gemm(out, x, w, partial, counters, M, N, K, ldx, ldo, w_rows, XRT_F32, 1, 0, sm_count, error_flag,
                          xrt::RowScale(), emit, stream);
}

// The same without a pending norm.
XRT_EXPORT int xrt_gemm_decode_tcgen05(void* out, const void* x, const void* w, float* partial, int* counters, int M,
                                       int N, int K, int ldx, int ldo, int w_rows, int out_dtype, int mode,
                                       int up_rows, int sm_count, int* error_flag, cudaStream_t stream) {
  return xrt_gemm_decode_tcgen05_normed(out, x, w, partial, counters, M, N, K, ldx, ldo, w_rows, out_dtype, mode, up_rows,
                                        sm_count, error_flag, nullptr, 0, 0.f, stream);
}
