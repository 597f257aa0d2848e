// A chain of norms and few-row matrix products run by ONE persistent kernel: the phases between two
// attention calls of a decode step (output product, norm, gate/up with SwiGLU, down, next norm,
// next q/k/v product) and the final norm with the output matrix.
//
// The reference runs a decode step as one pass per weight matrix, each a row-parallel dot product
// (crates/xrt-models/src/llama.rs:433-602; crates/xrt-kernels/src/cpu/matmul.rs:100-192).  On this GPU
// such a product reads 30 to 230 MB in 5 to 40 microseconds, and a kernel boundary (drain, launch,
// first-load latency) costs about as much as the smallest of them.  Here the weights of all the
// phases form one stream that never stops:
//
//  * one block per multiprocessor, launched cooperatively (all blocks are resident);
//  * a producer warp walks the phases ahead of everyone else and copies weight slabs (8 rows x 1,024
//    k, one 2 KB bulk asynchronous copy a row, completion on an mbarrier) into a ring of shared-memory
//    stages.  Weights do not depend on the step, so the producer never waits for a phase to finish:
//    while the blocks meet at the barrier between two phases, the next phase's weights are landing;
//  * eight compute warps take the slabs with tensor-core MMAs (mma.sync m16n8k16, batch rows as M,
//    weight rows as N, 32-bit accumulation).  The phase's activations [rows, K chunk] are staged in
//    shared memory once per phase.  Warp w takes an eighth of every slab's k range; at the end of a
//    unit the warps leave their partial sums in shared memory and go on with the next unit;
//  * an epilogue warp adds the eight partial sums in warp order and stores, adds into the residual
//    or applies SwiGLU, while the compute warps are already in the next unit (two areas, handed
//    back and forth with mbarriers);
//  * a work unit is 8 weight rows (SwiGLU: 8 gate rows and the 8 matching up rows) over all of K;
//    units go round the blocks, and where a product starts rotates so that the blocks with one
//    unit more are not always the same.  When the activations of a whole row do not fit in shared
//    memory (K above 4,096), K is walked in chunks with up to four units' accumulators alive at
//    once: chunk by chunk the activations are staged and every unit of the batch takes its slabs of
//    that chunk.  Every output is still one sum in one fixed order, by one block;
//  * between phases the blocks meet at a counter in global memory (one release-add to arrive, acquire
//    loads to wait; the last block to leave the kernel sets it back to zero).  Data written inside the
//    kernel is read back with loads that bypass L1.
//
// Every wait (mbarrier, grid barrier) is bounded: a wait that runs out raises the error flag and the
// block's abort flag; from then on every wait of the block returns at once, so that all its warps
// still reach every block-level barrier and the block runs to its end (with meaningless results);
// the producer waits (bounded) for its copies in flight before it returns.  Other blocks see the
// error flag in their own waits.
#include "common.cuh"

namespace xrt {

constexpr int DC_WARPS = 8;                       // compute warps
constexpr int DC_COMPUTE = DC_WARPS * 32;
constexpr int DC_WORKERS = DC_COMPUTE + 32;       // + the epilogue warp
constexpr int DC_THREADS = DC_WORKERS + 32;       // + the producer warp
constexpr int DC_STAGES = 8;                      // at most; fewer when the activations need the room
constexpr int DC_ROWS = 8;                        // weight rows of a stage and of a unit
constexpr int DC_SLAB = 1024;                     // k elements of a stage
constexpr int DC_W_STRIDE = DC_SLAB * 2 + 64;     // padded rows: a quarter warp reads 32 different banks
constexpr int DC_STAGE_BYTES = DC_ROWS * DC_W_STRIDE;
constexpr int DC_X_ROW_PAD = 64;
constexpr int DC_CHUNK = 4096;                    // k elements of the activations staged at a time
constexpr int DC_PARTIAL_FLOATS = DC_WARPS * 2 * 16 * 9;    // [warp][group][16 batch rows][8 + 1]
constexpr int DC_MAX_PHASES = 12;
constexpr int DC_MAX_ROWS = 16;
constexpr unsigned DC_SPIN_LIMIT = 1u << 24;
constexpr int DC_SMEM_FIXED = 2 * DC_PARTIAL_FLOATS * 4 + 256;  // partial sums and barriers
constexpr int DC_SMEM_MAX = 226 * 1024;  // dynamic; the limit of 227 KB a block counts the static words too

enum { DC_NORM = 0, DC_PRODUCT = 1 };

struct ChainPhase {
  const void* x;        // product: bfloat16 [m, ldx]; norm: float32 [.., ldx]
  const void* w;        // product: bfloat16 [n (and the up rows), k]; norm: the weight [k]
  void* out;            // [m, ldo]
  const int* rows;      // norm: output row r is the norm of input row rows[r] (null: row r)
  long long up_offset;  // SwiGLU: elements from a gate row to its up row
  int kind, mode;       // mode of a product: 0 store, 1 add into a float32 out, 2 SwiGLU
  int m, n, k, ldx, ldo;
  int out_dtype, w_dtype;
  int unit_rows;        // filled by the launcher: weight rows a unit (8)
  int first_unit;       //   rotation of the units over the blocks
  int splits, chunk;    //   chunks of K (the activations are staged chunk by chunk) and their width
  float eps;
  int reserved;
};

struct ChainPlan {
  ChainPhase phase[DC_MAX_PHASES];
  int n_phases;
  int stages;   // depth of the ring
  int x_bytes;  // room for the staged activations
};

__device__ __forceinline__ uint32_t dc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dc_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void dc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool dc_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (unsigned spin = 0; spin < DC_SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    // after a failure every wait returns at once: the block runs to its end without stopping
    if ((spin == 0 || (spin & 1023) == 1023) && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void dc_bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void dc_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DC_COMPUTE) : "memory"); }
__device__ __forceinline__ void dc_worker_sync() { asm volatile("bar.sync 2, %0;" ::"n"(DC_WORKERS) : "memory"); }
__device__ __forceinline__ void dc_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 dc_lds(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// How one block walks one product phase; the producer, the compute warps and the epilogue warp
// compute the same walk: units unit0, unit0 + blocks, ..., in batches of `batch` units whose
// accumulators are alive together; for each batch the chunks of K in order; for each chunk the
// batch's units; for each unit the slabs of that chunk (SwiGLU: gate stage, then up stage).
struct ChainWalk {
  int groups, batch, n_units, unit0, my_units;
  __device__ ChainWalk(const ChainPhase& ph) {
    groups = ph.mode == 2 ? 2 : 1;
    batch = ph.mode == 2 ? 2 : 4;
    const int blocks = (int)gridDim.x;
    unit0 = ((int)blockIdx.x + blocks - ph.first_unit % blocks) % blocks;
    n_units = (ph.n + DC_ROWS - 1) / DC_ROWS;
    my_units = unit0 < n_units ? (n_units - unit0 + blocks - 1) / blocks : 0;
  }
};

struct ChainShared {
  unsigned char* ring;
  unsigned char* xs;
  float* partial;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* part_full;
  uint64_t* part_empty;
  volatile int* abort_flag;
  int* error_flag;
  int stages;
};

// Where a role stands in the ring of stages and in the hand-over of partial sums; the roles keep
// their own copies and advance them alike.
struct ChainCursor {
  int stage = 0;
  uint32_t parity = 0;
  unsigned units = 0;  // units finished so far, over all phases
  __device__ __forceinline__ void next_stage(int stages) {
    if (++stage == stages) { stage = 0; parity ^= 1u; }
  }
};

// A wait ran out: tell this block and, through the error flag, every other block.
__device__ __forceinline__ void dc_fail(const ChainShared& sh, int code) {
  *sh.abort_flag = 1;
  atomicCAS(sh.error_flag, 0, code);
}

// The meeting of all blocks after phase `index` (from 1): every block adds one to a counter that
// only grows while the kernel runs, and waits until it reaches index * blocks.  Called by all
// worker threads.
__device__ __forceinline__ void dc_grid_barrier(unsigned int* sync, const ChainShared& sh, unsigned int index) {
  dc_worker_sync();
  if (threadIdx.x == 0 && !*sh.abort_flag) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(sync) : "memory");
    const unsigned int target = index * gridDim.x;
    bool passed = false;
    for (unsigned spin = 0; spin < DC_SPIN_LIMIT; ++spin) {
      unsigned int seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sync) : "memory");
      if (seen >= target) { passed = true; break; }
      if ((spin & 255) == 255) {
        if (*reinterpret_cast<volatile int*>(sh.error_flag) != 0) break;
        __nanosleep(64);
      }
    }
    if (!passed) dc_fail(sh, 4);
  }
  dc_worker_sync();
}

// ---- norm phase: block b takes rows b, b + blocks, ... -------------------------------------------
__device__ void dc_norm(const ChainPhase& ph, const ChainShared& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* scratch = sh.partial;
  for (int r = blockIdx.x; r < ph.m; r += gridDim.x) {
    const int src = ph.rows != nullptr ? ph.rows[r] : r;
    const float* xr = reinterpret_cast<const float*>(ph.x) + (size_t)src * ph.ldx;
    // a thread's first four pieces stay in registers for the second pass (rows up to 4,096 wide are read once);
    // the loads of a batch are issued together
    float acc = 0.f;
    float4 first[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (tid + i * DC_COMPUTE) * 4;
      first[i] = c < ph.k ? __ldcg(reinterpret_cast<const float4*>(xr + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc = fmaf(first[i].x, first[i].x, acc); acc = fmaf(first[i].y, first[i].y, acc);
      acc = fmaf(first[i].z, first[i].z, acc); acc = fmaf(first[i].w, first[i].w, acc);
    }
#pragma unroll 4
    for (int c = (tid + 4 * DC_COMPUTE) * 4; c < ph.k; c += DC_COMPUTE * 4) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + c));
      acc = fmaf(v.x, v.x, acc); acc = fmaf(v.y, v.y, acc); acc = fmaf(v.z, v.z, acc); acc = fmaf(v.w, v.w, acc);
    }
    acc = warp_sum(acc);
    dc_compute_sync();
    if (lane == 0) scratch[warp] = acc;
    dc_compute_sync();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) total += scratch[w];
    const float inv = 1.0f / sqrtf(total / (float)ph.k + ph.eps);
    auto scale_store = [&](int c, const float4& v) {
      float wv[4];
      if (ph.w_dtype == XRT_BF16) {
        const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(ph.w) + c);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        wv[0] = __low2float(a); wv[1] = __high2float(a); wv[2] = __low2float(b); wv[3] = __high2float(b);
      } else {
        const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ph.w) + c);
        wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
      }
      const float y0 = (v.x * inv) * wv[0], y1 = (v.y * inv) * wv[1], y2 = (v.z * inv) * wv[2], y3 = (v.w * inv) * wv[3];
      if (ph.out_dtype == XRT_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&a);
        t.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ph.out) + (size_t)r * ph.ldo + c) = t;
      } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(ph.out) + (size_t)r * ph.ldo + c) = make_float4(y0, y1, y2, y3);
      }
    };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (tid + i * DC_COMPUTE) * 4;
      if (c < ph.k) scale_store(c, first[i]);
    }
#pragma unroll 4
    for (int c = (tid + 4 * DC_COMPUTE) * 4; c < ph.k; c += DC_COMPUTE * 4)
      scale_store(c, __ldcg(reinterpret_cast<const float4*>(xr + c)));
  }
}

// one output value of a product: stored, added or passed through SwiGLU
__device__ __forceinline__ void dc_emit(const ChainPhase& ph, int m, int row, float first, float second) {
  const size_t at = (size_t)m * ph.ldo + row;
  if (ph.mode == 2) first = (first / (1.0f + expf(-first))) * second;
  if (ph.mode == 1) {
    float* p = reinterpret_cast<float*>(ph.out) + at;
    *p = __ldcg(p) + first;
  } else if (ph.out_dtype == XRT_BF16) {
    reinterpret_cast<__nv_bfloat16*>(ph.out)[at] = __float2bfloat16_rn(first);
  } else {
    reinterpret_cast<float*>(ph.out)[at] = first;
  }
}

// A warp's share of one whole slab (128 k): all loads first, then MMAs on four independent
// accumulators a group.
template <int GROUPS, bool TWO_TILES>
__device__ __forceinline__ void dc_slab(float (&acc)[GROUPS][4][4], uint32_t x_at, uint32_t x_hi,
                                        const uint32_t (&w_at)[GROUPS]) {
#pragma unroll
  for (int h = 0; h < 4; h += 2) {
    uint4 xa[2], xb[2], wv[GROUPS][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      xa[j] = dc_lds(x_at + (h + j) * 64);
      xb[j] = TWO_TILES ? dc_lds(x_at + x_hi + (h + j) * 64) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int gr = 0; gr < GROUPS; ++gr)
#pragma unroll
      for (int j = 0; j < 2; ++j) wv[gr][j] = dc_lds(w_at[gr] + (h + j) * 64);
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int gr = 0; gr < GROUPS; ++gr) {
        dc_mma(acc[gr][2 * j], xa[j].x, xb[j].x, xa[j].y, xb[j].y, wv[gr][j].x, wv[gr][j].y);
        dc_mma(acc[gr][2 * j + 1], xa[j].z, xb[j].z, xa[j].w, xb[j].w, wv[gr][j].z, wv[gr][j].w);
      }
  }
}

// ---- product phase, compute warps ----------------------------------------------------------------
template <int GROUPS>
__device__ void dc_compute(const ChainPhase& ph, const ChainShared& sh, ChainCursor& cur) {
  constexpr int BATCH = GROUPS == 2 ? 2 : 4;
  const ChainWalk walk(ph);
  if (walk.my_units == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const bool two_tiles = ph.m > 8;  // batch rows 8 .. 15 exist
  const int x_rows = two_tiles ? 16 : 8;
  const int x_stride = ph.chunk * 2 + DC_X_ROW_PAD;
  const uint32_t xs_lo = dc_smem(sh.xs) + g * x_stride + t * 16 + warp * 256;  // the warp's 128 k of a slab
  const uint32_t w_lane = g * DC_W_STRIDE + t * 16 + warp * 256;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  bool staged = false;

  for (int b0 = 0; b0 < walk.my_units; b0 += BATCH) {
    float acc[BATCH][GROUPS][4][4];  // four chains of dependent MMAs a unit and group
#pragma unroll
    for (int j = 0; j < BATCH; ++j)
#pragma unroll
      for (int gr = 0; gr < GROUPS; ++gr)
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[j][gr][c][i] = 0.f;

    for (int chunk = 0; chunk < ph.splits; ++chunk) {
      const int chunk_begin = chunk * ph.chunk, chunk_end = min(ph.k, chunk_begin + ph.chunk);
      if (ph.splits > 1 || !staged) {
        // this chunk of the activations into shared memory: asynchronous 16-byte copies that bypass
        // L1, all of a thread's pieces in flight at once; a piece beyond the rows or the chunk is
        // filled with zeros (source size 0)
        if (staged) dc_compute_sync();  // every warp is done with the chunk before
        const int pieces = ph.chunk / 8;
        const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(ph.x);
        const uint32_t xs = dc_smem(sh.xs);
        for (int i = tid; i < x_rows * pieces; i += DC_COMPUTE) {
          const int r = i / pieces, p = i - r * pieces;
          const int k = chunk_begin + p * 8;
          const bool live = r < ph.m && k < chunk_end;
          const __nv_bfloat16* src = live ? x + (size_t)r * ph.ldx + k : x;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(xs + r * x_stride + p * 16), "l"(src),
                       "r"(live ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
        dc_compute_sync();
        staged = true;
      }
#pragma unroll
      for (int j = 0; j < BATCH; ++j) {
        if (b0 + j >= walk.my_units) continue;
        for (int k0 = chunk_begin; k0 < chunk_end; k0 += DC_SLAB) {
          uint32_t w_at[GROUPS];
          int held[GROUPS];
#pragma unroll
          for (int gr = 0; gr < GROUPS; ++gr) {
            if (!dc_mbar_wait(dc_smem(&sh.full[cur.stage]), cur.parity, sh.abort_flag) && !*sh.abort_flag) dc_fail(sh, 5);
            w_at[gr] = dc_smem(sh.ring) + cur.stage * DC_STAGE_BYTES + w_lane;
            held[gr] = cur.stage;
            cur.next_stage(sh.stages);
          }
          const uint32_t x_at = xs_lo + (uint32_t)(k0 - chunk_begin) * 2;
          if (k0 + DC_SLAB <= chunk_end) {
            if (two_tiles) dc_slab<GROUPS, true>(acc[j], x_at, 8 * x_stride, w_at);
            else dc_slab<GROUPS, false>(acc[j], x_at, 8 * x_stride, w_at);
          } else {
            // the last, partial slab of K: pieces beyond its end count as zeros
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const bool inside = k0 + warp * 128 + h * 32 + t * 8 < chunk_end;
              const uint4 xa = inside ? dc_lds(x_at + h * 64) : zero;
              const uint4 xb = (inside && two_tiles) ? dc_lds(x_at + 8 * x_stride + h * 64) : zero;
#pragma unroll
              for (int gr = 0; gr < GROUPS; ++gr) {
                const uint4 wv = inside ? dc_lds(w_at[gr] + h * 64) : zero;
                dc_mma(acc[j][gr][0], xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
                dc_mma(acc[j][gr][1], xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
              }
            }
          }
          __syncwarp();
          if (lane == 0) {
#pragma unroll
            for (int gr = 0; gr < GROUPS; ++gr) dc_mbar_arrive(dc_smem(&sh.empty[held[gr]]));
          }
        }
      }
    }

    // each unit's partial sums into the area of its turn, once the epilogue warp has given it back
#pragma unroll
    for (int j = 0; j < BATCH; ++j) {
      if (b0 + j >= walk.my_units) continue;
      const int turn = cur.units & 1;
      if (!dc_mbar_wait(dc_smem(&sh.part_empty[turn]), ((cur.units >> 1) & 1u) ^ 1u, sh.abort_flag) && !*sh.abort_flag)
        dc_fail(sh, 7);
      float* partial = sh.partial + turn * DC_PARTIAL_FLOATS;
#pragma unroll
      for (int gr = 0; gr < GROUPS; ++gr) {
        float* p = partial + ((size_t)warp * 2 + gr) * 16 * 9;
        const float (&a)[4][4] = acc[j][gr];
        p[g * 9 + 2 * t] = (a[0][0] + a[1][0]) + (a[2][0] + a[3][0]);
        p[g * 9 + 2 * t + 1] = (a[0][1] + a[1][1]) + (a[2][1] + a[3][1]);
        p[(g + 8) * 9 + 2 * t] = (a[0][2] + a[1][2]) + (a[2][2] + a[3][2]);
        p[(g + 8) * 9 + 2 * t + 1] = (a[0][3] + a[1][3]) + (a[2][3] + a[3][3]);
      }
      __syncwarp();
      if (lane == 0) dc_mbar_arrive(dc_smem(&sh.part_full[turn]));
      ++cur.units;
    }
  }
}

// ---- product phase, epilogue warp ----------------------------------------------------------------
template <int GROUPS>
__device__ void dc_epilogue(const ChainPhase& ph, const ChainShared& sh, ChainCursor& cur) {
  const ChainWalk walk(ph);
  const int lane = threadIdx.x & 31;
  const int values = ph.m * DC_ROWS;  // (batch row, weight row) pairs of a unit: at most 128, four a lane
  for (int u = 0; u < walk.my_units; ++u) {
    const int row0 = (walk.unit0 + u * (int)gridDim.x) * DC_ROWS;
    const int turn = cur.units & 1;
    float old[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // the residual values first: their loads overlap the wait and the sums
      const int v = lane + 32 * i, m = v / DC_ROWS, n = v % DC_ROWS;
      old[i] = 0.f;
      if (ph.mode == 1 && v < values && row0 + n < ph.n)
        old[i] = __ldcg(reinterpret_cast<const float*>(ph.out) + (size_t)m * ph.ldo + row0 + n);
    }
    if (!dc_mbar_wait(dc_smem(&sh.part_full[turn]), (cur.units >> 1) & 1u, sh.abort_flag) && !*sh.abort_flag)
      dc_fail(sh, 8);
    const float* partial = sh.partial + turn * DC_PARTIAL_FLOATS;
    float sums[4][GROUPS];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = lane + 32 * i, m = v / DC_ROWS, n = v % DC_ROWS;
#pragma unroll
      for (int gr = 0; gr < GROUPS; ++gr) {
        float sum = 0.f;
        if (v < values) {
#pragma unroll
          for (int w = 0; w < DC_WARPS; ++w) sum += partial[(((size_t)w * 2 + gr) * 16 + m) * 9 + n];
        }
        sums[i][gr] = sum;
      }
    }
    __syncwarp();
    if (lane == 0) dc_mbar_arrive(dc_smem(&sh.part_empty[turn]));  // the compute warps may fill the area again
    ++cur.units;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = lane + 32 * i, m = v / DC_ROWS, n = v % DC_ROWS;
      if (v >= values || row0 + n >= ph.n) continue;
      if (ph.mode == 1) reinterpret_cast<float*>(ph.out)[(size_t)m * ph.ldo + row0 + n] = old[i] + sums[i][0];
      else dc_emit(ph, m, row0 + n, sums[i][0], sums[i][GROUPS - 1]);
    }
  }
}

// ---- the producer: weight slabs of every product phase, in the compute warps' order --------------
__device__ void dc_produce(const ChainPlan& plan, const ChainShared& sh) {
  const int lane = threadIdx.x & 31;
  ChainCursor cur;
  int fills[DC_STAGES];
#pragma unroll
  for (int s = 0; s < DC_STAGES; ++s) fills[s] = 0;
  bool ok = true;
  for (int p = 0; p < plan.n_phases && ok; ++p) {
    const ChainPhase& ph = plan.phase[p];
    if (ph.kind != DC_PRODUCT) continue;
    const ChainWalk walk(ph);
    const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(ph.w);
    for (int b0 = 0; b0 < walk.my_units && ok; b0 += walk.batch) {
      for (int chunk = 0; chunk < ph.splits && ok; ++chunk) {
        const int chunk_begin = chunk * ph.chunk, chunk_end = min(ph.k, chunk_begin + ph.chunk);
        for (int j = 0; j < walk.batch && b0 + j < walk.my_units && ok; ++j) {
          const int unit = walk.unit0 + (b0 + j) * (int)gridDim.x;
          const int row = min(unit * DC_ROWS + (lane & 7), ph.n - 1);  // rows beyond n repeat the last row: never stored
          const __nv_bfloat16* src_row = w + (size_t)row * ph.k;
          for (int k0 = chunk_begin; k0 < chunk_end && ok; k0 += DC_SLAB) {
            const uint32_t bytes = (uint32_t)min(DC_SLAB, chunk_end - k0) * 2u;
            for (int gr = 0; gr < walk.groups; ++gr) {  // gate rows, then the matching up rows
              if (!dc_mbar_wait(dc_smem(&sh.empty[cur.stage]), cur.parity ^ 1u, sh.abort_flag)) { ok = false; break; }
              const uint32_t bar = dc_smem(&sh.full[cur.stage]);
              if (lane == 0) dc_mbar_expect_tx(bar, bytes * DC_ROWS);
              __syncwarp();
              if (lane < DC_ROWS)
                dc_bulk_copy(dc_smem(sh.ring) + cur.stage * DC_STAGE_BYTES + lane * DC_W_STRIDE,
                             src_row + (gr == 1 ? ph.up_offset : 0) + k0, bytes, bar);
#pragma unroll
              for (int s = 0; s < DC_STAGES; ++s) fills[s] += (s == cur.stage);
              cur.next_stage(sh.stages);
            }
          }
        }
      }
    }
  }
  if (!ok) {
    if (!*sh.abort_flag) dc_fail(sh, 6);
    // copies in flight write this block's shared memory: they must have landed before it is given back
#pragma unroll
    for (int s = 0; s < DC_STAGES; ++s)
      if (fills[s] > 0) {
        const uint32_t bar = dc_smem(&sh.full[s]);
        for (unsigned spin = 0; spin < DC_SPIN_LIMIT; ++spin) {
          uint32_t done;
          asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                       : "=r"(done) : "r"(bar), "r"((uint32_t)((fills[s] - 1) & 1)) : "memory");
          if (done) break;
        }
      }
  }
}

__global__ void __launch_bounds__(DC_THREADS, 1)
decode_chain_kernel(const __grid_constant__ ChainPlan plan, unsigned int* sync, int* error_flag) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int abort_word;
  ChainShared sh;
  sh.stages = plan.stages;
  sh.ring = smem;
  sh.xs = smem + plan.stages * DC_STAGE_BYTES;
  sh.partial = reinterpret_cast<float*>(sh.xs + plan.x_bytes);
  sh.full = reinterpret_cast<uint64_t*>(sh.partial + 2 * DC_PARTIAL_FLOATS);
  sh.empty = sh.full + DC_STAGES;
  sh.part_full = sh.empty + DC_STAGES;
  sh.part_empty = sh.part_full + 2;
  sh.abort_flag = &abort_word;
  sh.error_flag = error_flag;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < DC_STAGES; ++s) {
      dc_mbar_init(dc_smem(&sh.full[s]), 1);
      dc_mbar_init(dc_smem(&sh.empty[s]), DC_WARPS);
    }
    for (int i = 0; i < 2; ++i) {
      dc_mbar_init(dc_smem(&sh.part_full[i]), DC_WARPS);
      dc_mbar_init(dc_smem(&sh.part_empty[i]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (threadIdx.x >= DC_WORKERS) {
    dc_produce(plan, sh);
    return;
  }
  const bool computes = threadIdx.x < DC_COMPUTE;
  ChainCursor cur;
  for (int p = 0; p < plan.n_phases; ++p) {
    const ChainPhase& ph = plan.phase[p];
    if (ph.kind == DC_NORM) {
      if (computes) dc_norm(ph, sh);
    } else if (ph.mode == 2) {
      if (computes) dc_compute<2>(ph, sh, cur);
      else dc_epilogue<2>(ph, sh, cur);
    } else {
      if (computes) dc_compute<1>(ph, sh, cur);
      else dc_epilogue<1>(ph, sh, cur);
    }
    if (p + 1 < plan.n_phases) dc_grid_barrier(sync, sh, (unsigned int)(p + 1));
  }
  // the last block to leave sets the barrier's counter back to zero for the next launch
  dc_worker_sync();
  if (threadIdx.x == 0 && !*sh.abort_flag) {
    __threadfence();
    if (atomicAdd(sync + 1, 1u) == gridDim.x - 1) {
      sync[0] = 0u;
      sync[1] = 0u;
    }
  }
}

}  // namespace xrt

XRT_EXPORT long long xrt_decode_chain_limits(int* max_phases, int* max_rows) {
  if (max_phases) *max_phases = xrt::DC_MAX_PHASES;
  if (max_rows) *max_rows = xrt::DC_MAX_ROWS;
  return 0;
}

// phases: n_phases entries in host memory (the launcher fills unit_rows, first_unit, splits, chunk).
// sync: two zeroed uint32 of device memory kept for this kernel.  Returns XRT_ERR_UNSUPPORTED for
// sizes outside what the kernel takes (the caller then runs the phases as separate kernels).
XRT_EXPORT int xrt_decode_chain(const void* phases_host, int n_phases, unsigned int* sync, int sm_count,
                                int* error_flag, cudaStream_t stream) {
  using namespace xrt;
  if (n_phases <= 0 || n_phases > DC_MAX_PHASES || sm_count <= 0) return XRT_ERR_ARGUMENT;
  ChainPlan plan;
  const ChainPhase* in = reinterpret_cast<const ChainPhase*>(phases_host);
  long long rot = 0;  // where the next product's first unit goes: remainders land on different blocks
  int x_bytes = 0;
  for (int i = 0; i < n_phases; ++i) {
    ChainPhase ph = in[i];
    if (ph.m <= 0 || ph.m > DC_MAX_ROWS || ph.k <= 0 || ph.ldo <= 0 || ph.ldx < ph.k) return XRT_ERR_ARGUMENT;
    if (ph.kind == DC_NORM) {
      if (ph.k % 4 != 0 || ph.ldx % 4 != 0 || ph.ldo % 4 != 0) return XRT_ERR_UNSUPPORTED;
      if (((uintptr_t)ph.x | (uintptr_t)ph.w | (uintptr_t)ph.out) & 15) return XRT_ERR_UNSUPPORTED;
    } else if (ph.kind == DC_PRODUCT) {
      if (ph.n <= 0 || ph.mode < 0 || ph.mode > 2 || ph.ldo < ph.n) return XRT_ERR_ARGUMENT;
      if (ph.mode == 1 && ph.out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
      if (ph.k % 8 != 0 || ph.ldx % 8 != 0 || (ph.up_offset % 8) != 0) return XRT_ERR_UNSUPPORTED;
      if (((uintptr_t)ph.x | (uintptr_t)ph.w) & 15) return XRT_ERR_UNSUPPORTED;
      ph.splits = (ph.k + DC_CHUNK - 1) / DC_CHUNK;
      ph.chunk = ph.splits > 1 ? DC_CHUNK : (ph.k + 255) / 256 * 256;
      ph.unit_rows = DC_ROWS;
      ph.first_unit = (int)(rot % sm_count);
      rot += (ph.n + DC_ROWS - 1) / DC_ROWS;
      const int need = (ph.m > 8 ? 16 : 8) * (ph.chunk * 2 + DC_X_ROW_PAD);
      if (need > x_bytes) x_bytes = need;
    } else {
      return XRT_ERR_ARGUMENT;
    }
    plan.phase[i] = ph;
  }
  plan.n_phases = n_phases;
  plan.x_bytes = (x_bytes + 127) / 128 * 128;
  plan.stages = (DC_SMEM_MAX - DC_SMEM_FIXED - plan.x_bytes) / DC_STAGE_BYTES;
  if (plan.stages > DC_STAGES) plan.stages = DC_STAGES;
  if (plan.stages < 3) return XRT_ERR_UNSUPPORTED;
  const int smem = plan.stages * DC_STAGE_BYTES + plan.x_bytes + DC_SMEM_FIXED;
  static bool prepared = false;
  if (!prepared) {
    cudaError_t err = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DC_SMEM_MAX);
    if (err != cudaSuccess) return (int)err;
    int resident = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, decode_chain_kernel, DC_THREADS, DC_SMEM_MAX);
    if (err != cudaSuccess) return (int)err;
    if (resident < 1) return XRT_ERR_UNSUPPORTED;
    prepared = true;
  }
  void* args[] = {(void*)&plan, (void*)&sync, (void*)&error_flag};
  cudaError_t err = cudaLaunchCooperativeKernel((const void*)decode_chain_kernel, dim3(sm_count), dim3(DC_THREADS), args,
                                                smem, stream);
  if (err != cudaSuccess) return (int)err;
  return launch_status();
}
