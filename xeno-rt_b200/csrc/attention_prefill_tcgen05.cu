// Causal grouped-query attention for prompts on the fifth-generation tensor cores (head size 128).
// (The reference's prefill form: crates/xrt-models/src/llama.rs:728-770: for token t the keys
// 0 .. start + t, read from the cache so that earlier context is included.)
//
// A block owns 128 consecutive new tokens of one sequence for one query head and walks the
// sequence's keys in steps of 128 (two cache blocks of 64).  Six warps:
//   warp 0    TMA: the Q tile once, then for each step its K and V tiles ([128 keys x 128], as boxes
//             of 64 keys x 64 dims, 128-byte swizzle) into a ring of three stages.  K and V of a stage
//             have barriers of their own: K is free again after the step's QK^T, a whole step before V.
//   warp 1    owns TMEM and issues the MMAs: S = Q K^T (128 x 128, eight tcgen05.mma over the head
//             size) into one of two S buffers, and O += P V (128 x 128, eight tcgen05.mma over the
//             step's keys) accumulated in TMEM over all steps.  K is a K-major operand as stored; V
//             ([key][dim]) is an MN-major operand as stored: no transposition anywhere.  QK^T of the
//             next step is issued before PV of this one, so the tensor core works while the softmax
//             runs.
//   warps 2-5 softmax and output, one thread a query row (TMEM lane).  A thread reads its row of S
//             (tcgen05.ld), masks (only steps that reach the diagonal), keeps the row's sum in 32-bit,
//             and writes P as bfloat16 pairs into one of two buffers in tensor memory (tcgen05.st),
//             from where P V reads it as its A operand.  The exponents are taken
//             against a reference value m of the row that only moves when the row's maximum has
//             grown by more than 8 (a factor 256) beyond it: softmax does not depend on m as long as
//             P and the sum use the same one, P stays within 2^8 (bfloat16 keeps its 8 bits of
//             precision at any magnitude), and the accumulated O in TMEM has to be rescaled (read,
//             multiplied, written back by the row's thread, after the products issued so far have
//             completed) only on those rare moves instead of once a step.
// Every mbarrier wait is bounded; a wait that runs out raises the error flag and an abort flag, all
// roles leave their loops, TMEM is freed and the block returns.
#include "tcgen05.cuh"

namespace xrt {

using namespace sm100;

constexpr int FA_ROWS = 128, FA_KEYS = 128, FA_HD = 128, FA_STAGES = 3;
constexpr int FA_Q_BYTES = FA_ROWS * FA_HD * 2;        // 32 KB (two halves of 16 KB)
constexpr int FA_BOX = 64 * 64 * 2;                    // 8 KB: what one tensor copy brings, 64 keys x 64 dims
constexpr int FA_KV_HALF = FA_KEYS * 64 * 2;           // 16 KB: 128 keys (two cache blocks) x 64 dims
constexpr int FA_STAGE_BYTES = 4 * FA_KV_HALF;         // K halves, then V halves: 64 KB
constexpr int FA_P_COLS = FA_KEYS / 2;                 // P in TMEM: bfloat16 pairs, 64 columns of 32 bits a step
constexpr int FA_P_BUFFERS = 2;                        // P of a step is written while the product before it still reads its own
constexpr int fa_smem_bytes(int nh) { return nh * FA_Q_BYTES + FA_STAGES * FA_STAGE_BYTES + 512 + 1024; }

// 2^x by the special-function unit; exp2(-inf) = 0.  Inputs are differences to a running maximum
// (at most 0) and the result feeds a bfloat16 product or a 32-bit sum: the unit's 2 ulp are far
// inside bfloat16's 8 bits.
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NH = query heads of one kv head that a block serves; its K and V tiles are fetched once for all of
// them.  With steps of 128 keys (two cache blocks: a tcgen05.mma costs about a hundred cycles
// whatever its N, so QK^T is issued with N = 128, and a step's chain of barrier hand-overs is paid
// half as often) the two S buffers and O of one head take 384 of the 512 TMEM columns: NH = 1.
template <int NH>
__global__ void __launch_bounds__(64 + 128 * NH, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                                 const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                                 const int* __restrict__ seq_start, const int* __restrict__ block_table, int max_blocks,
                                 int n_heads, int n_kv_heads, float scale_log2, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_tiles = smem;                                   // [NH] x 32 KB
  unsigned char* kv_ring = smem + NH * FA_Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_ring + FA_STAGES * FA_STAGE_BYTES);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [FA_STAGES] each: K and V of a step have barriers of their own,
  uint64_t* k_empty = k_full + FA_STAGES;  //   since a step's K is free again (after its QK^T) a whole step
  uint64_t* v_full = k_empty + FA_STAGES;  //   before its V (after its PV): the next K is fetched that much earlier
  uint64_t* v_empty = v_full + FA_STAGES;
  uint64_t* s_full = v_empty + FA_STAGES;  // [2]
  uint64_t* s_empty = s_full + 2;          // [2]
  uint64_t* p_full = s_empty + 2;          // [2]
  uint64_t* p_empty = p_full + 2;          // [2]
  uint64_t* pv_done = p_empty + 2;         // [1]: completes once for every step's P V
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // later query tiles walk more keys: they are scheduled first, the longest tiles of ALL heads before any shorter one
  // (the heads are the grid's fastest dimension).  With the query tiles fastest, the last heads' long tiles started
  // when most multiprocessors were already idle: a prompt of 2,048 tokens is 512 blocks of 1 to 16 steps on 148
  // multiprocessors, 42 steps on the busiest that way against 33 this way (71.5 -> 61.2 us a layer).
  // Of several prompts, every prompt's tiles at a query index come before any tile at a lower one (a tile beyond a
  // shorter prompt's end leaves at once): the prompts are the grid's second dimension, the query tiles its slowest.
  const int q_index = gridDim.z - 1 - blockIdx.z, head0 = blockIdx.x * NH, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  const int tok0 = cu_seqlens[seq];
  const int n_new = cu_seqlens[seq + 1] - tok0;
  const int row0 = q_index * FA_ROWS;
  if (slot < 0 || row0 >= n_new) return;  // the whole block leaves before any barrier or allocation
  const int start = seq_start[seq];
  const int kv_head = head0 / (n_heads / n_kv_heads);  // the same for all NH heads: NH divides the group
  const int last_row = min(row0 + FA_ROWS, n_new) - 1;
  const int n_tiles = (start + last_row + 1 + FA_KEYS - 1) / FA_KEYS;  // keys 0 .. position of the last row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  static_assert(NH * (2 * FA_KEYS + FA_HD + FA_P_BUFFERS * FA_P_COLS) <= 512, "S buffers, O and P buffers must fit in TMEM");
  constexpr int TMEM_COLS = 512;  // S: NH x 2 buffers x 128 columns; O: NH x 128; P: NH x 2 buffers x 64

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1); mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1); mbar_init(smem_u32(&v_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      // the softmax warps arrive once each (lane 0, after the warp has synchronised): hundreds of
      // arrivals on one shared-memory word would serialise
      mbar_init(smem_u32(&s_full[b]), 1);
      mbar_init(smem_u32(&s_empty[b]), 4 * NH);
    }
    for (int b = 0; b < FA_P_BUFFERS; ++b) {
      mbar_init(smem_u32(&p_full[b]), 4 * NH);
      mbar_init(smem_u32(&p_empty[b]), 1);
    }
    mbar_init(smem_u32(pv_done), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;                        // [head][buffer] x 64 columns
  const uint32_t tmem_o = tmem_base + NH * 2 * FA_KEYS;     // [head] x 128 columns
  const uint32_t tmem_p = tmem_o + NH * FA_HD;              // [head][buffer] x 64 columns

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      mbar_arrive_expect_tx(smem_u32(q_full), NH * FA_Q_BYTES);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_2d(smem_u32(q_tiles + h * FA_Q_BYTES), &map_q, (head0 + h) * FA_HD, tok0 + row0, smem_u32(q_full));
        tma_load_2d(smem_u32(q_tiles + h * FA_Q_BYTES + FA_Q_BYTES / 2), &map_q, (head0 + h) * FA_HD + 64, tok0 + row0,
                       smem_u32(q_full));
      }
      const int* blocks = block_table + (size_t)slot * max_blocks;
      const int n_blocks = (start + last_row + 1 + XRT_BLOCK_TOKENS - 1) / XRT_BLOCK_TOKENS;  // cache blocks the rows see
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % FA_STAGES;
        unsigned char* stage = kv_ring + s * FA_STAGE_BYTES;
        int pool_row[2];  // the step's two cache blocks; beyond the last one the last again (masked)
#pragma unroll
        for (int part = 0; part < 2; ++part)
          pool_row[part] = (blocks[min(2 * j + part, n_blocks - 1)] * n_kv_heads + kv_head) * XRT_BLOCK_TOKENS;
        ok = mbar_wait(smem_u32(&k_empty[s]), ((j / FA_STAGES) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&k_full[s]), 2 * FA_KV_HALF);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          tma_load_2d(smem_u32(stage + part * FA_BOX), &map_k, 0, pool_row[part], smem_u32(&k_full[s]));
          tma_load_2d(smem_u32(stage + FA_KV_HALF + part * FA_BOX), &map_k, 64, pool_row[part], smem_u32(&k_full[s]));
        }
        ok = mbar_wait(smem_u32(&v_empty[s]), ((j / FA_STAGES) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&v_full[s]), 2 * FA_KV_HALF);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          tma_load_2d(smem_u32(stage + 2 * FA_KV_HALF + part * FA_BOX), &map_v, 0, pool_row[part], smem_u32(&v_full[s]));
          tma_load_2d(smem_u32(stage + 3 * FA_KV_HALF + part * FA_BOX), &map_v, 64, pool_row[part], smem_u32(&v_full[s]));
        }
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 5); }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc(FA_ROWS, FA_KEYS, false);
      constexpr uint32_t idesc_pv = instr_desc(FA_ROWS, FA_HD, true);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag);
      auto issue_qk = [&](int j) {
        const int s = j % FA_STAGES, b = j & 1;
        if (!mbar_wait(smem_u32(&k_full[s]), (j / FA_STAGES) & 1, abort_flag)) return false;
        if (!mbar_wait(smem_u32(&s_empty[b]), ((j >> 1) & 1) ^ 1, abort_flag)) return false;
        fence_after();
        unsigned char* stage = kv_ring + s * FA_STAGE_BYTES;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
#pragma unroll
          for (int ks = 0; ks < FA_HD / 16; ++ks) {  // 16 dims a step; 4 steps a 64-dim half
            const uint64_t a = desc_k_major(smem_u32(q_tiles + h * FA_Q_BYTES + (ks / 4) * (FA_Q_BYTES / 2))) + 2 * (ks % 4);
            const uint64_t bd = desc_k_major(smem_u32(stage + (ks / 4) * FA_KV_HALF)) + 2 * (ks % 4);
            mma_f16(tmem_s + (h * 2 + b) * FA_KEYS, a, bd, idesc_qk, ks > 0);
          }
        }
        commit(smem_u32(&s_full[b]));
        commit(smem_u32(&k_empty[s]));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const int s = j % FA_STAGES;
        const int pb = j & 1;
        ok = mbar_wait(smem_u32(&p_full[pb]), (uint32_t)(j >> 1) & 1u, abort_flag) &&  // P is written, and O rescaled if it had to be
             mbar_wait(smem_u32(&v_full[s]), (j / FA_STAGES) & 1, abort_flag);
        if (!ok) break;
        fence_after();
        unsigned char* stage = kv_ring + s * FA_STAGE_BYTES;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
#pragma unroll
          for (int ks = 0; ks < FA_KEYS / 16; ++ks) {  // 16 keys a step
            const uint64_t bd = desc_mn_major(smem_u32(stage + 2 * FA_KV_HALF + ks * 2048), FA_KV_HALF);
            mma_f16_a_tmem(tmem_o + h * FA_HD, tmem_p + (h * FA_P_BUFFERS + pb) * FA_P_COLS + ks * 8, bd, idesc_pv, j > 0 || ks > 0);
          }
        }
        commit(smem_u32(pv_done));
        commit(smem_u32(&v_empty[s]));
        commit(smem_u32(&p_empty[pb]));
      }
      if (!ok) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 5); }
    }
  } else {
    // ---------------------------------------------------------------- softmax and output: one thread a row and head
    const int quarter = warp & 3;
    const int h = (warp - 2) >> 2;               // which of the block's heads
    const int head = head0 + h;
    const int r = quarter * 32 + lane;           // row of the tile = TMEM lane
    const int row = row0 + r;                    // new-token index in the sequence
    const bool row_live = row < n_new;
    const int key_hi = row_live ? start + row + 1 : 0;  // keys [0, key_hi) are visible
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t my_s = tmem_s + lane_base + h * 2 * FA_KEYS, my_o = tmem_o + lane_base + h * FA_HD;
    float m_ref = -INFINITY, l_run = 0.f;  // the reference value of the exponents (scaled, base 2) and the sum
    bool ok = true;

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      ok = mbar_wait(smem_u32(&s_full[b]), (j >> 1) & 1, abort_flag);
      if (!ok) break;
      fence_after();
      float s[FA_KEYS];
      {
        uint32_t v0[32], v1[32], v2[32], v3[32];  // the whole row on its way before the one wait
        tmem_ld32(v0, my_s + b * FA_KEYS);
        tmem_ld32(v1, my_s + b * FA_KEYS + 32);
        tmem_ld32(v2, my_s + b * FA_KEYS + 64);
        tmem_ld32(v3, my_s + b * FA_KEYS + 96);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(v0[i]); s[32 + i] = __uint_as_float(v1[i]);
          s[64 + i] = __uint_as_float(v2[i]); s[96 + i] = __uint_as_float(v3[i]);
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[b]));  // the tensor core may write the block after next into this buffer
      const int key0 = j * FA_KEYS;
      // Only blocks that reach past the first row's last visible key can hide a key from a row
      // (uniform over the thread block); every other block skips the comparisons.
      if (key0 + FA_KEYS > start + row0 + 1) {
#pragma unroll
        for (int i = 0; i < FA_KEYS; ++i) s[i] = (key0 + i < key_hi) ? s[i] : -INFINITY;
      }
      // the maximum of the raw scores (the scale is positive and is applied inside the exponent)
      float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < FA_KEYS; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) part_max[u] = fmaxf(part_max[u], s[i + u]);
      }
      const float m_tile = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])) * scale_log2;
      // move the reference only when the maximum has outgrown it by more than 8; the first visible key sets it
      const bool moves = m_tile > m_ref + 8.0f || (m_ref == -INFINITY && m_tile != -INFINITY);
      if (__any_sync(0xffffffffu, moves)) {
        const float factor = (moves && m_ref != -INFINITY) ? fa_exp2(m_ref - m_tile) : 1.0f;
        if (j > 0) {  // O holds the products of the blocks so far: they must have completed before it is rewritten
          ok = mbar_wait(smem_u32(pv_done), (uint32_t)(j - 1) & 1u, abort_flag);
          if (!ok) break;
          fence_after();
          if (__any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll
            for (int c = 0; c < FA_HD; c += 32) {
              uint32_t v[32];
              tmem_ld32(v, my_o + c);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
              tmem_st32(my_o + c, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            fence_before();
          }
        }
        l_run *= factor;
        if (moves) m_ref = m_tile;
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;  // a row without visible keys: exp2(-inf) = 0 all the same
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};
      // P goes into tensor memory as the A operand of P V: the row's lane, bfloat16 pairs of
      // consecutive keys a column.  Two P buffers a head: with one, the exponents of a step could
      // only be stored when the product of the step before had completed, and that product only
      // when they all were: the tensor core and the softmax threads took turns.
      ok = mbar_wait(smem_u32(&p_empty[b]), ((uint32_t)(j >> 1) & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      fence_after();
      const uint32_t my_p = tmem_p + lane_base + (h * FA_P_BUFFERS + b) * FA_P_COLS;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float p0 = fa_exp2(fmaf(s[half * 64 + 2 * i], scale_log2, neg_m));
          const float p1 = fa_exp2(fmaf(s[half * 64 + 2 * i + 1], scale_log2, neg_m));
          part_sum[i & 3] += p0 + p1;
          __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          packed[i] = *reinterpret_cast<uint32_t*>(&pair);
        }
        tmem_st32(my_p + half * 32, packed);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[b]));
      l_run += (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(smem_u32(pv_done), (uint32_t)(n_tiles - 1) & 1u, abort_flag);
    if (ok && n_tiles > 0) {
      fence_after();
      const float inv = row_live ? 1.0f / l_run : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(tok0 + row) * n_heads + head) * FA_HD;
#pragma unroll
      for (int c = 0; c < FA_HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(v, my_o + c);  // all lanes take part; rows beyond the sequence store nothing
        tmem_wait_ld();
        if (row_live) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * i]) * inv,
                                                          __uint_as_float(v[d + 2 * i + 1]) * inv);
              packed[i] = *reinterpret_cast<uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
      }
      fence_before();
    }
    if (!ok && lane == 0) { *abort_flag = 1; if (error_flag != nullptr) atomicExch(error_flag, 5); }
  }

  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS));
  }
}

// A map over a row-major bfloat16 matrix [rows, cols], boxes of box_rows x 64 columns, 128-byte swizzle.
static bool fa_make_map(CUtensorMap* map, const void* base, long long rows, int cols, int box_rows) {
  return sm100::make_map_bf16_2d(map, base, rows, cols, cols, box_rows);
}

}  // namespace xrt

// q, out: bfloat16 [n_tokens, n_heads * 128], the sequences' new tokens end to end (cu_seqlens[n_seqs + 1]);
// pools: bfloat16 [n_blocks, n_kv_heads, 64, 128]; seq_slot[n_seqs] (< 0: skipped), seq_start[n_seqs] = tokens each
// sequence held before this step; max_new = the most new tokens any sequence brings.  Head size 128 only, no window.
// error_flag (may be null) is set to 5 if a bounded wait ran out.
XRT_EXPORT int xrt_attention_prefill_tcgen05(void* out, const void* q, const void* k_pool, const void* v_pool,
                                             const int* cu_seqlens, const int* seq_slot, const int* seq_start,
                                             const int* block_table, int max_blocks, int n_blocks, int n_tokens,
                                             int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim,
                                             float scale, int* error_flag, cudaStream_t stream) {
  if (n_seqs < 0 || max_new < 0 || n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 ||
      n_blocks <= 0)
    return XRT_ERR_ARGUMENT;
  if (head_dim != xrt::FA_HD || n_seqs > 65535 || (max_new + xrt::FA_ROWS - 1) / xrt::FA_ROWS > 65535) return XRT_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)out & 15))
    return XRT_ERR_UNSUPPORTED;
  if (n_seqs == 0 || max_new == 0 || n_tokens == 0) return XRT_OK;
  CUtensorMap map_q, map_k, map_v;
  const long long pool_rows = (long long)n_blocks * n_kv_heads * XRT_BLOCK_TOKENS;
  if (!xrt::fa_make_map(&map_q, q, n_tokens, n_heads * xrt::FA_HD, xrt::FA_ROWS) ||
      !xrt::fa_make_map(&map_k, k_pool, pool_rows, xrt::FA_HD, XRT_BLOCK_TOKENS) ||
      !xrt::fa_make_map(&map_v, v_pool, pool_rows, xrt::FA_HD, XRT_BLOCK_TOKENS))
    return XRT_ERR_UNSUPPORTED;
  static bool allowed = false;
  if (!allowed) {
    cudaError_t err = cudaFuncSetAttribute(xrt::attention_prefill_tcgen05_kernel<1>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, xrt::fa_smem_bytes(1));
    if (err != cudaSuccess) return (int)err;
    allowed = true;
  }
  dim3 grid(n_heads, n_seqs, (max_new + xrt::FA_ROWS - 1) / xrt::FA_ROWS);
  // launched without programmatic dependent launch: a block needs a multiprocessor to itself, so nothing of it can
  // run beside the kernel before it, and the early launch was measured slower (28.2 against 27.8 ms a prompt of 2,048)
  xrt::attention_prefill_tcgen05_kernel<1><<<grid, 64 + 128, xrt::fa_smem_bytes(1), stream>>>(
      map_q, map_k, map_v, (__nv_bfloat16*)out, cu_seqlens, seq_slot, seq_start, block_table, max_blocks, n_heads,
      n_kv_heads, scale * 1.4426950408889634f, error_flag);
  return xrt::launch_status();
}
