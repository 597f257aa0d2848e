// Decode attention in bfloat16: one new token a sequence against the keys and values of its cache
// blocks, split along the sequence so that a handful of sequences still fill the GPU, then a
// combine step.  (The reference's decode form: crates/xrt-models/src/llama.rs:504-574, an online
// softmax over the cached positions, parallel over kv heads with the group's query heads inside.)
//
// Grid (splits, kv heads, tokens).  A block of four warps serves one kv head of one token for the
// keys [split * chunk, (split + 1) * chunk), counted from the cache block of the token's first visible key
// (position 0 without a window): the group's query heads (up to 16) are the rows of the
// MMA, so the group shares every key and value that is read.  Tiles of 64 keys (one cache block,
// contiguous in memory) are copied to shared memory with cp.async, double-buffered; warp w takes
// keys 16w .. 16w+16 of each tile with its own online-softmax state; the four states are merged
// through shared memory in warp order.  With one split the block writes the output, otherwise
// (m, l, o) partials that the combine kernel merges in split order.  Nothing depends on how many
// other tokens the launch carries, and launch shapes depend on `chunk` and the grid only, so the
// launch can be captured in a CUDA graph and replayed for other lengths.
#include "tcgen05.cuh"

#include "attention_mma.cuh"

namespace xrt {

constexpr int DEC_WARPS = 4;

// Keys of split s of a token that sees the keys [first_key, len): splits are counted from the cache block
// that holds the first visible key (position 0 without a window), `chunk` keys each, so that a windowed
// layer's splits all hold keys however long the sequence is.  The kernels and both combine steps share this.
__device__ __forceinline__ int split_begin(int split, int chunk, int first_key) {
  return (first_key / XRT_BLOCK_TOKENS) * XRT_BLOCK_TOKENS + split * chunk;
}
__device__ __forceinline__ int split_end(int split, int chunk, int first_key, int len) {
  return min(split_begin(split, chunk, first_key) + chunk, len);
}
__device__ __forceinline__ bool split_live(int split, int chunk, int first_key, int len) {
  return split_begin(split, chunk, first_key) < len;
}

// What every form of the kernel does once its four warps have left their running state in the merge
// area [warps][16 rows] of shared memory: merge them in warp order, write the output (one split) or
// this split's partials, and, with counters, let the block that brings the last split merge all.
__device__ __forceinline__ void decode_finish(unsigned char* smem, __nv_bfloat16* __restrict__ out,
                                              float* __restrict__ part_o, float* __restrict__ part_ml,
                                              int* __restrict__ counters, int tok, int kv_head, int split,
                                              int n_splits, int chunk, int first_key, int len, int group, int n_heads,
                                              int n_kv_heads, int head_dim) {
  float* merge_m = reinterpret_cast<float*>(smem);                 // [warps][16]
  float* merge_l = merge_m + DEC_WARPS * 16;                       // [warps][16]
  float* merge_o = merge_l + DEC_WARPS * 16;                       // [warps][16][head_dim + 8]: rows in different banks
  const int merge_stride = head_dim + 8;
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * head_dim; idx += blockDim.x) {
    const int row = idx / head_dim, d = idx - row * head_dim;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, merge_m[w * 16 + row]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = merge_m[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      l += f * merge_l[w * 16 + row];
      o += f * merge_o[((size_t)w * 16 + row) * merge_stride + d];
    }
    const int head = kv_head * group + row;
    if (n_splits == 1) {
      out[((size_t)tok * n_heads + head) * head_dim + d] = __float2bfloat16_rn(o / l);
    } else {
      const size_t p = ((size_t)tok * n_heads + head) * n_splits + split;
      part_o[p * head_dim + d] = o;
      if (d == 0) { part_ml[p * 2] = m; part_ml[p * 2 + 1] = l; }
    }
  }
  if (n_splits == 1 || counters == nullptr) return;

  // The block that brings the last live split of this (token, kv head) merges all of them, in
  // split order (no block waits for another; which block is last does not change the result).
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int n_live = 0;
    for (int s = 0; s < n_splits; ++s) n_live += split_live(s, chunk, first_key, len);
    int* counter = counters + tok * n_kv_heads + kv_head;
    const int before = atomicAdd(counter, 1);
    is_last = before == n_live - 1;
    if (is_last) *counter = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* all_m = reinterpret_cast<float*>(smem);      // [group][n_splits]: the split's maximum, then its weight
  float* all_l = all_m + group * n_splits;            // [group][n_splits]
  float* row_l = all_l + group * n_splits;            // [group]
  for (int i = threadIdx.x; i < group * n_splits; i += blockDim.x) {
    const int row = i / n_splits, s = i - row * n_splits;
    const bool live = split_live(s, chunk, first_key, len);
    const size_t p = ((size_t)tok * n_heads + kv_head * group + row) * n_splits + s;
    all_m[i] = live ? __ldcg(part_ml + p * 2) : -INFINITY;
    all_l[i] = live ? __ldcg(part_ml + p * 2 + 1) : 0.f;
  }
  __syncthreads();
  if (threadIdx.x < group) {
    const int row = threadIdx.x;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, all_m[row * n_splits + s]);
    float l = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = all_m[row * n_splits + s];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
      all_m[row * n_splits + s] = f;
      l += f * all_l[row * n_splits + s];
    }
    row_l[row] = l;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * head_dim; idx += blockDim.x) {
    const int row = idx / head_dim, d = idx - row * head_dim;
    const int head = kv_head * group + row;
    const float* po = part_o + ((size_t)tok * n_heads + head) * n_splits * head_dim + d;
    float o = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) {
      const float f = all_m[row * n_splits + s];  // 0 for a split without visible keys: its partials are never read
      const float v = f != 0.f ? __ldcg(po + (size_t)s * head_dim) : 0.f;
      o += f * v;
    }
    out[((size_t)tok * n_heads + head) * head_dim + d] = __float2bfloat16_rn(o / row_l[row]);
  }
}

// BY_HEADS: the group has at most 8 query heads; they are the MMA's columns and the keys its rows
// (half the MMAs and half the softmax work per key; see attend_16_keys_heads).  Otherwise the heads
// (up to 16) are the rows.  Both leave the same per-warp state in shared memory for the merge.
template <int HD_MAX, bool BY_HEADS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ tok_slot,
                        const int* __restrict__ tok_pos, const int* __restrict__ block_table, int max_blocks,
                        int n_heads, int n_kv_heads, int head_dim, float scale_log2, int window, int chunk,
                        int n_splits, int* __restrict__ counters) {
  constexpr int D_TILES = HD_MAX / 8;
  extern __shared__ __align__(16) unsigned char smem[];
  pdl_trigger();
  pdl_wait();
  const int split = blockIdx.x, kv_head = blockIdx.y, tok = blockIdx.z;
  const int slot = tok_slot[tok];
  if (slot < 0) {  // a padding row: zeros (with several splits and no counters the combine kernel writes them)
    if (n_splits == 1 || (counters != nullptr && split == 0)) {
      const int group = n_heads / n_kv_heads;
      __nv_bfloat16* dst = out + ((size_t)tok * n_heads + (size_t)kv_head * group) * head_dim;
      for (int i = threadIdx.x; i < group * head_dim; i += blockDim.x) dst[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int pos = tok_pos[tok];
  const int len = pos + 1;
  const int first_key = window > 0 ? max(0, len - window) : 0;
  const int begin = split_begin(split, chunk, first_key);
  const int end = split_end(split, chunk, first_key, len);
  if (begin >= end) return;  // this split holds no visible key: the combine step skips it too

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int group = n_heads / n_kv_heads;
  const int row_bytes = tile_row_bytes(head_dim);
  const int tile_bytes = XRT_BLOCK_TOKENS * row_bytes;
  unsigned char* k_tiles = smem;                   // [2][64 rows]
  unsigned char* v_tiles = smem + 2 * tile_bytes;  // [2][64 rows]

  const int* blocks = block_table + (size_t)slot * max_blocks;
  const size_t head_stride = (size_t)XRT_BLOCK_TOKENS * head_dim;
  TileCopier copier;
  copier.init(head_dim);
  auto issue_tile = [&](int tile_index, int buffer) {
    const int key0 = begin + tile_index * XRT_BLOCK_TOKENS;
    const int block = blocks[key0 / XRT_BLOCK_TOKENS];
    const size_t base = ((size_t)block * n_kv_heads + kv_head) * head_stride;
    const int live = min(XRT_BLOCK_TOKENS, len - key0);
    copier.copy(k_tiles + buffer * tile_bytes, k_pool + base, XRT_BLOCK_TOKENS, live);
    copier.copy(v_tiles + buffer * tile_bytes, v_pool + base, XRT_BLOCK_TOKENS, live);
    cp_async_commit();
  };

  const int n_tiles = (end - begin + XRT_BLOCK_TOKENS - 1) / XRT_BLOCK_TOKENS;  // begin is a multiple of 64
  float* merge_m = reinterpret_cast<float*>(smem);                 // [warps][16]
  float* merge_l = merge_m + DEC_WARPS * 16;                       // [warps][16]
  float* merge_o = merge_l + DEC_WARPS * 16;                       // [warps][16][head_dim + 8]: rows in different banks
  const int merge_stride = head_dim + 8;
  const __nv_bfloat16* qt = q + ((size_t)tok * n_heads + (size_t)kv_head * group) * head_dim;

  if constexpr (BY_HEADS) {
    // query operand: column g = head g of the group (zero at or beyond the group)
    uint32_t qb[D_TILES / 2][2];
#pragma unroll
    for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int dim = ks * 16 + e * 8 + 2 * t;
        qb[ks][e] = (g < group && dim < head_dim) ? *reinterpret_cast<const uint32_t*>(qt + (size_t)g * head_dim + dim) : 0u;
      }
    HeadColumnState<D_TILES> st;
    st.init();
    issue_tile(0, 0);
    for (int i = 0; i < n_tiles; ++i) {
      if (i + 1 < n_tiles) { issue_tile(i + 1, (i + 1) & 1); cp_async_wait<1>(); }
      else cp_async_wait<0>();
      __syncthreads();
      const int key_abs = begin + i * XRT_BLOCK_TOKENS + warp * 16;
      if (key_abs < end)  // only the first and the last 16 keys a warp sees can hold a hidden key
        attend_16_keys_heads<D_TILES>(st, qb, k_tiles + (i & 1) * tile_bytes, v_tiles + (i & 1) * tile_bytes, warp * 16,
                                      key_abs, first_key, len, key_abs < first_key || key_abs + 16 > len, head_dim,
                                      scale_log2);
      __syncthreads();  // the buffer is free for the tile after next
    }
    // this warp's state into the merge area: row = head; the sums are spread over the lanes of a t
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 4);
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 8);
      st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 16);
      if (g == 0) { merge_m[warp * 16 + 2 * t + h] = st.m[h]; merge_l[warp * 16 + 2 * t + h] = st.l[h]; }
    }
#pragma unroll
    for (int dt = 0; dt < D_TILES / 2; ++dt) {
      if (dt * 16 < head_dim) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          merge_o[((size_t)warp * 16 + 2 * t + (e & 1)) * merge_stride + dt * 16 + g + (e >> 1) * 8] = st.o[dt][e];
      }
    }
  } else {
    // query fragments: rows = the group's heads (rows at or beyond the group are zero)
    uint32_t qf[D_TILES / 2][4];
    {
  #pragma unroll
      for (int ks = 0; ks < D_TILES / 2; ++ks) {
  #pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = g + (e & 1) * 8, dim = ks * 16 + (e >> 1) * 8 + 2 * t;
          qf[ks][e] = (row < group && dim < head_dim)
                          ? *reinterpret_cast<const uint32_t*>(qt + (size_t)row * head_dim + dim) : 0u;
        }
      }
    }

    SoftmaxState<D_TILES> st;
    st.init();
    const int key_lo[2] = {first_key, first_key};
    const int key_hi[2] = {len, len};
    issue_tile(0, 0);
    for (int i = 0; i < n_tiles; ++i) {
      if (i + 1 < n_tiles) { issue_tile(i + 1, (i + 1) & 1); cp_async_wait<1>(); }
      else cp_async_wait<0>();
      __syncthreads();
      const int key_abs = begin + i * XRT_BLOCK_TOKENS + warp * 16;
      if (key_abs < end)  // only the first and the last 16 keys a warp sees can hold a hidden key
        attend_16_keys<D_TILES>(st, qf, k_tiles + (i & 1) * tile_bytes, v_tiles + (i & 1) * tile_bytes, warp * 16,
                                key_abs, key_lo, key_hi, key_abs < first_key || key_abs + 16 > len, head_dim, scale_log2);
      __syncthreads();  // the buffer is free for the tile after next
    }

    // merge the four warps: maxima first, then the rescaled sums and outputs in warp order
  #pragma unroll
    for (int r = 0; r < 2; ++r) {
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
      if (t == 0) { merge_m[warp * 16 + g + r * 8] = st.m[r]; merge_l[warp * 16 + g + r * 8] = st.l[r]; }
    }
  #pragma unroll
    for (int dt = 0; dt < D_TILES; ++dt) {
      if (dt * 8 < head_dim) {
  #pragma unroll
        for (int e = 0; e < 4; ++e)
          merge_o[((size_t)warp * 16 + g + (e >> 1) * 8) * merge_stride + dt * 8 + 2 * t + (e & 1)] = st.o[dt][e];
      }
    }
  }
  decode_finish(smem, out, part_o, part_ml, counters, tok, kv_head, split, n_splits, chunk, first_key, len, group, n_heads,
                n_kv_heads, head_dim);
}

// One warp per (token, head): merges the splits' partials in split order.
__global__ void attention_combine_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, const int* __restrict__ tok_slot,
                                         const int* __restrict__ tok_pos, int n_tokens, int n_heads, int head_dim,
                                         int window, int chunk, int n_splits) {
  pdl_trigger();
  pdl_wait();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp_global >= n_tokens * n_heads) return;
  const int tok = warp_global / n_heads;
  __nv_bfloat16* dst = out + (size_t)warp_global * head_dim;
  if (tok_slot[tok] < 0) {
    for (int d = lane; d < head_dim; d += 32) dst[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const int len = tok_pos[tok] + 1;
  const int first_key = window > 0 ? max(0, len - window) : 0;
  const size_t base = (size_t)warp_global * n_splits;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) {
    const bool live = split_live(s, chunk, first_key, len);
    if (live) m = fmaxf(m, part_ml[(base + s) * 2]);
  }
  float l = 0.f;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  // splits in order; loads are predicated rather than skipped so that several splits' loads are
  // in flight at once (a dead split's partials are never read: they may hold anything)
#pragma unroll 4
  for (int s = 0; s < n_splits; ++s) {
    const bool live = split_live(s, chunk, first_key, len);
    const float ms = live ? part_ml[(base + s) * 2] : -INFINITY;
    const float ls = live ? part_ml[(base + s) * 2 + 1] : 0.f;
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
    l += f * ls;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      const float o = (live && d < head_dim) ? part_o[(base + s) * head_dim + d] : 0.f;
      acc[j] += f * o;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = lane + 32 * j;
    if (d < head_dim) dst[d] = __float2bfloat16_rn(acc[j] / l);
  }
}

// The form with the heads as columns, fed by TMA: a cache block's keys and values for one kv head
// are 64 x head_dim contiguous bfloat16, which one thread fetches with one tensor copy per 64 dims
// (cp.async.bulk.tensor, 128-byte swizzle so that ldmatrix meets no bank conflict) instead of every
// thread issuing 16-byte copies: the copies were more than half of the instructions of the kernel
// above, which is bound by instruction issue.  Two buffers; the copy of tile i + 1 is issued before
// the wait for tile i.  The wait is bounded: if it runs out the block raises the error flag, waits
// (bounded) for its copies in flight and leaves without writing.
constexpr int DEC_BOX_BYTES = 64 * 128;
// Tiles of 64 keys and of 64 values in shared memory, each kind in a ring and on barriers of its own: one tile being
// worked on, the others on their way.  A tile's copy takes about 1.1 microseconds to land and a block's four warps
// about 0.8 to work a tile off, so with two buffers (one copy in flight) a tile costs (1.1 + 0.8) / 2 = 1
// microsecond, with three what the warps need.  The values are read in the second half of a tile's work, so two
// buffers are enough for them when the keys have three: 81 KB a block at head size 128 instead of 97.  The size
// matters beyond this kernel: what a block leaves free of a multiprocessor's shared memory is where the blocks
// of the next product wait with their first weights (the same kernel with 32 KB of unused shared memory: 3.59
// against 3.35 ms a step at 4 sequences).  Three key buffers where two blocks a multiprocessor hold the whole launch;
// two where more blocks have to be resident to fill the device (64 sequences with three: 9.17 against 8.80 ms).
constexpr int DEC_MAX_STAGES = 3;   // buffers of keys at most
constexpr int DEC_VALUE_STAGES = 2;  // buffers of values
constexpr unsigned DEC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t dec_map_rank(uint32_t local_smem, int rank) {  // the same place in another block of the cluster
  uint32_t remote;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem), "r"(rank));
  return remote;
}
constexpr int DEC_MAX_CLUSTER = 16;  // the most splits that merge as one cluster
__device__ __forceinline__ float dec_ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

__device__ __forceinline__ bool dec_mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned spin = 0; spin < DEC_SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// What the kernel needs to do the step between the q/k/v product and attention itself (head norms,
// rotation, the newest key and value into the cache: crates/xrt-models/src/llama.rs:488-503) instead of
// a kernel of its own before it.  qkv == nullptr: q comes rotated in bfloat16 as before.
struct DecodeFusedInput {
  const float* qkv = nullptr;        // [tokens, row_stride] 32-bit: q at 0, k at k_offset, v at v_offset
  int row_stride = 0, k_offset = 0, v_offset = 0;
  const void* q_norm_w = nullptr;    // [head_dim] or null (no head norm); both or neither
  const void* k_norm_w = nullptr;
  int norm_dtype = XRT_F32;
  float eps = 0.f;
  const float2* cos_sin = nullptr;   // [tokens, head_dim / 2] (cos, sin), or null: no rotation
  __nv_bfloat16* k_pool = nullptr;   // null: the newest key and value are in the cache already (a layer that reads another's)
  __nv_bfloat16* v_pool = nullptr;
};

__device__ __forceinline__ float dec_norm_weight(const void* w, int dtype, int d) {
  return dtype == XRT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[d])
                           : reinterpret_cast<const float*>(w)[d];
}

template <int HD_MAX>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                            const __nv_bfloat16* __restrict__ q, const int* __restrict__ tok_slot,
                            const int* __restrict__ tok_pos, const int* __restrict__ block_table, int max_blocks,
                            int n_heads, int n_kv_heads, int head_dim, float scale_log2, int window, int chunk,
                            int n_splits, int* __restrict__ counters, int* __restrict__ error_flag, int clustered,
                            int stages, const DecodeFusedInput fused) {
  constexpr int D_TILES = HD_MAX / 8;
  __shared__ __align__(16) __nv_bfloat16 newest[2][HD_MAX];  // the step's own key and value of this kv head
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full[DEC_MAX_STAGES + DEC_VALUE_STAGES];  // keys' buffers, then values'
  pdl_trigger();
  // The step's arrays (slots, positions, block table) were written before the step began: they may be
  // read, and tiles of old keys fetched, while the kernel before this one (which writes q and the
  // newest key and value) is still running.
  const int split = blockIdx.x, kv_head = blockIdx.y, tok = blockIdx.z;
  const int slot = tok_slot[tok];
  const int group = n_heads / n_kv_heads;
  if (slot < 0) {  // a padding row: zeros (with several splits and no counters the combine kernel writes them)
    // (the same for every block of a cluster: all of them leave here, none waits for another)
    pdl_wait();
    if (n_splits == 1 || ((counters != nullptr || clustered) && split == 0)) {
      __nv_bfloat16* dst = out + ((size_t)tok * n_heads + (size_t)kv_head * group) * head_dim;
      for (int i = threadIdx.x; i < group * head_dim; i += blockDim.x) dst[i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int len = tok_pos[tok] + 1;
  const int first_key = window > 0 ? max(0, len - window) : 0;
  const int begin = split_begin(split, chunk, first_key);
  const int end = split_end(split, chunk, first_key, len);
  const bool has_keys = begin < end;
  if (!has_keys && !clustered) { pdl_wait(); return; }  // this split holds no visible key: the combine step skips it too

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int boxes = head_dim / 64;
  const int tile_bytes = boxes * DEC_BOX_BYTES;
  unsigned char* k_tiles = smem;                   // [stages][boxes][64 rows x 128 bytes]
  unsigned char* v_tiles = smem + stages * tile_bytes;  // [DEC_VALUE_STAGES][boxes][64 rows x 128 bytes]
  const uint32_t full_base = smem_addr(&full[0]);
  auto k_full = [full_base](int stage) { return full_base + 8u * (uint32_t)stage; };
  auto v_full = [full_base](int stage) { return full_base + 8u * (uint32_t)(DEC_MAX_STAGES + stage); };
  if (threadIdx.x == 0) {
#pragma unroll
    for (int j = 0; j < DEC_MAX_STAGES + DEC_VALUE_STAGES; ++j)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full_base + 8u * (uint32_t)j));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int* blocks = block_table + (size_t)slot * max_blocks;
  const int n_tiles = has_keys ? (end - begin + XRT_BLOCK_TOKENS - 1) / XRT_BLOCK_TOKENS : 0;  // begin is a multiple of 64
  // keys and values are read once a step: their lines are the first to leave the L2
  const uint64_t once = sm100::policy_evict_first();
  // Lane 0 of warp 0 asks for the tiles of keys, lane 0 of warp 1 for the tiles of values (a copy instruction costs
  // the thread that issues it about 200 cycles, and its warp has its 16 keys to work on like the others).  Each has
  // the cache block's number of the tile it asks for next in a register, read from the block table a tile earlier:
  // that read's latency is not in the way of the copy.
  const bool asks = lane == 0 && warp < 2;
  const int my_stages = warp == 0 ? stages : DEC_VALUE_STAGES;  // of the ring this thread asks for
  auto block_of = [&](int tile_index) { return __ldg(blocks + begin / XRT_BLOCK_TOKENS + tile_index); };
  int next_block = 0;
  auto issue_tile = [&](int tile_index, int buffer, int block) {  // the two asking threads, each into its own ring
    const int row0 = (block * n_kv_heads + kv_head) * XRT_BLOCK_TOKENS;
    const uint32_t bar = warp == 0 ? k_full(buffer) : v_full(buffer);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tile_bytes) : "memory");
    // one copy a tile: the map's third dimension walks the row's pieces of 64 dims, so that the boxes of 64 rows x
    // 128 bytes land one behind the other
    if (warp == 0)
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
                   ::"r"(smem_addr(k_tiles + buffer * tile_bytes)), "l"(&map_k), "r"(0), "r"(row0), "r"(0), "r"(bar), "l"(once)
                   : "memory");
    else
      asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
                   ::"r"(smem_addr(v_tiles + buffer * tile_bytes)), "l"(&map_v), "r"(0), "r"(row0), "r"(0), "r"(bar), "l"(once)
                   : "memory");
    if (tile_index + 1 < n_tiles) next_block = block_of(tile_index + 1);
  };

  // query operand: column g = head g of the group (zero at or beyond the group)
  // The first tile before the wait, unless it holds the newest key (position len - 1) and the kernel
  // before this one writes that key; when this kernel writes it itself, the tile's row is patched below.
  const bool holds_newest = has_keys && len - 1 >= begin && len - 1 < end;
  const bool writes_newest = fused.qkv != nullptr && fused.k_pool != nullptr && holds_newest;
  const bool early = has_keys && (fused.qkv != nullptr || begin + XRT_BLOCK_TOKENS <= len - 1);
  if (asks && early) issue_tile(0, 0, block_of(0));
  pdl_wait();
  uint32_t qb[D_TILES / 2][2];
  if (fused.qkv == nullptr) {
    const __nv_bfloat16* qt = q + ((size_t)tok * n_heads + (size_t)kv_head * group) * head_dim;
#pragma unroll
    for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int dim = ks * 16 + e * 8 + 2 * t;
        qb[ks][e] = (g < group && dim < head_dim) ? *reinterpret_cast<const uint32_t*>(qt + (size_t)g * head_dim + dim) : 0u;
      }
  } else {
    // head_dim == HD_MAX here.  This lane holds dims ks * 16 + e * 8 + 2t, +1 of head g: the partner of a
    // dim in the rotation, head_dim / 2 further on, is in the same lane (ks + D_TILES / 4).
    constexpr int HALF_KS = D_TILES / 4;
    const float* qrow = fused.qkv + (size_t)tok * fused.row_stride + ((size_t)kv_head * group + g) * HD_MAX;
    float x[D_TILES / 2][2][2];
    float sq = 0.f;
#pragma unroll
    for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float2 two = g < group ? *reinterpret_cast<const float2*>(qrow + ks * 16 + e * 8 + 2 * t) : make_float2(0.f, 0.f);
        x[ks][e][0] = two.x;
        x[ks][e][1] = two.y;
        sq = fmaf(two.x, two.x, sq);
        sq = fmaf(two.y, two.y, sq);
      }
    if (fused.q_norm_w != nullptr) {
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      const float inv = 1.0f / sqrtf(sq / (float)HD_MAX + fused.eps);
#pragma unroll
      for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            x[ks][e][j] = (x[ks][e][j] * inv) * dec_norm_weight(fused.q_norm_w, fused.norm_dtype, ks * 16 + e * 8 + 2 * t + j);
    }
    if (fused.cos_sin != nullptr) {
      const float2* cs = fused.cos_sin + (size_t)tok * (HD_MAX / 2);
#pragma unroll
      for (int ks = 0; ks < HALF_KS; ++ks)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float4 a = *reinterpret_cast<const float4*>(cs + ks * 16 + e * 8 + 2 * t);  // (cos, sin) of two dims
          const float c2[2] = {a.x, a.z}, s2[2] = {a.y, a.w};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float x0 = x[ks][e][j], x1 = x[ks + HALF_KS][e][j];
            x[ks][e][j] = x0 * c2[j] - x1 * s2[j];
            x[ks + HALF_KS][e][j] = x0 * s2[j] + x1 * c2[j];
          }
        }
    }
#pragma unroll
    for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
      for (int e = 0; e < 2; ++e) qb[ks][e] = g < group ? pack_bf16(x[ks][e][0], x[ks][e][1]) : 0u;
    if (writes_newest) {
      // Warp 0: the newest key (head norm, rotation); warp 1: the newest value.  A lane holds dims
      // lane + 32 j; the rotation's partner of a dim is in the same lane.  Both go to the cache for the
      // steps to come and to shared memory for this step (the tile's row is patched when it has landed).
      if (warp < 2) {
        constexpr int PER_LANE = HD_MAX / 32;
        const float* row = fused.qkv + (size_t)tok * fused.row_stride + (warp == 0 ? fused.k_offset : fused.v_offset) +
                           (size_t)kv_head * HD_MAX;
        float y[PER_LANE];
        float ssq = 0.f;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
          y[j] = row[lane + 32 * j];
          ssq = fmaf(y[j], y[j], ssq);
        }
        if (warp == 0 && fused.k_norm_w != nullptr) {
          const float inv = 1.0f / sqrtf(warp_sum(ssq) / (float)HD_MAX + fused.eps);
#pragma unroll
          for (int j = 0; j < PER_LANE; ++j) y[j] = (y[j] * inv) * dec_norm_weight(fused.k_norm_w, fused.norm_dtype, lane + 32 * j);
        }
        if (warp == 0 && fused.cos_sin != nullptr) {
          const float2* cs = fused.cos_sin + (size_t)tok * (HD_MAX / 2);
#pragma unroll
          for (int j = 0; j < PER_LANE / 2; ++j) {
            const float2 a = cs[lane + 32 * j];
            const float x0 = y[j], x1 = y[j + PER_LANE / 2];
            y[j] = x0 * a.x - x1 * a.y;
            y[j + PER_LANE / 2] = x0 * a.y + x1 * a.x;
          }
        }
        const int block = blocks[(len - 1) / XRT_BLOCK_TOKENS];
        __nv_bfloat16* pool = warp == 0 ? fused.k_pool : fused.v_pool;
        __nv_bfloat16* dst = pool + (((size_t)block * n_kv_heads + kv_head) * XRT_BLOCK_TOKENS + (len - 1) % XRT_BLOCK_TOKENS) * HD_MAX;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
          const __nv_bfloat16 b = __float2bfloat16_rn(y[j]);
          newest[warp][lane + 32 * j] = b;
          if (block >= 0) dst[lane + 32 * j] = b;
        }
      }
      __syncthreads();
    }
  }
  HeadColumnState<D_TILES> st;
  st.init();
  if (asks) {
    if (n_tiles > 0 && !early) issue_tile(0, 0, block_of(0));
    for (int j = 1; j < my_stages - 1 && j < n_tiles; ++j) issue_tile(j, j, next_block);
  }
  int failed = 0, i = 0;
  int k_stage = 0, v_stage = 0;             // i % stages, i % DEC_VALUE_STAGES
  int ahead_stage = my_stages - 1;          // an asking thread: (i + its ring's buffers - 1) % its ring's buffers
  uint32_t k_parity = 0, v_parity = 0;      // (i / buffers) % 2
  for (; i < n_tiles; ++i) {
    // the buffer of tile i + buffers - 1 held tile i - 1, which every warp left before the barrier that ended the last round
    const int ahead = i + my_stages - 1;
    if (asks && ahead < n_tiles) issue_tile(ahead, ahead_stage, next_block);
    if (!dec_mbar_wait(k_full(k_stage), k_parity)) failed = 1;
    if (writes_newest && i == n_tiles - 1) {
      if (!dec_mbar_wait(v_full(v_stage), v_parity)) failed = 1;
      // the newest key and value into their row of the tile that has just landed (whatever the copy
      // read there): piece c of row r lies at piece c ^ (r % 8) of its box of 64 dims
      const int r = (len - 1) % XRT_BLOCK_TOKENS;
      if (threadIdx.x < 2 * (HD_MAX / 8)) {
        const int which = threadIdx.x / (HD_MAX / 8), piece = threadIdx.x % (HD_MAX / 8);
        unsigned char* tile = which == 0 ? k_tiles + k_stage * tile_bytes : v_tiles + v_stage * tile_bytes;
        *reinterpret_cast<uint4*>(tile + (piece >> 3) * DEC_BOX_BYTES + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) =
            *reinterpret_cast<const uint4*>(&newest[which][piece * 8]);
      }
      __syncthreads();
    }
    const int key_abs = begin + i * XRT_BLOCK_TOKENS + warp * 16;
    if (!failed && key_abs < end) {  // only the first and the last 16 keys a warp sees can hold a hidden key
      const uint32_t values_bar = v_full(v_stage);
      if (!attend_16_keys_heads<D_TILES, true>(st, qb, k_tiles + k_stage * tile_bytes, v_tiles + v_stage * tile_bytes,
                                               warp * 16, key_abs, first_key, len,
                                               key_abs < first_key || key_abs + 16 > len, head_dim, scale_log2,
                                               [&] { return dec_mbar_wait(values_bar, v_parity); }))
        failed = 1;
    }
    if (__syncthreads_or(failed)) { failed = 1; break; }
    ahead_stage = warp == 0 ? k_stage : v_stage;
    if (++k_stage == stages) { k_stage = 0; k_parity ^= 1u; }
    if (++v_stage == DEC_VALUE_STAGES) { v_stage = 0; v_parity ^= 1u; }
  }
  if (failed) {
    if (threadIdx.x == 0) {
      if (error_flag != nullptr) atomicCAS(error_flag, 0, 6);
      // copies in flight write this block's shared memory: they must have landed before it is given back
      for (int j = i; j < i + stages && j < n_tiles; ++j)
        dec_mbar_wait(k_full(j % stages), (uint32_t)(j / stages) & 1u);
      for (int j = i; j < i + DEC_VALUE_STAGES && j < n_tiles; ++j)
        dec_mbar_wait(v_full(j % DEC_VALUE_STAGES), (uint32_t)(j / DEC_VALUE_STAGES) & 1u);
    }
    __syncthreads();
    if (!clustered) return;  // in a cluster the block still meets the others (its state below is meaningless)
  }

  // this warp's state into the merge area: row = head; the sums are spread over the lanes of a t
  float* merge_m = reinterpret_cast<float*>(smem);
  float* merge_l = merge_m + DEC_WARPS * 16;
  float* merge_o = merge_l + DEC_WARPS * 16;
  const int merge_stride = head_dim + 8;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 4);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 8);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 16);
    if (g == 0) { merge_m[warp * 16 + 2 * t + h] = st.m[h]; merge_l[warp * 16 + 2 * t + h] = st.l[h]; }
  }
#pragma unroll
  for (int dt = 0; dt < D_TILES / 2; ++dt) {
    if (dt * 16 < head_dim) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        merge_o[((size_t)warp * 16 + 2 * t + (e & 1)) * merge_stride + dt * 16 + g + (e >> 1) * 8] = st.o[dt][e];
    }
  }
  if (!clustered) {
    decode_finish(smem, out, part_o, part_ml, counters, tok, kv_head, split, n_splits, chunk, first_key, len, group, n_heads,
                  n_kv_heads, head_dim);
    return;
  }

  // The splits of a (token, kv head) are the blocks of one thread-block cluster: each leaves its
  // merged (m, l, o) in its own shared memory, the cluster meets, and block `split` merges one slice
  // of the outputs from all blocks' shared memory (distributed shared memory), in split order.
  // No partials in global memory, no second kernel, no counter.
  __syncthreads();
  float* cta_ml = merge_o + DEC_WARPS * 16 * merge_stride;  // [group][2], behind the warps' states
  float* cta_o = cta_ml + 2 * 16;                           // [group][head_dim]
  for (int idx = threadIdx.x; idx < group * head_dim; idx += blockDim.x) {
    const int row = idx / head_dim, d = idx - row * head_dim;
    float m = -INFINITY, l = 0.f, o = 0.f;
    if (has_keys) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, merge_m[w * 16 + row]);
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float mw = merge_m[w * 16 + row];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
        l += f * merge_l[w * 16 + row];
        o += f * merge_o[((size_t)w * 16 + row) * merge_stride + d];
      }
    }
    cta_o[idx] = o;
    if (d == 0) { cta_ml[row * 2] = m; cta_ml[row * 2 + 1] = l; }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
  {
    const int total = group * head_dim;
    const int per = (total + n_splits - 1) / n_splits;
    const uint32_t ml_local = smem_addr(cta_ml), o_local = smem_addr(cta_o);
    for (int idx = split * per + threadIdx.x; idx < min(total, (split + 1) * per); idx += blockDim.x) {
      const int row = idx / head_dim;
      // every block's (m, l, o) of this output asked for before the first is used: the remote loads are in
      // flight together (one after the other they were most of a step's attention at one sequence)
      float ms[DEC_MAX_CLUSTER], ls[DEC_MAX_CLUSTER], os[DEC_MAX_CLUSTER];
#pragma unroll
      for (int s2 = 0; s2 < DEC_MAX_CLUSTER; ++s2) {
        ms[s2] = -INFINITY; ls[s2] = 0.f; os[s2] = 0.f;
        if (s2 < n_splits) {
          ms[s2] = dec_ld_cluster(dec_map_rank(ml_local + row * 8, s2));
          ls[s2] = dec_ld_cluster(dec_map_rank(ml_local + row * 8 + 4, s2));
          os[s2] = dec_ld_cluster(dec_map_rank(o_local + idx * 4, s2));
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < DEC_MAX_CLUSTER; ++s2) m = fmaxf(m, ms[s2]);
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < DEC_MAX_CLUSTER; ++s2) {  // in split order
        const float f = ms[s2] == -INFINITY ? 0.f : exp2f(ms[s2] - m);
        l += f * ls[s2];
        o += f * os[s2];
      }
      out[((size_t)tok * n_heads + (size_t)kv_head * group) * head_dim + idx] = __float2bfloat16_rn(o / l);
    }
  }
  // nobody leaves while another block may still read its shared memory
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// A map over a cache pool, a row-major bfloat16 matrix [blocks * kv heads * 64, head_dim], seen as
// [head_dim / 64 pieces][rows][64 dims]: a box is 64 dims x 64 rows x all pieces, 128-byte swizzle, so one copy
// brings a whole tile of 64 keys as head_dim / 64 boxes of 64 rows x 128 bytes, one behind the other.
static bool dec_make_map(CUtensorMap* map, const void* base, long long rows, int head_dim) {
  sm100::TensorMapEncodeFn encode = sm100::tensor_map_encoder();
  if (encode == nullptr) return false;
  const cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(head_dim / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, 128u};
  const cuuint32_t box[3] = {64u, 64u, (cuuint32_t)(head_dim / 64)};
  const cuuint32_t elem[3] = {1u, 1u, 1u};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// shared memory of the TMA kernel: the tiles (or the warps' states that reuse their room), then a
// block's merged state for the cluster merge
inline int decode_tma_smem(int head_dim, int stages = 2) {
  const int merge_bytes = DEC_WARPS * 16 * (2 + head_dim + 8) * (int)sizeof(float) + (2 * 16 + 8 * head_dim) * (int)sizeof(float);
  return 1024 + max((stages + DEC_VALUE_STAGES) * (head_dim / 64) * DEC_BOX_BYTES, merge_bytes);
}

// Three buffers where the blocks that fit a multiprocessor with three (at most three a multiprocessor, as with
// two) hold the whole launch; else two.
inline int decode_tma_stages(int head_dim, long long blocks) {
  static int sms = 0;
  if (sms == 0) {
    int device = 0, count = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      return 2;
    sms = count;
  }
  const int each = decode_tma_smem(head_dim, DEC_MAX_STAGES) + 2048;  // with the kernel's static arrays
  const int resident = min(3, 226 * 1024 / each);
  return blocks <= (long long)sms * resident ? DEC_MAX_STAGES : 2;
}

// Tuning::decode_attention = 3 keeps the merge by a second kernel or by the last block, for comparison.
// Only for few (token, kv head) pairs: measured at the 8B shape, clusters win at 1 to 4 sequences (3.77
// against 3.87 ms and 4.12 against 4.25 ms a step) and lose at 8 (4.90 against 4.68 ms: clusters of 6
// blocks of 66 KB each are harder to place than single blocks).
constexpr int DEC_CLUSTER_MAX_PAIRS = 32;

inline bool decode_cluster_wanted(int n_splits, int pairs) {
  const bool off = tuning().decode_attention == 3;
  return !off && n_splits >= 2 && n_splits <= DEC_MAX_CLUSTER && pairs <= tuning().decode_cluster_pairs;
}

template <int HD_MAX>
int launch_decode_tma(__nv_bfloat16* out, float* part_o, float* part_ml, const __nv_bfloat16* q,
                      const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, long long pool_rows, const int* tok_slot,
                      const int* tok_pos, const int* block_table, int max_blocks, int n_tokens, int n_heads, int n_kv_heads,
                      int head_dim, float scale, int window, int chunk, int n_splits, int* counters, int* error_flag,
                      cudaStream_t stream, bool* merged, const DecodeFusedInput& fused, bool clusters) {
  CUtensorMap map_k, map_v;
  if (!dec_make_map(&map_k, k_pool, pool_rows, head_dim) || !dec_make_map(&map_v, v_pool, pool_rows, head_dim))
    return XRT_ERR_UNSUPPORTED;
  auto kernel = attention_decode_tma_kernel<HD_MAX>;
  static int smem_allowed = 0;  // raised once a size class; not a stream operation
  auto allow = [&](int bytes) {
    if (bytes > 48 * 1024 && bytes > smem_allowed) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
      if (err != cudaSuccess) return (int)err;
      smem_allowed = bytes;
    }
    return 0;
  };
  // 2 to 16 splits: the splits of a (token, kv head) as one thread-block cluster that merges itself
  // through distributed shared memory, if the device can hold such a cluster (asked once a size)
  // by splits, head-size class and buffers: 0 unknown, else 1 + the clusters that the device holds at once
  static int cluster_room[DEC_MAX_CLUSTER + 1][5][DEC_MAX_STAGES + 1] = {};
  auto clusters_held = [&](int buffers) {
    int& known = cluster_room[n_splits][HD_MAX / 64][buffers];
    if (known == 0) {
      known = 1;
      const int bytes = decode_tma_smem(head_dim, buffers);
      if (allow(bytes) == 0 &&
          (n_splits <= 8 || cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess)) {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(n_splits, 1, 1);
        probe.blockDim = dim3(DEC_WARPS * 32);
        probe.dynamicSmemBytes = bytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = n_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        probe.attrs = attr;
        probe.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &probe) == cudaSuccess && clusters >= 1) known = 1 + clusters;
        cudaGetLastError();  // a refusal here is an answer, not an error of the stream
      }
    }
    return known - 1;
  };
  int stages = decode_tma_stages(head_dim, (long long)n_splits * n_kv_heads * n_tokens);
  bool clustered = false;
  if (clusters && decode_cluster_wanted(n_splits, n_tokens * n_kv_heads)) {
    // clusters of larger blocks are harder to place: three buffers of keys only for clusters of up to four blocks (8
    // splits of 4 sequences with three: 3.59 against 3.35 ms a step; 16 splits of 2 sequences: 3.44 against 3.38)
    // and where all of the launch's clusters still run at once
    if (stages > 2 && (n_splits > 4 || clusters_held(stages) < n_tokens * n_kv_heads)) stages = 2;
    clustered = clusters_held(stages) >= 1;
  }
  const int smem = decode_tma_smem(head_dim, stages);
  if (int err = allow(smem)) return err;
  *merged = clustered;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(n_splits, n_kv_heads, n_tokens);
  config.blockDim = dim3(DEC_WARPS * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n_attrs = 0;
  if (pdl_enabled()) {
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  if (clustered) {
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = n_splits; attrs[n_attrs].val.clusterDim.y = 1; attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  config.attrs = n_attrs ? attrs : nullptr;
  config.numAttrs = n_attrs;
  cudaLaunchKernelEx(&config, kernel, map_k, map_v, out, part_o, part_ml, q, tok_slot, tok_pos, block_table, max_blocks,
                     n_heads, n_kv_heads, head_dim, scale * 1.4426950408889634f, window, chunk, n_splits, counters, error_flag,
                     clustered ? 1 : 0, stages, fused);
  return launch_status();
}

template <int HD_MAX, bool BY_HEADS>
int launch_decode_as(__nv_bfloat16* out, float* part_o, float* part_ml, const __nv_bfloat16* q,
                  const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, const int* tok_slot, const int* tok_pos,
                  const int* block_table, int max_blocks, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                  float scale, int window, int chunk, int n_splits, int* counters, cudaStream_t stream) {
  const int tile_bytes = XRT_BLOCK_TOKENS * (head_dim * 2 + 16);
  const int merge_bytes = DEC_WARPS * 16 * (2 + head_dim + 8) * (int)sizeof(float);
  const int smem = max(4 * tile_bytes, merge_bytes);
  auto kernel = attention_decode_kernel<HD_MAX, BY_HEADS>;
  static int smem_allowed = 0;  // raised once a size class; not a stream operation
  if (smem > 48 * 1024 && smem > smem_allowed) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return (int)err;
    smem_allowed = smem;
  }
  dim3 grid(n_splits, n_kv_heads, n_tokens);
  launch_kernel(kernel, grid, dim3(DEC_WARPS * 32), (size_t)smem, stream, out, part_o, part_ml, q, k_pool, v_pool,
                tok_slot, tok_pos, block_table, max_blocks, n_heads, n_kv_heads, head_dim,
                scale * 1.4426950408889634f, window, chunk, n_splits, counters);
  return launch_status();
}

// Groups of at most 8 query heads take the form with the heads as the MMA's columns, fed by TMA when
// the head size is a multiple of 64 and the caller says how many blocks the pools hold.
// Tuning::decode_attention, for comparison: 1 keeps the heads-as-rows form everywhere, 2 keeps the
// 16-byte asynchronous copies, 3 keeps clusters off.
template <int HD_MAX>
int launch_decode(__nv_bfloat16* out, float* part_o, float* part_ml, const __nv_bfloat16* q,
                  const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool, long long pool_rows, const int* tok_slot,
                  const int* tok_pos, const int* block_table, int max_blocks, int n_tokens, int n_heads, int n_kv_heads,
                  int head_dim, float scale, int window, int chunk, int n_splits, int* counters, int* error_flag,
                  cudaStream_t stream, bool* merged, const DecodeFusedInput& fused, bool clusters) {
  *merged = false;
  const bool rows_only = tuning().decode_attention == 1, copies_only = tuning().decode_attention == 2;
  if (n_heads / n_kv_heads <= 8 && !rows_only && !copies_only && pool_rows > 0 && head_dim % 64 == 0 &&
      (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0) {
    // the kernel's own rotation walks a head of exactly the class's size in 32-bit pairs and quads
    if (fused.qkv != nullptr && (head_dim != HD_MAX || fused.row_stride % 4 != 0 || fused.k_offset % 4 != 0 ||
                                 fused.v_offset % 4 != 0 || (((uintptr_t)fused.qkv | (uintptr_t)fused.cos_sin) & 15) != 0))
      return XRT_ERR_UNSUPPORTED;
    return launch_decode_tma<HD_MAX>(out, part_o, part_ml, q, k_pool, v_pool, pool_rows, tok_slot, tok_pos, block_table,
                                     max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits,
                                     counters, error_flag, stream, merged, fused, clusters);
  }
  if (fused.qkv != nullptr) return XRT_ERR_UNSUPPORTED;  // only the kernel above rotates and writes the cache itself
  if (n_heads / n_kv_heads <= 8 && !rows_only)
    return launch_decode_as<HD_MAX, true>(out, part_o, part_ml, q, k_pool, v_pool, tok_slot, tok_pos, block_table,
                                          max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk,
                                          n_splits, counters, stream);
  return launch_decode_as<HD_MAX, false>(out, part_o, part_ml, q, k_pool, v_pool, tok_slot, tok_pos, block_table,
                                         max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk,
                                         n_splits, counters, stream);
}

// The merge by a (token, kv head)'s last block keeps group * (2 * n_splits + 1) floats in the block's
// dynamic shared memory.  The most splits for which that fits the smallest launch of any variant
// (the cp.async tiles, the TMA tiles after their alignment slack); beyond it the second kernel merges.
inline int decode_fused_max_splits(int head_dim, int group) {
  const int tile_bytes = XRT_BLOCK_TOKENS * (head_dim * 2 + 16);
  const int merge_bytes = DEC_WARPS * 16 * (2 + head_dim + 8) * (int)sizeof(float);
  int smallest = max(4 * tile_bytes, merge_bytes);
  if (head_dim % 64 == 0) smallest = min(smallest, decode_tma_smem(head_dim) - 1024);
  return (smallest / (int)sizeof(float) / group - 1) / 2;
}

}  // namespace xrt


XRT_EXPORT int xrt_attention_decode_fused_max_splits(int head_dim, int group) {
  if (head_dim < 16 || head_dim > 256 || head_dim % 16 != 0 || group < 1 || group > 16) return XRT_ERR_UNSUPPORTED;
  return xrt::decode_fused_max_splits(head_dim, group);
}

namespace xrt {

// counters == nullptr: partials, then the combine kernel.  Otherwise the last block of a
// (token, kv head) combines, and `counters` (int32 [n_tokens * n_kv_heads], zero before the call)
// is left zero.
static int attention_decode_impl(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool,
                                 const void* v_pool, int n_blocks, const int* tok_slot, const int* tok_pos,
                                 const int* block_table, int max_blocks, int n_tokens, int n_heads, int n_kv_heads,
                                 int head_dim, float scale, int window, int chunk, int n_splits, int* counters,
                                 int* error_flag, cudaStream_t stream, int* merged_out = nullptr,
                                 const DecodeFusedInput& fused = DecodeFusedInput(), bool clusters = true) {
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || chunk <= 0 || n_splits <= 0)
    return XRT_ERR_ARGUMENT;
  if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 256 || n_heads / n_kv_heads > 16 ||
      chunk % XRT_BLOCK_TOKENS != 0 || n_tokens > 65535 || n_kv_heads > 65535 || n_splits > 512)
    return XRT_ERR_UNSUPPORTED;
  if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  // more splits than the merging block's shared memory holds: the second kernel merges them
  if (counters != nullptr && n_splits > decode_fused_max_splits(head_dim, n_heads / n_kv_heads)) counters = nullptr;
  auto* o = (__nv_bfloat16*)out;
  auto* qp = (const __nv_bfloat16*)q;
  auto* kp = (const __nv_bfloat16*)k_pool;
  auto* vp = (const __nv_bfloat16*)v_pool;
  int status;
  bool merged = false;  // the attention kernel merged its splits itself (as clusters)
  const long long pool_rows = (long long)n_blocks * n_kv_heads * XRT_BLOCK_TOKENS;  // 0: the pools' size is not known
#define XRT_DECODE(HD) status = launch_decode<HD>(o, part_o, part_ml, qp, kp, vp, pool_rows, tok_slot, tok_pos, block_table, \
                                                  max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window,      \
                                                  chunk, n_splits, counters, error_flag, stream, &merged, fused, clusters)
  if (head_dim <= 32) XRT_DECODE(32);
  else if (head_dim <= 64) XRT_DECODE(64);
  else if (head_dim <= 128) XRT_DECODE(128);
  else XRT_DECODE(256);
#undef XRT_DECODE
  if (status != XRT_OK) return status;
  if (merged_out != nullptr) *merged_out = merged ? 1 : 0;
  if (n_splits > 1 && counters == nullptr && !merged) {
    const int warps = n_tokens * n_heads;
    launch_kernel(attention_combine_kernel, dim3((warps * 32 + 255) / 256), dim3(256), 0, stream, o,
                  (const float*)part_o, (const float*)part_ml, tok_slot, tok_pos, n_tokens, n_heads, head_dim, window,
                  chunk, n_splits);
    return launch_status();
  }
  return XRT_OK;
}

}  // namespace xrt

// q, out: bfloat16 [n_tokens, n_heads * head_dim], one token a sequence; pools bfloat16
// [blocks, kv heads, 64, head_dim].  `chunk` (a multiple of 64) keys a split, `n_splits` splits
// cover the longest sequence the launch may meet (with a window: the window and what is left of the cache
// block that holds its first key, window + 63 keys at most; splits are counted from that block).  part_o: float32 [n_tokens * n_heads * n_splits *
// head_dim] and part_ml: float32 [n_tokens * n_heads * n_splits * 2] are scratch, needed when
// n_splits > 1.  The group n_heads / n_kv_heads is at most 16; n_tokens at most 65535.
// n_blocks: blocks in each pool (0 if unknown: the kernels fed by TMA are then not used); error_flag
// (may be null): raised if a bounded wait on a copy ran out; *merged (may be null) is set to 1 when
// the attention kernel merged its splits itself, as thread-block clusters (then the partials are not
// touched and no second kernel runs), else 0.  clusters = 0 keeps the splits from merging as clusters:
// a cluster lives until its longest block is done, so where the sequences' lengths are far apart the
// blocks of a short sequence's splits would hold their places for nothing.
// This entry point merges the splits with a second kernel.
XRT_EXPORT int xrt_attention_decode(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool,
                                    const void* v_pool, int n_blocks, const int* tok_slot, const int* tok_pos,
                                    const int* block_table, int max_blocks, int n_tokens, int n_heads, int n_kv_heads,
                                    int head_dim, float scale, int window, int chunk, int n_splits, int* error_flag,
                                    cudaStream_t stream, int* merged, int clusters) {
  return xrt::attention_decode_impl(out, part_o, part_ml, q, k_pool, v_pool, n_blocks, tok_slot, tok_pos, block_table,
                                    max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits,
                                    nullptr, error_flag, stream, merged, xrt::DecodeFusedInput(), clusters != 0);
}

// The same, with the merge done by the block that brings a (token, kv head)'s last split: one
// launch instead of two.  counters: int32 [at least n_tokens * n_kv_heads], zero before the first
// call (the kernel leaves them zero).
XRT_EXPORT int xrt_attention_decode_fused(void* out, float* part_o, float* part_ml, int* counters, const void* q,
                                          const void* k_pool, const void* v_pool, int n_blocks, const int* tok_slot,
                                          const int* tok_pos, const int* block_table, int max_blocks, int n_tokens,
                                          int n_heads, int n_kv_heads, int head_dim, float scale, int window, int chunk,
                                          int n_splits, int* error_flag, cudaStream_t stream, int* merged, int clusters) {
  if (counters == nullptr) return XRT_ERR_ARGUMENT;
  return xrt::attention_decode_impl(out, part_o, part_ml, q, k_pool, v_pool, n_blocks, tok_slot, tok_pos, block_table,
                                    max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits,
                                    counters, error_flag, stream, merged, xrt::DecodeFusedInput(), clusters != 0);
}

// The same, fed with the 32-bit output of the q/k/v product instead of a rotated q: the kernel applies
// the head norms (q_norm_w, k_norm_w: [head_dim] in norm_dtype, or both null) and the split-half rotation
// over the whole head (cos_sin: float32 [n_tokens, head_dim / 2, 2], or null), and the block that holds a
// sequence's newest position writes its key and value into the cache (write_kv = 0: they are there
// already).  Only where the kernel fed by TMA runs: head_dim 64, 128 or 256, at most 8 query heads a kv
// head, n_blocks known; anything else is refused (-2) and the caller runs the rotation as a kernel of
// its own.  counters may be null (then a second kernel merges splits that did not merge as clusters).
XRT_EXPORT int xrt_attention_decode_qkv(void* out, float* part_o, float* part_ml, int* counters, const float* qkv,
                                        int row_stride, int k_offset, int v_offset, const void* q_norm_w,
                                        const void* k_norm_w, int norm_dtype, float eps, const float* cos_sin,
                                        int write_kv, void* k_pool, void* v_pool, int n_blocks, const int* tok_slot,
                                        const int* tok_pos, const int* block_table, int max_blocks, int n_tokens,
                                        int n_heads, int n_kv_heads, int head_dim, float scale, int window, int chunk,
                                        int n_splits, int* error_flag, cudaStream_t stream, int* merged, int clusters) {
  if (qkv == nullptr || (q_norm_w == nullptr) != (k_norm_w == nullptr) || n_blocks <= 0) return XRT_ERR_ARGUMENT;
  if (norm_dtype != XRT_F32 && norm_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  xrt::DecodeFusedInput fused;
  fused.qkv = qkv;
  fused.row_stride = row_stride; fused.k_offset = k_offset; fused.v_offset = v_offset;
  fused.q_norm_w = q_norm_w; fused.k_norm_w = k_norm_w; fused.norm_dtype = norm_dtype; fused.eps = eps;
  fused.cos_sin = (const float2*)cos_sin;
  fused.k_pool = write_kv ? (__nv_bfloat16*)k_pool : nullptr;
  fused.v_pool = write_kv ? (__nv_bfloat16*)v_pool : nullptr;
  return xrt::attention_decode_impl(out, part_o, part_ml, nullptr, k_pool, v_pool, n_blocks, tok_slot, tok_pos, block_table,
                                    max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits,
                                    counters, error_flag, stream, merged, fused, clusters != 0);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate: the scratch lives in this library's device
// image.  See attention_decode_static.h for who needs this and what the limits are.
#include <stdio.h>

#include <mutex>

#include "attention_decode_static.h"

namespace xrt {

constexpr size_t STATIC_SCRATCH_FLOATS = XRT_DECODE_STATIC_SCRATCH_BYTES / sizeof(float);
constexpr int STATIC_MAX_DEVICES = 64;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float decode_static_scratch[STATIC_SCRATCH_FLOATS];
static float* decode_static_scratch_address[STATIC_MAX_DEVICES] = {};
static std::mutex decode_static_setup;

static void refuse(char* message, int message_len, const char* text) {
  if (message != nullptr && message_len > 0) snprintf(message, (size_t)message_len, "%s", text);
}

}  // namespace xrt

int xrt_attention_decode_static(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int* tok_slot, const int* tok_pos, const int* block_table, int max_blocks,
                                int n_tokens, int n_heads, int n_kv_heads, int head_dim, float scale, int window,
                                int chunk, int n_splits, cudaStream_t stream, char* message, int message_len) {
  char text[256];
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_splits <= 0) {
    xrt::refuse(message, message_len, "xrt_attention_decode_static: a size is not positive");
    return XRT_ERR_ARGUMENT;
  }
  // floats of scratch: the (maximum, sum) pairs first, rounded up to 64 floats, then the outputs
  const size_t rows = (size_t)n_tokens * n_heads * n_splits;
  const size_t ml_floats = (rows * 2 + 63) / 64 * 64;
  const size_t need = n_splits > 1 ? ml_floats + rows * head_dim : 0;
  if (need > xrt::STATIC_SCRATCH_FLOATS) {
    snprintf(text, sizeof(text),
             "xrt_attention_decode_static: %d tokens x %d heads x %d splits need %zu bytes of scratch, the "
             "built-in scratch holds %u; use fewer splits or tokens, or xrt_attention_decode with scratch of your own",
             n_tokens, n_heads, n_splits, need * sizeof(float), (unsigned)XRT_DECODE_STATIC_SCRATCH_BYTES);
    xrt::refuse(message, message_len, text);
    return XRT_ERR_SCRATCH;
  }
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    xrt::refuse(message, message_len, "xrt_attention_decode_static: cudaGetDevice failed");
    return (int)err;
  }
  if (device < 0 || device >= xrt::STATIC_MAX_DEVICES) {
    xrt::refuse(message, message_len, "xrt_attention_decode_static: device ordinal out of range");
    return XRT_ERR_UNSUPPORTED;
  }
  // Set-up, once a device, with that device current: the device address of the scratch array.  Two host
  // threads that make a device's first call at the same moment are serialised here.
  std::lock_guard<std::mutex> guard(xrt::decode_static_setup);
  if (xrt::decode_static_scratch_address[device] == nullptr) {
    float* address = nullptr;
    err = cudaGetSymbolAddress((void**)&address, xrt::decode_static_scratch);
    if (err != cudaSuccess || address == nullptr) {
      snprintf(text, sizeof(text), "xrt_attention_decode_static: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(err));
      xrt::refuse(message, message_len, text);
      return err != cudaSuccess ? (int)err : XRT_ERR_UNSUPPORTED;
    }
    xrt::decode_static_scratch_address[device] = address;
  }
  float* scratch = xrt::decode_static_scratch_address[device];
  // the pools' size is not among this entry's arguments: 0 keeps it on the kernels that need no tensor map
  const int status = xrt_attention_decode(out, scratch + ml_floats, scratch, q, k_pool, v_pool, 0, tok_slot, tok_pos,
                                          block_table, max_blocks, n_tokens, n_heads, n_kv_heads, head_dim, scale,
                                          window, chunk, n_splits, nullptr, stream, nullptr, 1);
  if (status == XRT_ERR_ARGUMENT) xrt::refuse(message, message_len, "xrt_attention_decode_static: the kernel refused its arguments");
  if (status == XRT_ERR_UNSUPPORTED)
    xrt::refuse(message, message_len, "xrt_attention_decode_static: head_dim must be a multiple of 16 up to 256, at most "
                                      "16 query heads a kv head, chunk a multiple of 64, at most 65535 tokens");
  return status;
}
