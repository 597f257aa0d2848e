// Causal grouped-query attention for steps that bring several tokens a sequence (prompts), in
// bfloat16 on the tensor cores, sequences of unequal lengths laid end to end.
// (The reference's prefill form: crates/xrt-models/src/llama.rs:728-770: for token t the keys
// 0 .. start + t, read from the cache so that earlier context is included.)
//
// Grid (query tiles, heads, sequences).  A block of four warps owns 64 consecutive new tokens of one
// sequence for one query head, 16 rows a warp, and walks the sequence's cache blocks (64 keys each,
// contiguous in memory) from the first visible key to the last row's own position; tiles are
// copied to shared memory with cp.async, double-buffered, and every warp runs the same online
// softmax (32-bit maxima, sums and accumulators) over all keys of a tile.  The keys of this step
// were written to the cache before this kernel runs, so a step that continues a sequence and a
// step that starts one are the same case.  A row's result depends on its own query and the keys of
// its sequence only, not on what else the launch carries.
#include "attention_mma.cuh"

namespace xrt {

constexpr int PRE_WARPS = 4;
constexpr int PRE_ROWS = PRE_WARPS * 16;

template <int HD_MAX>
__global__ void __launch_bounds__(PRE_WARPS * 32)
attention_prefill_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q,
                         const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_start, const int* __restrict__ block_table, int max_blocks,
                         int n_heads, int n_kv_heads, int head_dim, float scale_log2, int window) {
  constexpr int D_TILES = HD_MAX / 8;
  extern __shared__ __align__(16) unsigned char smem[];
  // later query tiles walk more keys: they are scheduled first, the longest tiles of all heads and of all the step's
  // prompts before any shorter one (heads are the grid's fastest dimension, query tiles its slowest)
  const int q_tile = gridDim.z - 1 - blockIdx.z, head = blockIdx.x, seq = blockIdx.y;
  const int slot = seq_slot[seq];
  if (slot < 0) return;
  const int tok0 = cu_seqlens[seq];
  const int n_new = cu_seqlens[seq + 1] - tok0;
  const int row0 = q_tile * PRE_ROWS;
  if (row0 >= n_new) return;
  const int start = seq_start[seq];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int kv_head = head / (n_heads / n_kv_heads);
  const int row_bytes = tile_row_bytes(head_dim);
  const int tile_bytes = XRT_BLOCK_TOKENS * row_bytes;
  unsigned char* k_tiles = smem;
  unsigned char* v_tiles = smem + 2 * tile_bytes;

  // this lane's two query rows (new-token indices) and their key ranges
  const int rows[2] = {row0 + warp * 16 + g, row0 + warp * 16 + g + 8};
  int key_lo[2], key_hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int pos = start + rows[r];
    key_hi[r] = rows[r] < n_new ? pos + 1 : 0;  // a row beyond the sequence sees nothing
    key_lo[r] = window > 0 ? max(0, pos + 1 - window) : 0;
  }
  uint32_t qf[D_TILES / 2][4];
#pragma unroll
  for (int ks = 0; ks < D_TILES / 2; ++ks)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e & 1, dim = ks * 16 + (e >> 1) * 8 + 2 * t;
      qf[ks][e] = (rows[r] < n_new && dim < head_dim)
                      ? *reinterpret_cast<const uint32_t*>(q + ((size_t)(tok0 + rows[r]) * n_heads + head) * head_dim + dim)
                      : 0u;
    }

  // keys the block needs: from the first row's window edge to the last row's position
  const int last_row = min(row0 + PRE_ROWS, n_new) - 1;
  const int block_hi = start + last_row + 1;                                        // exclusive
  const int block_lo = window > 0 ? max(0, start + row0 + 1 - window) : 0;
  const int first_tile = block_lo / XRT_BLOCK_TOKENS;
  const int n_tiles = (block_hi + XRT_BLOCK_TOKENS - 1) / XRT_BLOCK_TOKENS - first_tile;
  // the warp's own range (uniform over the warp): rows warp*16 .. +16
  const int warp_first_row = row0 + warp * 16;
  const int warp_last_row = min(warp_first_row + 15, n_new - 1);
  const int warp_hi = warp_first_row < n_new ? start + warp_last_row + 1 : 0;
  const int warp_lo = window > 0 ? max(0, start + warp_first_row + 1 - window) : 0;
  // every row of the warp sees the keys in [warp_max_lo, warp_min_hi): a tile inside needs no mask
  const int warp_min_hi = warp_first_row < n_new ? start + warp_first_row + 1 : 0;
  const int warp_max_lo = window > 0 ? max(0, start + warp_last_row + 1 - window) : 0;
  const bool partial_warp = warp_first_row + 15 >= n_new;  // some rows lie beyond the sequence and see nothing

  const int* blocks = block_table + (size_t)slot * max_blocks;
  const size_t head_stride = (size_t)XRT_BLOCK_TOKENS * head_dim;
  TileCopier copier;
  copier.init(head_dim);
  auto issue_tile = [&](int tile_index, int buffer) {
    const int key0 = (first_tile + tile_index) * XRT_BLOCK_TOKENS;
    const int block = blocks[key0 / XRT_BLOCK_TOKENS];
    const size_t base = ((size_t)block * n_kv_heads + kv_head) * head_stride;
    const int live = min(XRT_BLOCK_TOKENS, block_hi - key0);
    copier.copy(k_tiles + buffer * tile_bytes, k_pool + base, XRT_BLOCK_TOKENS, live);
    copier.copy(v_tiles + buffer * tile_bytes, v_pool + base, XRT_BLOCK_TOKENS, live);
    cp_async_commit();
  };

  SoftmaxState<D_TILES> st;
  st.init();
  issue_tile(0, 0);
  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) { issue_tile(i + 1, (i + 1) & 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int key0 = (first_tile + i) * XRT_BLOCK_TOKENS;
    // uniform over the warp: does the tile hold any key this warp's rows see, and may it hide one?
    if (key0 < warp_hi && key0 + XRT_BLOCK_TOKENS > warp_lo) {
      const bool masked = partial_warp || key0 + XRT_BLOCK_TOKENS > warp_min_hi || key0 < warp_max_lo;
      attend_keys<D_TILES, XRT_BLOCK_TOKENS / 8>(st, qf, k_tiles + (i & 1) * tile_bytes, v_tiles + (i & 1) * tile_bytes,
                                                 0, key0, key_lo, key_hi, masked, head_dim, scale_log2);
    }
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
  }
#pragma unroll
  for (int dt = 0; dt < D_TILES; ++dt) {
    if (dt * 8 < head_dim) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (rows[r] < n_new) {
          const float inv = 1.0f / st.l[r];
          __nv_bfloat162 v = __floats2bfloat162_rn(st.o[dt][2 * r] * inv, st.o[dt][2 * r + 1] * inv);
          *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + rows[r]) * n_heads + head) * head_dim + dt * 8 + 2 * t) = v;
        }
      }
    }
  }
}

template <int HD_MAX>
int launch_prefill(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_bfloat16* k_pool, const __nv_bfloat16* v_pool,
                   const int* cu_seqlens, const int* seq_slot, const int* seq_start, const int* block_table,
                   int max_blocks, int n_seqs, int max_new, int n_heads, int n_kv_heads, int head_dim, float scale,
                   int window, cudaStream_t stream) {
  const int smem = 4 * XRT_BLOCK_TOKENS * (head_dim * 2 + 16);
  auto kernel = attention_prefill_kernel<HD_MAX>;
  static int smem_allowed = 0;
  if (smem > 48 * 1024 && smem > smem_allowed) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return (int)err;
    smem_allowed = smem;
  }
  dim3 grid(n_heads, n_seqs, (max_new + PRE_ROWS - 1) / PRE_ROWS);
  kernel<<<grid, PRE_WARPS * 32, smem, stream>>>(out, q, k_pool, v_pool, cu_seqlens, seq_slot, seq_start, block_table,
                                                max_blocks, n_heads, n_kv_heads, head_dim,
                                                scale * 1.4426950408889634f, window);
  return launch_status();
}

}  // namespace xrt

// q, out: bfloat16 [total new tokens, n_heads * head_dim], the sequences' new tokens end to end
// (cu_seqlens[n_seqs + 1]); seq_slot[n_seqs] (< 0: skipped), seq_start[n_seqs] = tokens each sequence
// held before this step; max_new = the most new tokens any sequence brings.  Rows of skipped
// sequences are not written.
XRT_EXPORT int xrt_attention_prefill(void* out, const void* q, const void* k_pool, const void* v_pool,
                                     const int* cu_seqlens, const int* seq_slot, const int* seq_start,
                                     const int* block_table, int max_blocks, int n_seqs, int max_new, int n_heads,
                                     int n_kv_heads, int head_dim, float scale, int window, cudaStream_t stream) {
  if (n_seqs < 0 || max_new < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return XRT_ERR_ARGUMENT;
  if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 256 || n_seqs > 65535 || (max_new + xrt::PRE_ROWS - 1) / xrt::PRE_ROWS > 65535) return XRT_ERR_UNSUPPORTED;
  if (n_seqs == 0 || max_new == 0) return XRT_OK;
  auto* o = (__nv_bfloat16*)out;
  auto* qp = (const __nv_bfloat16*)q;
  auto* kp = (const __nv_bfloat16*)k_pool;
  auto* vp = (const __nv_bfloat16*)v_pool;
#define XRT_PREFILL(HD) return xrt::launch_prefill<HD>(o, qp, kp, vp, cu_seqlens, seq_slot, seq_start, block_table, \
                                                       max_blocks, n_seqs, max_new, n_heads, n_kv_heads, head_dim,  \
                                                       scale, window, stream)
  if (head_dim <= 32) XRT_PREFILL(32);
  if (head_dim <= 64) XRT_PREFILL(64);
  if (head_dim <= 128) XRT_PREFILL(128);
  XRT_PREFILL(256);
#undef XRT_PREFILL
}
