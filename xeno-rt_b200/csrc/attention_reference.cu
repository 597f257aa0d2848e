// Causal grouped-query attention over the cache blocks, one warp per (token, query head).
// This is the kernel of the 32-bit path, for prompts and for single tokens alike: every
// (token, head) walks its keys in tiles of 32 from the same starting point in the same order,
// so its result does not depend on how tokens were cut into steps or batched.
//
// Formulas of the reference (crates/xrt-models/src/llama.rs):
//   kv head of query head h = h / (n_heads / n_kv_heads)                       :741
//   s_j = dot(q, k_j) / sqrt(head_dim), j = 0 .. pos (the causal mask is the bound)  :506, 736-751
//   online softmax: running maximum and sum, rescale on a new maximum, divide at the end  :514-574
// `window` > 0 keeps only keys with pos - j < window (absent in the reference; 0 = all keys).
#include "common.cuh"

namespace xrt {

template <typename TQ, typename TC, typename TO, int MAX_PER_LANE>
__global__ void attention_reference_kernel(
    TO* __restrict__ out, const TQ* __restrict__ q, const TC* __restrict__ k_pool,
    const TC* __restrict__ v_pool, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks, int n_heads, int n_kv_heads, int head_dim,
    float scale, int window) {
  extern __shared__ float q_staged[];  // [warps][head_dim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  if (head >= n_heads) return;
  const int slot = tok_slot[t];
  TO* dst = out + ((size_t)t * n_heads + head) * head_dim;
  if (slot < 0) {
    for (int d = lane; d < head_dim; d += 32) dst[d] = from_float<TO>(0.f);
    return;
  }
  const int pos = tok_pos[t];
  const int kv_head = head / (n_heads / n_kv_heads);
  float* qs = q_staged + warp * head_dim;
  const TQ* qr = q + ((size_t)t * n_heads + head) * head_dim;
  for (int d = lane; d < head_dim; d += 32) qs[d] = to_float(qr[d]);
  __syncwarp();

  float acc[MAX_PER_LANE];
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) acc[j] = 0.f;
  float running_max = -INFINITY, running_sum = 0.f;
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int* blocks = block_table + (size_t)slot * max_blocks;

  for (int base = (first_key / 32) * 32; base <= pos; base += 32) {
    const int block = blocks[base / XRT_BLOCK_TOKENS];
    const size_t tile = (((size_t)block * n_kv_heads + kv_head) * XRT_BLOCK_TOKENS + base % XRT_BLOCK_TOKENS) * head_dim;
    const int key = base + lane;
    const bool live = key >= first_key && key <= pos;
    float s = -INFINITY;
    if (live) {
      const TC* kr = k_pool + tile + (size_t)lane * head_dim;
      float dot = 0.f;
      for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
      s = dot * scale;
    }
    const float tile_max = warp_max(s);
    const float new_max = fmaxf(running_max, tile_max);
    const float correction = expf(running_max - new_max);  // exp(-inf) = 0 on the first tile
    const float p = live ? expf(s - new_max) : 0.f;
    running_sum = running_sum * correction + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) acc[j] *= correction;
    const int n_live = min(32, pos - base + 1);
    for (int kk = 0; kk < n_live; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const TC* vr = v_pool + tile + (size_t)kk * head_dim;
#pragma unroll
      for (int j = 0; j < MAX_PER_LANE; ++j) {
        const int d = lane + 32 * j;
        if (d < head_dim) acc[j] = fmaf(pk, to_float(vr[d]), acc[j]);
      }
    }
  }
  const float inv = 1.0f / running_sum;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int d = lane + 32 * j;
    if (d < head_dim) dst[d] = from_float<TO>(acc[j] * inv);
  }
}

}  // namespace xrt

// q: [n_tokens, n_heads * head_dim]; pools: [n_blocks, n_kv_heads, 64, head_dim]; out like q.
XRT_EXPORT int xrt_attention_reference(void* out, const void* q, const void* k_pool, const void* v_pool,
                                       const int* tok_slot, const int* tok_pos, const int* block_table,
                                       int max_blocks, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       float scale, int window, int q_dtype, int cache_dtype, int out_dtype,
                                       cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_heads % n_kv_heads != 0)
    return XRT_ERR_ARGUMENT;
  if (head_dim > 256) return XRT_ERR_UNSUPPORTED;
  if (n_tokens == 0) return XRT_OK;
  const int warps = 4;
  dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  XRT_DISPATCH_DTYPE(q_dtype, TQ, {
    XRT_DISPATCH_DTYPE(cache_dtype, TC, {
      XRT_DISPATCH_DTYPE(out_dtype, TO, {
        xrt::attention_reference_kernel<TQ, TC, TO, 8><<<grid, warps * 32, smem, stream>>>(
            (TO*)out, (const TQ*)q, (const TC*)k_pool, (const TC*)v_pool, tok_slot, tok_pos, block_table,
            max_blocks, n_heads, n_kv_heads, head_dim, scale, window);
      });
    });
  });
  return xrt::launch_status();
}
