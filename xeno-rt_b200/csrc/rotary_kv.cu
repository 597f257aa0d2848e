// Rotation tables, and the fused step between the q/k/v product and attention:
// optional per-head RMSNorm of q and k, rotation of q and k, q written for the attention kernel
// and k, v written into the cache blocks of each token's sequence.
//
// Formulas of the reference:
//   angle = pos * scale / base^(2i/rope_dim), in 32-bit   crates/xrt-kernels/src/cpu/rope.rs:59-68
//   h[i]      = x0 * cos - x1 * sin                        crates/xrt-kernels/src/cpu/rope.rs:19-35
//   h[i+half] = x0 * sin + x1 * cos      (x0 = h[i], x1 = h[i + half]; split-half pairing)
// The reference pairs (i, i + half) only.  `interleaved` pairs (2i, 2i + 1) instead, for position
// encodings that rotate neighbours; dims from 2 * rope_half on are left as they are either way.
//   head norm = RMSNorm over each head slice, one weight   crates/xrt-models/src/llama.rs:1025-1040
//   order     = projection, head norm, rotation, cache     crates/xrt-models/src/llama.rs:488-503
#include "common.cuh"

namespace xrt {

// cos_sin[t, i] = (cos, sin) of pos[t] * scale / freq[i]; freq is the divisor table base^(2i/rd).
__global__ void rope_table_kernel(float2* __restrict__ cos_sin, const int* __restrict__ pos,
                                  const float* __restrict__ freq, float scale, int n_tokens, int half) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * half) return;
  const int t = i / half, p = i - t * half;
  const float angle = __fdiv_rn(__fmul_rn((float)pos[t], scale), freq[p]);
  float s, c;
  sincosf(angle, &s, &c);
  cos_sin[i] = make_float2(c, s);
}

// One warp per (token, head) among [q heads | k heads | v heads].  MAX_PER_LANE * 32 >= head_dim.
template <typename TN, typename TQ, typename TC, int MAX_PER_LANE>
__global__ void qk_rope_kv_write_kernel(
    TQ* __restrict__ q_out, TC* __restrict__ k_pool, TC* __restrict__ v_pool,
    const float* __restrict__ qkv, int row_stride, int k_offset, int v_offset,
    const TN* __restrict__ q_norm_w, const TN* __restrict__ k_norm_w, float eps,
    const float2* __restrict__ cos_sin, int rope_half,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks,
    int n_heads, int n_kv_heads, int head_dim, int write_kv, int interleaved) {
  extern __shared__ float staged[];  // [warps][head_dim]
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head_slot = blockIdx.y * (blockDim.x >> 5) + warp;
  const int n_slots = n_heads + (write_kv ? 2 * n_kv_heads : 0);
  if (head_slot >= n_slots) return;
  const int slot = tok_slot[t];
  const int pos = tok_pos[t];

  // which of q / k / v, and which head of it
  int kind, head;
  if (head_slot < n_heads) { kind = 0; head = head_slot; }
  else if (head_slot < n_heads + n_kv_heads) { kind = 1; head = head_slot - n_heads; }
  else { kind = 2; head = head_slot - n_heads - n_kv_heads; }

  if (slot < 0) {  // a padding row: q is zeroed, the cache is not touched
    if (kind == 0)
      for (int d = lane; d < head_dim; d += 32)
        q_out[(size_t)t * n_heads * head_dim + head * head_dim + d] = from_float<TQ>(0.f);
    return;
  }

  const float* src = qkv + (size_t)t * row_stride +
                     (kind == 0 ? 0 : (kind == 1 ? k_offset : v_offset)) + head * head_dim;
  float v[MAX_PER_LANE];
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int d = lane + 32 * j;
    v[j] = d < head_dim ? src[d] : 0.f;
    sq = fmaf(v[j], v[j], sq);
  }
  const TN* norm_w = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
  if (norm_w != nullptr) {
    const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)head_dim + eps);
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int d = lane + 32 * j;
      if (d < head_dim) v[j] = (v[j] * inv) * to_float(norm_w[d]);
    }
  }

  float* mine = staged + warp * head_dim;
  if (kind != 2 && rope_half > 0) {
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int d = lane + 32 * j;
      if (d < head_dim) mine[d] = v[j];
    }
    __syncwarp();
    const float2* cs = cos_sin + (size_t)t * rope_half;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int d = lane + 32 * j;
      if (interleaved) {
        if (d < 2 * rope_half) {
          const float2 a = cs[d >> 1];
          v[j] = (d & 1) ? mine[d - 1] * a.y + mine[d] * a.x : mine[d] * a.x - mine[d + 1] * a.y;
        }
      } else if (d < rope_half) {
        const float2 a = cs[d];
        v[j] = mine[d] * a.x - mine[d + rope_half] * a.y;
      } else if (d < 2 * rope_half) {
        const float2 a = cs[d - rope_half];
        v[j] = mine[d - rope_half] * a.y + mine[d] * a.x;
      }
    }
  }

  if (kind == 0) {
    TQ* dst = q_out + (size_t)t * n_heads * head_dim + head * head_dim;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int d = lane + 32 * j;
      if (d < head_dim) dst[d] = from_float<TQ>(v[j]);
    }
  } else {
    const int block = block_table[(size_t)slot * max_blocks + pos / XRT_BLOCK_TOKENS];
    if (block < 0) return;  // the host reserves blocks before the step; nothing to write into
    TC* pool = kind == 1 ? k_pool : v_pool;
    TC* dst = pool + (((size_t)block * n_kv_heads + head) * XRT_BLOCK_TOKENS + pos % XRT_BLOCK_TOKENS) * head_dim;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int d = lane + 32 * j;
      if (d < head_dim) dst[d] = from_float<TC>(v[j]);
    }
  }
}

// The same for head size 128 with the rotation over all of the head (or none): a lane holds four
// consecutive dims (one 16-byte load), the partner of dim d, d +- 64, sits sixteen lanes away (a
// shuffle instead of shared memory), and a block of eight warps walks all heads of one token, so a
// prompt launches one block a token instead of twelve.
__device__ __forceinline__ void store4_as(float* dst, const float (&v)[4]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4_as(__nv_bfloat16* dst, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<uint32_t*>(&a);
  t.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(dst) = t;
}

template <typename TN, typename TQ, typename TC>
__global__ void __launch_bounds__(256)
qk_rope_kv_write_128_kernel(
    TQ* __restrict__ q_out, TC* __restrict__ k_pool, TC* __restrict__ v_pool,
    const float* __restrict__ qkv, int row_stride, int k_offset, int v_offset,
    const TN* __restrict__ q_norm_w, const TN* __restrict__ k_norm_w, float eps,
    const float2* __restrict__ cos_sin, int rope_half,
    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks,
    int n_heads, int n_kv_heads, int write_kv) {
  constexpr int HD = 128;
  pdl_trigger();
  // The step's arrays (slots, positions, block table) were written before the step began, and the norm
  // weights never change: they are read while the kernel before this one finishes.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int n_slots = n_heads + (write_kv ? 2 * n_kv_heads : 0);
  const int slot = tok_slot[t];
  const int pos = tok_pos[t];
  int block = -1;
  if (slot >= 0 && write_kv) block = block_table[(size_t)slot * max_blocks + pos / XRT_BLOCK_TOKENS];
  float qn[4] = {1.f, 1.f, 1.f, 1.f}, kn[4] = {1.f, 1.f, 1.f, 1.f};
  if (q_norm_w != nullptr) {
#pragma unroll
    for (int j = 0; j < 4; ++j) { qn[j] = to_float(q_norm_w[4 * lane + j]); kn[j] = to_float(k_norm_w[4 * lane + j]); }
  }
  pdl_wait();
  // (cos, sin) of this lane's four pairs: dims 4 * (lane % 16) .. of the first half
  float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
  if (rope_half > 0 && slot >= 0) {
    const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)t * rope_half + 4 * (lane & 15));
    const float4 a = cs[0], b = cs[1];
    c[0] = a.x; sn[0] = a.y; c[1] = a.z; sn[1] = a.w; c[2] = b.x; sn[2] = b.y; c[3] = b.z; sn[3] = b.w;
  }
  // A warp takes head slots warp, warp + 8, ...; it asks for the rows of up to four of them before it
  // works on the first (the rows come from the L2, and one load in flight a warp left the kernel waiting).
  constexpr int AHEAD = 4;
  for (int first = warp; first < n_slots; first += 8 * AHEAD) {
    float4 raw[AHEAD];
    if (slot >= 0) {
#pragma unroll
      for (int a = 0; a < AHEAD; ++a) {
        const int head_slot = first + 8 * a;
        if (head_slot < n_slots) {
          const int kind = head_slot < n_heads ? 0 : (head_slot < n_heads + n_kv_heads ? 1 : 2);
          const int head = head_slot - (kind == 0 ? 0 : (kind == 1 ? n_heads : n_heads + n_kv_heads));
          const float* src = qkv + (size_t)t * row_stride + (kind == 0 ? 0 : (kind == 1 ? k_offset : v_offset)) + head * HD;
          raw[a] = *reinterpret_cast<const float4*>(src + 4 * lane);
        }
      }
    }
#pragma unroll
    for (int a = 0; a < AHEAD; ++a) {
      const int head_slot = first + 8 * a;
      if (head_slot >= n_slots) break;
      const int kind = head_slot < n_heads ? 0 : (head_slot < n_heads + n_kv_heads ? 1 : 2);
      const int head = head_slot - (kind == 0 ? 0 : (kind == 1 ? n_heads : n_heads + n_kv_heads));
      float v[4];
      if (slot < 0) {  // a padding row: q is zeroed, the cache is not touched
        if (kind == 0) {
          v[0] = v[1] = v[2] = v[3] = 0.f;
          store4_as(q_out + (size_t)t * n_heads * HD + head * HD + 4 * lane, v);
        }
        continue;
      }
      v[0] = raw[a].x; v[1] = raw[a].y; v[2] = raw[a].z; v[3] = raw[a].w;
      const TN* norm_w = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
      if (norm_w != nullptr) {
        float sq = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) sq = fmaf(v[j], v[j], sq);
        const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)HD + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = (v[j] * inv) * (kind == 0 ? qn[j] : kn[j]);
      }
      if (kind != 2 && rope_half > 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
          // first half: x0 cos - x1 sin; second half: x0 sin + x1 cos, with x0 the first-half element
          v[j] = lane < 16 ? v[j] * c[j] - other * sn[j] : other * sn[j] + v[j] * c[j];
        }
      }
      if (kind == 0) {
        store4_as(q_out + (size_t)t * n_heads * HD + head * HD + 4 * lane, v);
      } else if (block >= 0) {  // the host reserves blocks before the step; otherwise nothing to write into
        TC* pool = kind == 1 ? k_pool : v_pool;
        store4_as(pool + (((size_t)block * n_kv_heads + head) * XRT_BLOCK_TOKENS + pos % XRT_BLOCK_TOKENS) * HD + 4 * lane, v);
      }
    }
  }
}

}  // namespace xrt


XRT_EXPORT int xrt_rope_table(float* cos_sin, const int* pos, const float* freq, float scale, int n_tokens,
                              int half, cudaStream_t stream) {
  if (n_tokens < 0 || half < 0) return XRT_ERR_ARGUMENT;
  const int total = n_tokens * half;
  if (total == 0) return XRT_OK;
  xrt::launch_kernel(xrt::rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, (float2*)cos_sin, pos, freq,
                     scale, n_tokens, half);
  return xrt::launch_status();
}

// qkv: 32-bit rows of `row_stride` floats holding q at 0, k at k_offset, v at v_offset.
// q_out: [n_tokens, n_heads * head_dim] in q_dtype.  k_pool / v_pool: the cache blocks of this
// layer, [n_blocks, n_kv_heads, 64, head_dim] in cache_dtype.  Norm weights may be null (no head
// norm) and share norm_dtype.  write_kv = 0 leaves the cache alone (a layer reading another's).
XRT_EXPORT int xrt_qk_rope_kv_write(void* q_out, void* k_pool, void* v_pool, const float* qkv, int row_stride,
                                    int k_offset, int v_offset, const void* q_norm_w, const void* k_norm_w,
                                    float eps, const float* cos_sin, int rope_half, const int* tok_slot,
                                    const int* tok_pos, const int* block_table, int max_blocks, int n_tokens,
                                    int n_heads, int n_kv_heads, int head_dim, int write_kv, int interleaved,
                                    int norm_dtype, int q_dtype, int cache_dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) return XRT_ERR_ARGUMENT;
  if (head_dim > 256 || 2 * rope_half > head_dim) return XRT_ERR_UNSUPPORTED;
  if ((q_norm_w == nullptr) != (k_norm_w == nullptr)) return XRT_ERR_ARGUMENT;
  if (n_tokens == 0) return XRT_OK;
  const bool fast = head_dim == 128 && (rope_half == 0 || (rope_half == 64 && !interleaved)) && row_stride % 4 == 0 && k_offset % 4 == 0 &&
                    v_offset % 4 == 0 &&
                    (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)cos_sin) & 15) == 0;
  if (fast) {
    XRT_DISPATCH_DTYPE(norm_dtype, TN, {
      XRT_DISPATCH_DTYPE(q_dtype, TQ, {
        XRT_DISPATCH_DTYPE(cache_dtype, TC, {
          xrt::launch_kernel(xrt::qk_rope_kv_write_128_kernel<TN, TQ, TC>, dim3(n_tokens), dim3(256), 0, stream,
              (TQ*)q_out, (TC*)k_pool, (TC*)v_pool, qkv, row_stride, k_offset, v_offset, (const TN*)q_norm_w,
              (const TN*)k_norm_w, eps, (const float2*)cos_sin, rope_half, tok_slot, tok_pos, block_table,
              max_blocks, n_heads, n_kv_heads, write_kv);
        });
      });
    });
    return xrt::launch_status();
  }
  const int warps = 4;
  const int n_slots = n_heads + (write_kv ? 2 * n_kv_heads : 0);
  dim3 grid(n_tokens, (n_slots + warps - 1) / warps);
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  XRT_DISPATCH_DTYPE(norm_dtype, TN, {
    XRT_DISPATCH_DTYPE(q_dtype, TQ, {
      XRT_DISPATCH_DTYPE(cache_dtype, TC, {
        xrt::launch_kernel(xrt::qk_rope_kv_write_kernel<TN, TQ, TC, 8>, grid, dim3(warps * 32), smem, stream,
            (TQ*)q_out, (TC*)k_pool, (TC*)v_pool, qkv, row_stride, k_offset, v_offset, (const TN*)q_norm_w,
            (const TN*)k_norm_w, eps, (const float2*)cos_sin, rope_half, tok_slot, tok_pos, block_table,
            max_blocks, n_heads, n_kv_heads, head_dim, write_kv, interleaved);
      });
    });
  });
  return xrt::launch_status();
}
