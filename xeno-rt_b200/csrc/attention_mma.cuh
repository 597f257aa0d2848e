// Building blocks of the bfloat16 attention kernels: asynchronous copies of key/value tiles from
// the cache blocks into padded shared-memory rows, ldmatrix loads of the MMA operands, the
// m16n8k16 tensor-core instruction and the online-softmax update of one 16-row query tile against
// 16 keys.  Scores, running maxima and sums, and the output accumulators are 32-bit.
#pragma once

#include "common.cuh"

namespace xrt {

// A row of a key/value tile holds head_dim bfloat16 and 16 bytes of padding, so that the eight rows
// an ldmatrix reads fall into different banks for every head_dim that is a multiple of 16.
__device__ __forceinline__ int tile_row_bytes(int head_dim) { return head_dim * 2 + 16; }

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// 16 bytes global -> shared; src_bytes = 0 writes zeros (used for keys beyond the sequence)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// How one thread takes part in copying tiles of `rows` x head_dim bfloat16 (contiguous in global
// memory) into padded shared rows: computed once a kernel, so that a tile costs a thread a few
// additions and its 16-byte asynchronous copies.  When the block's threads are a multiple of the
// 16-byte pieces of a row (head sizes 16, 32, 64, 128, 256 with 128 threads) a thread keeps one
// column of pieces and steps down the rows; other head sizes divide per piece.
struct TileCopier {
  int pieces_per_row, row_bytes, head_dim;
  int first_row, piece, row_step;  // the regular case
  bool regular;
  __device__ __forceinline__ void init(int head_dim_) {
    head_dim = head_dim_;
    pieces_per_row = head_dim / 8;
    row_bytes = tile_row_bytes(head_dim);
    regular = blockDim.x % pieces_per_row == 0;
    first_row = threadIdx.x / pieces_per_row;
    piece = threadIdx.x - first_row * pieces_per_row;
    row_step = blockDim.x / pieces_per_row;
  }
  // Rows at or beyond `live_rows` are zero-filled.  All threads of the block take part.
  __device__ __forceinline__ void copy(unsigned char* dst, const __nv_bfloat16* src, int rows, int live_rows) const {
    if (regular) {
      uint32_t d = smem_addr(dst + first_row * row_bytes + piece * 16);
      const __nv_bfloat16* s = src + (size_t)first_row * head_dim + piece * 8;
      const uint32_t d_step = (uint32_t)(row_step * row_bytes);
      const size_t s_step = (size_t)row_step * head_dim;
      for (int r = first_row; r < rows; r += row_step, d += d_step, s += s_step) cp_async_16(d, s, r < live_rows ? 16 : 0);
    } else {
      for (int c = threadIdx.x; c < rows * pieces_per_row; c += blockDim.x) {
        const int r = c / pieces_per_row, j = c - r * pieces_per_row;
        cp_async_16(smem_addr(dst + r * row_bytes + j * 16), src + (size_t)r * head_dim + j * 8, r < live_rows ? 16 : 0);
      }
    }
  }
};

// The running state of one warp's 16 query rows: lane (g = lane / 4, t = lane % 4) holds rows g
// and g + 8; `o` holds, for each 8-wide slice of head_dim, the four accumulators of the MMA layout.
template <int D_TILES>
struct SoftmaxState {
  float m[2];        // running maximum of the scaled scores (base-2 exponent domain)
  float l[2];        // this lane's share of the running sum
  float o[D_TILES][4];
  __device__ __forceinline__ void init() {
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
#pragma unroll
    for (int i = 0; i < D_TILES; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  }
};

// One warp: scores of its 16 query rows (fragments qf[ks]) against the 16 keys that start at row
// `key_row` of the key tile `ks_tile`, the online-softmax update, and the product with the same 16
// rows of the value tile `vs_tile`.  `scale_log2` = scale * log2(e).  Keys whose absolute index is
// not in [key_lo[r], key_hi[r]) are masked for row r (r = 0: row g, r = 1: row g + 8).
template <int D_TILES>
__device__ __forceinline__ void attend_16_keys(SoftmaxState<D_TILES>& st, const uint32_t (*qf)[4],
                                               const unsigned char* ks_tile, const unsigned char* vs_tile,
                                               int key_row, int key_abs, const int (&key_lo)[2], const int (&key_hi)[2],
                                               bool masked, int head_dim, float scale_log2) {
  const int lane = threadIdx.x & 31, t = lane & 3;
  const int row_bytes = tile_row_bytes(head_dim);
  const int j = lane >> 3, r = lane & 7;
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  // K operand: matrix j of an x4 load = keys (j / 2) * 8 .., dims ks * 16 + (j % 2) * 8 ..
  const uint32_t k_base = smem_addr(ks_tile + (key_row + (j >> 1) * 8 + r) * row_bytes + (j & 1) * 16);
#pragma unroll
  for (int ks = 0; ks < D_TILES / 2; ++ks) {
    if (ks * 16 < head_dim) {
      uint32_t kf[4];
      ldmatrix_x4(kf, k_base + ks * 32);
      mma_16816(s[0], qf[ks], kf[0], kf[1]);
      mma_16816(s[1], qf[ks], kf[2], kf[3]);
    }
  }
  // mask, scale, row maxima
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = e >> 1;
      bool live = true;
      if (masked) {  // uniform over the warp: only tiles at an edge of a row's key range pay for the comparisons
        const int key = key_abs + nt * 8 + 2 * t + (e & 1);
        live = key >= key_lo[row] && key < key_hi[row];
      }
      s[nt][e] = live ? s[nt][e] * scale_log2 : -INFINITY;
      tile_max[row] = fmaxf(tile_max[row], s[nt][e]);
    }
  float corr[2];
#pragma unroll
  for (int row = 0; row < 2; ++row) {
    tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 1));
    tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 2));
    const float m_new = fmaxf(st.m[row], tile_max[row]);
    // a row with no live key so far keeps m = -inf; exp2(-inf - -inf) must not be NaN
    corr[row] = m_new == -INFINITY ? 1.f : exp2f(st.m[row] - m_new);
    st.m[row] = m_new;
    st.l[row] *= corr[row];
  }
  // once a row's maximum has settled the accumulators need no rescaling: skip it for the whole warp
  const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f);
  uint32_t pf[4];
  {
    float p[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = e >> 1;
        p[nt][e] = st.m[row] == -INFINITY ? 0.f : exp2f(s[nt][e] - st.m[row]);
        st.l[row] += p[nt][e];
      }
    pf[0] = pack_bf16(p[0][0], p[0][1]);
    pf[1] = pack_bf16(p[0][2], p[0][3]);
    pf[2] = pack_bf16(p[1][0], p[1][1]);
    pf[3] = pack_bf16(p[1][2], p[1][3]);
  }
  // V operand (transposed load): matrix j = keys (j % 2) * 8 .., dims d0 + (j / 2) * 8 ..
  const uint32_t v_base = smem_addr(vs_tile + (key_row + (j & 1) * 8 + r) * row_bytes + (j >> 1) * 16);
#pragma unroll
  for (int dt = 0; dt < D_TILES; dt += 2) {
    if (dt * 8 < head_dim) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, v_base + dt * 16);
      if (rescale) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          st.o[dt][e] *= corr[e >> 1];
          st.o[dt + 1][e] *= corr[e >> 1];
        }
      }
      mma_16816(st.o[dt], pf, vf[0], vf[1]);
      mma_16816(st.o[dt + 1], pf, vf[2], vf[3]);
    }
  }
}

// One warp: scores of its 16 query rows against KEY_TILES * 8 keys that start at row `key_row` of
// the key tile, one online-softmax update for all of them (one rescale of the output accumulators
// a call, which is what makes long steps cheap), and the product with the same rows of the value
// tile.  `masked` (uniform over the warp) says whether any key of the range may be hidden from a
// row; without it the comparisons are skipped.
template <int D_TILES, int KEY_TILES>
__device__ __forceinline__ void attend_keys(SoftmaxState<D_TILES>& st, const uint32_t (*qf)[4],
                                            const unsigned char* ks_tile, const unsigned char* vs_tile, int key_row,
                                            int key_abs, const int (&key_lo)[2], const int (&key_hi)[2], bool masked,
                                            int head_dim, float scale_log2) {
  static_assert(KEY_TILES % 2 == 0, "keys come in groups of 16");
  const int lane = threadIdx.x & 31, t = lane & 3;
  const int row_bytes = tile_row_bytes(head_dim);
  const int j = lane >> 3, r = lane & 7;
  float s[KEY_TILES][4];
#pragma unroll
  for (int nt = 0; nt < KEY_TILES; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
  const uint32_t k_base = smem_addr(ks_tile + (key_row + (j >> 1) * 8 + r) * row_bytes + (j & 1) * 16);
#pragma unroll
  for (int ks = 0; ks < D_TILES / 2; ++ks) {
    if (ks * 16 < head_dim) {
#pragma unroll
      for (int kp = 0; kp < KEY_TILES / 2; ++kp) {
        uint32_t kf[4];
        ldmatrix_x4(kf, k_base + kp * 16 * row_bytes + ks * 32);
        mma_16816(s[2 * kp], qf[ks], kf[0], kf[1]);
        mma_16816(s[2 * kp + 1], qf[ks], kf[2], kf[3]);
      }
    }
  }
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < KEY_TILES; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = e >> 1;
      bool live = true;
      if (masked) {
        const int key = key_abs + nt * 8 + 2 * t + (e & 1);
        live = key >= key_lo[row] && key < key_hi[row];
      }
      s[nt][e] = live ? s[nt][e] * scale_log2 : -INFINITY;
      tile_max[row] = fmaxf(tile_max[row], s[nt][e]);
    }
  float corr[2];
#pragma unroll
  for (int row = 0; row < 2; ++row) {
    tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 1));
    tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 2));
    const float m_new = fmaxf(st.m[row], tile_max[row]);
    corr[row] = m_new == -INFINITY ? 1.f : exp2f(st.m[row] - m_new);
    st.m[row] = m_new;
    st.l[row] *= corr[row];
  }
#pragma unroll
  for (int nt = 0; nt < KEY_TILES; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = e >> 1;
      s[nt][e] = st.m[row] == -INFINITY ? 0.f : exp2f(s[nt][e] - st.m[row]);
      st.l[row] += s[nt][e];
    }
  if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {  // not once the maxima have settled
#pragma unroll
    for (int dt = 0; dt < D_TILES; ++dt)
#pragma unroll
      for (int e = 0; e < 4; ++e) st.o[dt][e] *= corr[e >> 1];
  }
  const uint32_t v_base = smem_addr(vs_tile + (key_row + (j & 1) * 8 + r) * row_bytes + (j >> 1) * 16);
#pragma unroll
  for (int kp = 0; kp < KEY_TILES / 2; ++kp) {
    uint32_t pf[4];
    pf[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
    pf[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
    pf[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
    pf[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
#pragma unroll
    for (int dt = 0; dt < D_TILES; dt += 2) {
      if (dt * 8 < head_dim) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, v_base + kp * 16 * row_bytes + dt * 16);
        mma_16816(st.o[dt], pf, vf[0], vf[1]);
        mma_16816(st.o[dt + 1], pf, vf[2], vf[3]);
      }
    }
  }
}

// ---- the same update with the roles swapped (decode) ------------------------------------------------
// One new token a sequence has only its group's query heads as rows: 4 or 8 of the MMA's 16.  With
// the KEYS as the MMA's 16 rows and the heads as its 8 columns nothing but columns beyond the group
// is padding, the scores of 16 keys cost half the MMAs, and a thread holds 4 scores instead of 8:
//   S^T[key][head] = sum_d K[key][d] Q[head][d]      A = K rows (ldmatrix), B = Q from registers
//   O^T[dim][head] += sum_key V[key][dim] P[key][head]   A = V^T (ldmatrix.trans), B = P, brought from
//                                                     the accumulator layout by two 8x8 transposes
// Lane (g, t) holds heads 2t and 2t + 1: their running maxima (equal in all lanes of a t), its share
// of their sums, and for every 16 dims the outputs (dim g, dim g + 8) x (head 2t, head 2t + 1).

constexpr float DEC_REFERENCE_SLACK = 8.f;  // how far (base 2) a score may outgrow the reference of a head's exponents

__device__ __forceinline__ float fast_exp2(float x) {  // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t transpose_8x8(uint32_t fragment) {
  uint32_t out;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(out) : "r"(fragment));
  return out;
}

template <int D_TILES>
struct HeadColumnState {
  float m[2];
  float l[2];
  float o[D_TILES / 2][4];
  __device__ __forceinline__ void init() {
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
#pragma unroll
    for (int i = 0; i < D_TILES / 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  }
};

// qb[ks] = the two 32-bit words Q[head g][ks * 16 + 2t ..] and Q[head g][ks * 16 + 8 + 2t ..]
// (zero for g at or beyond the group).  Keys outside [key_lo, key_hi) are masked.
// SWIZZLED: the tiles were written by TMA with the 128-byte swizzle: boxes of 64 rows x 64 dims
// (8 KB each, the boxes of a tile one after another), the 16-byte piece c of row r stored at piece
// c ^ (r % 8).  Such a tile holds the whole cache block, also rows beyond the sequence, which may be
// anything: masked keys' values are cleared in the registers (0 x NaN would poison the sum).
// `values_ready` is called once the weights are known and before the values' tile is read: a kernel whose
// values land on a barrier of their own waits there; false (a bounded wait ran out) leaves the output as it was.
template <int D_TILES, bool SWIZZLED = false, class ValuesReady>
__device__ __forceinline__ bool attend_16_keys_heads(HeadColumnState<D_TILES>& st, const uint32_t (*qb)[2],
                                                     const unsigned char* ks_tile, const unsigned char* vs_tile,
                                                     int key_row, int key_abs, int key_lo, int key_hi, bool masked,
                                                     int head_dim, float scale_log2, ValuesReady&& values_ready) {
  const int lane = threadIdx.x & 31, g = lane >> 2;
  const int row_bytes = tile_row_bytes(head_dim);
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // two chains of dependent MMAs
  // K as the A operand: matrix j of an x4 load = keys (j % 2) * 8 .., dims ks * 16 + (j / 2) * 8 ..
  const uint32_t k_base = SWIZZLED ? smem_addr(ks_tile + (key_row + (lane & 15)) * 128)
                                   : smem_addr(ks_tile + (key_row + (lane & 15)) * row_bytes + (lane >> 4) * 16);
  const uint32_t k_piece = (uint32_t)((lane >> 4) ^ (lane & 7));  // this lane's piece of a step, before the step's own bits
  // The loads of LOADS_AHEAD steps are asked for before the first of their products: the instructions run in the
  // order they are written, and a product straight after its own load waited out that load's latency every step.
  constexpr int LOADS_AHEAD = D_TILES / 2 < 8 ? D_TILES / 2 : 8;
#pragma unroll
  for (int ks0 = 0; ks0 < D_TILES / 2; ks0 += LOADS_AHEAD) {
    uint32_t kf[LOADS_AHEAD][4];
#pragma unroll
    for (int j = 0; j < LOADS_AHEAD; ++j) {
      const int ks = ks0 + j;
      if (ks * 16 < head_dim) {
        if (SWIZZLED) ldmatrix_x4(kf[j], k_base + (ks >> 2) * 8192 + ((k_piece ^ ((2 * ks) & 7)) << 4));
        else ldmatrix_x4(kf[j], k_base + ks * 32);
      }
    }
#pragma unroll
    for (int j = 0; j < LOADS_AHEAD; ++j) {
      const int ks = ks0 + j;
      if (ks * 16 < head_dim) mma_16816(s[ks & 1], kf[j], qb[ks][0], qb[ks][1]);
    }
  }
  // c0, c1: key g x heads 2t, 2t+1; c2, c3: key g + 8
  float v[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    bool live = true;
    if (masked) {  // uniform over the warp: only the 16 keys at an edge of the range pay for the comparisons
      const int key = key_abs + g + (e >> 1) * 8;
      live = key >= key_lo && key < key_hi;
    }
    v[e] = live ? (s[0][e] + s[1][e]) * scale_log2 : -INFINITY;
  }
  // st.m is the reference value of a head's exponents, not its running maximum: it moves only when a score has
  // outgrown it by more than 8 in base 2 (weights then reach 2^8 at most, far inside bfloat16 and the 32-bit
  // sums), so most tiles need neither the maximum over the keys (three shuffles a head, one after the other)
  // nor a rescaled output.  The vote is uniform over the warp.
  float corr[2] = {1.f, 1.f};
  const bool rescale = __any_sync(0xffffffffu, fmaxf(v[0], v[2]) - st.m[0] > DEC_REFERENCE_SLACK ||
                                                   fmaxf(v[1], v[3]) - st.m[1] > DEC_REFERENCE_SLACK);
  if (rescale) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tile_max = fmaxf(v[h], v[h + 2]);
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
      const float m_new = fmaxf(st.m[h], tile_max);
      // a head with no live key so far keeps m = -inf; 2^(-inf - -inf) must not be NaN
      corr[h] = m_new == -INFINITY ? 1.f : fast_exp2(st.m[h] - m_new);
      st.m[h] = m_new;
      st.l[h] *= corr[h];
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float base = st.m[h] == -INFINITY ? 0.f : st.m[h];  // then every score is -inf and every weight 0
    v[h] = fast_exp2(v[h] - base);
    v[h + 2] = fast_exp2(v[h + 2] - base);
    st.l[h] += v[h] + v[h + 2];
  }
  const uint32_t p_lo = transpose_8x8(pack_bf16(v[0], v[1]));  // keys 2t, 2t+1 of head g
  const uint32_t p_hi = transpose_8x8(pack_bf16(v[2], v[3]));  // keys 2t+8, 2t+9
  if (!values_ready()) return false;
  // V^T as the A operand (transposed load): matrix j = keys (j / 2) * 8 .., dims dt * 16 + (j % 2) * 8 ..
  const int j = lane >> 3, r = lane & 7;
  const uint32_t v_base = SWIZZLED ? smem_addr(vs_tile + (key_row + (j >> 1) * 8 + r) * 128)
                                   : smem_addr(vs_tile + (key_row + (j >> 1) * 8 + r) * row_bytes + (j & 1) * 16);
  const uint32_t v_piece = (uint32_t)((j & 1) ^ r);
  uint32_t keep_lo = 0xffffffffu, keep_hi = 0xffffffffu;  // values of keys 2t, 2t+1 and of keys 2t+8, 2t+9
  if (SWIZZLED && masked) {
    const int t = lane & 3;
    auto live = [&](int key) { return key >= key_lo && key < key_hi; };
    keep_lo = (live(key_abs + 2 * t) ? 0x0000ffffu : 0u) | (live(key_abs + 2 * t + 1) ? 0xffff0000u : 0u);
    keep_hi = (live(key_abs + 2 * t + 8) ? 0x0000ffffu : 0u) | (live(key_abs + 2 * t + 9) ? 0xffff0000u : 0u);
  }
#pragma unroll
  for (int dt0 = 0; dt0 < D_TILES / 2; dt0 += LOADS_AHEAD) {
    uint32_t vf[LOADS_AHEAD][4];
#pragma unroll
    for (int j = 0; j < LOADS_AHEAD; ++j) {
      const int dt = dt0 + j;
      if (dt * 16 < head_dim) {
        if (SWIZZLED) ldmatrix_x4_trans(vf[j], v_base + (dt >> 2) * 8192 + ((v_piece ^ ((2 * dt) & 7)) << 4));
        else ldmatrix_x4_trans(vf[j], v_base + dt * 32);
      }
    }
#pragma unroll
    for (int j = 0; j < LOADS_AHEAD; ++j) {
      const int dt = dt0 + j;
      if (dt * 16 < head_dim) {
        if (SWIZZLED && masked) { vf[j][0] &= keep_lo; vf[j][1] &= keep_lo; vf[j][2] &= keep_hi; vf[j][3] &= keep_hi; }
        if (rescale) {
          st.o[dt][0] *= corr[0];
          st.o[dt][1] *= corr[1];
          st.o[dt][2] *= corr[0];
          st.o[dt][3] *= corr[1];
        }
        mma_16816(st.o[dt], vf[j], p_lo, p_hi);
      }
    }
  }
  return true;
}

template <int D_TILES, bool SWIZZLED = false>
__device__ __forceinline__ void attend_16_keys_heads(HeadColumnState<D_TILES>& st, const uint32_t (*qb)[2],
                                                     const unsigned char* ks_tile, const unsigned char* vs_tile,
                                                     int key_row, int key_abs, int key_lo, int key_hi, bool masked,
                                                     int head_dim, float scale_log2) {
  attend_16_keys_heads<D_TILES, SWIZZLED>(st, qb, ks_tile, vs_tile, key_row, key_abs, key_lo, key_hi, masked, head_dim,
                                          scale_log2, [] { return true; });
}

}  // namespace xrt
