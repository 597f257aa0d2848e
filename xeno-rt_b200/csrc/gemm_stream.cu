// Y[M, N] = X[M, K] . W[N, K]^T for few rows (decode steps): the weight is streamed from HBM once
// through a ring of shared-memory stages filled by asynchronous copies (cp.async), and consumed by
// tensor-core MMAs (mma.sync m16n8k16, bfloat16 operands, 32-bit accumulation).
//
// The reference streams each weight row once per token through a row-parallel dot product
// (crates/xrt-kernels/src/cpu/matmul.rs:100-192; 194-320 for several tokens sharing one pass over
// the weight).  On this GPU the product's time is the time to read W, so the kernel is built around
// bytes in flight: a block of eight warps owns 8 weight rows (SwiGLU: 8 gate rows and the 8 matching
// up rows); for each 512-wide slab of K every thread issues 16-byte asynchronous copies (a warp
// covers 512 contiguous bytes of one row) into one of three stages, so two slabs are always in
// flight per block, and the small footprint (26 KB) lets eight blocks share a multiprocessor.
// Warp w then takes k in [64w, 64w + 64) of the slab: lane (g = lane / 4, t = lane % 4) reads the
// 16 bytes W[row g][k0 + 8t ..] from shared memory and the matching 16 bytes of up to two X rows
// from global memory (X is small and stays in L1/L2).  A dot product does not care in which order
// k is visited as long as both operands agree, so the four 32-bit words of such a load feed two
// MMAs as the fragment slots (2t, 2t+1), (2t+8, 2t+9) without any shuffle.  The batch rows are the
// MMA's M (16 a tile), the weight rows its N.  The warps' partial sums meet in shared memory and
// are added in warp order: a row's result does not depend on the number of rows M.
// Measured on a B200 with M = 8: 5.97 TB/s on the output matrix (1.05 GB), 5.2 TB/s on gate/up.
//
// A product that adds into the residual stream can also prepare the RMSNorm that follows it (NormEmit,
// common.cuh): here the parts of a row's sum of squares are one a block (its 8 or 16 weight rows); and
// the kernel can finish a norm that the product before prepared (RowScale).  Those products keep four
// stages.  Every 64 weight rows start their walk over K at another slab, and the weight is marked as
// streaming in the L2 by the launch's access-policy window (it is read once a step).
#include "common.cuh"

namespace xrt {

constexpr int GS_WARPS = 8;
constexpr int GS_THREADS = GS_WARPS * 32;
constexpr int GS_ROWS = 8;                      // weight rows of one group
constexpr int GS_SLAB = 512;                    // k elements a stage
constexpr int GS_ROW_BYTES = GS_SLAB * 2 + 64;  // padded: a quarter warp (two rows x four 16-byte pieces) hits 32 banks

__device__ __forceinline__ void gs_cp_async(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}

__device__ __forceinline__ void gs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: store, 1: add into float out, 2: SwiGLU (two groups of rows: gate and up)
template <int M_TILES, int MODE, int GS_STAGES, int ROW_GROUPS, typename TO>
__global__ void __launch_bounds__(GS_THREADS, (M_TILES >= 4 ? 2 : 1))
gemm_stream_kernel(TO* __restrict__ out, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   int M, int N, int K, int ldx, int ldo, long long up_offset, const NormEmit emit, const RowScale scale) {
  // ROW_GROUPS groups of 8 weight rows a block (SwiGLU: as many gate groups and as many up groups);
  // every X fragment a warp loads is used for all of them, which is what keeps the L1 traffic of
  // many batch rows below the shared-memory traffic of the weights
  constexpr int GROUPS = ROW_GROUPS * (MODE == 2 ? 2 : 1);
  constexpr int BLOCK_ROWS = ROW_GROUPS * GS_ROWS;
  constexpr int STAGE_ROWS = GROUPS * GS_ROWS;
  constexpr int STAGE_BYTES = STAGE_ROWS * GS_ROW_BYTES;
  constexpr int CHUNKS_PER_ROW = GS_SLAB / 8;                       // 16-byte pieces of a row's slab
  constexpr int COPIES = STAGE_ROWS * CHUNKS_PER_ROW / GS_THREADS;  // per thread and stage
  extern __shared__ __align__(128) unsigned char smem[];

  pdl_trigger();
  // the weight of the norm that follows never changes: this thread's element of it is on its way now
  float emit_w = 0.f;
  if (MODE == 1 && emit.scaled != nullptr) {
    const int wrow = min(blockIdx.x * (ROW_GROUPS * GS_ROWS) + (int)(threadIdx.x % (ROW_GROUPS * GS_ROWS)), N - 1);
    emit_w = emit.weight_dtype == XRT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(emit.weight)[wrow])
                                           : reinterpret_cast<const float*>(emit.weight)[wrow];
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * BLOCK_ROWS;
  const int n_slabs = (K + GS_SLAB - 1) / GS_SLAB;
  // Every block starts its walk over K at another slab and wraps around: blocks that all run at once
  // would else ask for the same columns of every weight row at the same time, addresses a whole row
  // apart, which a few memory channels serve (measured alone, 8 rows: N 5,120 / K 8,192 29.8 -> 23.8 us,
  // K 25,600 85.0 -> 71.8 us; N 4,096 / K 14,336 the same).  The start follows the weight row (by
  // 64 rows, which every block size divides), so a row's sum has the same order whatever the batch.
  const int first_slab = (int)(((unsigned)(row0 / 64) * 5u) % (unsigned)n_slabs);
  auto slab_of = [&](int turn) { const int at = turn + first_slab; return at >= n_slabs ? at - n_slabs : at; };

  // where this thread's copies come from and go to (the same for every slab, shifted by the slab)
  const __nv_bfloat16* copy_src[COPIES];
  uint32_t copy_dst[COPIES];
  int copy_k[COPIES];
#pragma unroll
  for (int i = 0; i < COPIES; ++i) {
    const int c = threadIdx.x + i * GS_THREADS, r = c / CHUNKS_PER_ROW, j = c % CHUNKS_PER_ROW;
    const int row = min(row0 + (r % BLOCK_ROWS), N - 1);  // clamped rows are read twice and never stored
    copy_src[i] = w + (size_t)row * K + (r >= BLOCK_ROWS ? up_offset : 0) + j * 8;
    copy_dst[i] = (uint32_t)__cvta_generic_to_shared(smem + r * GS_ROW_BYTES + j * 16);
    copy_k[i] = j * 8;
  }
  auto issue = [&](int s) {
    const int k0 = slab_of(s) * GS_SLAB;
    const uint32_t stage = (uint32_t)((s % GS_STAGES) * STAGE_BYTES);
#pragma unroll
    for (int i = 0; i < COPIES; ++i)  // K is a multiple of 8: a piece is wholly inside (16) or outside (zeros)
      gs_cp_async(copy_dst[i] + stage, copy_src[i] + k0, k0 + copy_k[i] < K ? 16 : 0);
  };
#pragma unroll
  for (int s = 0; s < GS_STAGES - 1; ++s) {
    if (s < n_slabs) issue(s);
    asm volatile("cp.async.commit_group;");
  }

  // The weights do not depend on the step: the first slabs are on their way while the kernel before
  // this one finishes.  X and the output do: wait for it here.
  pdl_wait();
  // x with a pending norm (the product before this one left residual * norm weight and the parts of every
  // row's sum of squares): warp w adds the parts of rows w, w + 8, ... in a fixed order; the factors
  // 1 / sqrt(mean square + eps) multiply the finished sums below
  __shared__ float row_inv[M_TILES * 16];
  __shared__ float inv_shares[GS_THREADS];
  if (MODE != 1 && scale.squares != nullptr) {
    if (GS_THREADS % M == 0) {
      // the parts lie [part][row]: thread t adds elements t, t + 256, ... (whole 128-byte lines a warp), all of
      // one row since 256 is a multiple of M; then the row's 256 / M shares are added in thread order
      const int total = scale.parts * M;
      float sum = 0.f;
#pragma unroll 4
      for (int e = threadIdx.x; e < total; e += GS_THREADS) sum += __ldcg(scale.squares + e);
      // lanes of a warp that meet the same row (every M-th) add up by a fixed tree, then the warps in order
      for (int o = 16; o >= M; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      inv_shares[threadIdx.x] = sum;
      __syncthreads();
      if (threadIdx.x < M) {
        const int step = M > 32 ? M : 32;
        float row = 0.f;
        for (int j = threadIdx.x; j < GS_THREADS; j += step) row += inv_shares[j];
        row_inv[threadIdx.x] = rsqrtf(row / (float)scale.width + scale.eps);
      }
    } else {
      for (int m = warp; m < M; m += GS_WARPS) {
        float sum = 0.f;
        for (int p = lane; p < scale.parts; p += 32) sum += __ldcg(scale.squares + (size_t)p * M + m);
        sum = warp_sum(sum);
        if (lane == 0) row_inv[m] = rsqrtf(sum / (float)scale.width + scale.eps);
      }
    }
  }
  const __nv_bfloat16* xlo[M_TILES];
  const __nv_bfloat16* xhi[M_TILES];
#pragma unroll
  for (int mt = 0; mt < M_TILES; ++mt) {  // rows at or beyond M are clamped: computed and never stored
    xlo[mt] = x + (size_t)min(mt * 16 + g, M - 1) * ldx;
    xhi[mt] = x + (size_t)min(mt * 16 + g + 8, M - 1) * ldx;
  }
  float acc[GROUPS][M_TILES][4];
#pragma unroll
  for (int gr = 0; gr < GROUPS; ++gr)
#pragma unroll
    for (int mt = 0; mt < M_TILES; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[gr][mt][i] = 0.f;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  constexpr bool EARLY_X = M_TILES < 4;  // few batch rows: X of a slab is loaded before the wait and hides under it;
  //                                        many: one half slab at a time, to keep the registers for accumulators
  for (int s = 0; s < n_slabs; ++s) {
    uint4 xa[2][M_TILES], xb[2][M_TILES];
    auto load_x = [&](int h) {
      const int k = slab_of(s) * GS_SLAB + warp * 64 + h * 32 + t * 8;
      const bool inside = k < K;  // differs between lanes; only loads are conditional, every lane runs the MMAs
#pragma unroll
      for (int mt = 0; mt < M_TILES; ++mt) {
        xa[h][mt] = inside ? *reinterpret_cast<const uint4*>(xlo[mt] + k) : zero;
        xb[h][mt] = inside ? *reinterpret_cast<const uint4*>(xhi[mt] + k) : zero;
      }
    };
    if (EARLY_X) { load_x(0); load_x(1); }
    asm volatile("cp.async.wait_group %0;" ::"n"(GS_STAGES - 2));
    __syncthreads();  // slab s has landed for every thread, and every warp is done with slab s - 1
    if (s + GS_STAGES - 1 < n_slabs) issue(s + GS_STAGES - 1);  // into the stage that slab s - 1 used
    asm volatile("cp.async.commit_group;");
    const unsigned char* base = smem + (s % GS_STAGES) * STAGE_BYTES;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!EARLY_X) load_x(h);
      const int kk = warp * 64 + h * 32 + t * 8;
#pragma unroll
      for (int gr = 0; gr < GROUPS; ++gr) {
        const uint4 wv = *reinterpret_cast<const uint4*>(base + (gr * GS_ROWS + g) * GS_ROW_BYTES + kk * 2);
#pragma unroll
        for (int mt = 0; mt < M_TILES; ++mt) {
          gs_mma(acc[gr][mt], xa[h][mt].x, xb[h][mt].x, xa[h][mt].y, xb[h][mt].y, wv.x, wv.y);
          gs_mma(acc[gr][mt], xa[h][mt].z, xb[h][mt].z, xa[h][mt].w, xb[h][mt].w, wv.z, wv.w);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;");
  __syncthreads();  // the ring is free for the partial sums

  // partial[warp][group][m tile][16 rows][8 + 1]; c0, c1: (m = g, n = 2t, 2t+1); c2, c3: (m = g + 8, same n)
  constexpr int P_ROW = GS_ROWS + 1;
  float* partial = reinterpret_cast<float*>(smem);
#pragma unroll
  for (int gr = 0; gr < GROUPS; ++gr)
#pragma unroll
    for (int mt = 0; mt < M_TILES; ++mt) {
      float* p = partial + (((size_t)warp * GROUPS + gr) * M_TILES + mt) * 16 * P_ROW;
      p[g * P_ROW + 2 * t] = acc[gr][mt][0];
      p[g * P_ROW + 2 * t + 1] = acc[gr][mt][1];
      p[(g + 8) * P_ROW + 2 * t] = acc[gr][mt][2];
      p[(g + 8) * P_ROW + 2 * t + 1] = acc[gr][mt][3];
    }
  __syncthreads();
  for (int e = threadIdx.x; e < M_TILES * 16 * BLOCK_ROWS; e += blockDim.x) {  // the same trips for a whole warp
    const int nb = e % BLOCK_ROWS, m = e / BLOCK_ROWS;
    const int rg = nb / GS_ROWS, n = nb % GS_ROWS;
    const int mt = m / 16, mr = m % 16;
    const int row = row0 + nb;
    const bool live = m < M && row < N;
    auto total = [&](int gr) {
      float sum = 0.f;
#pragma unroll
      for (int ww = 0; ww < GS_WARPS; ++ww)
        sum += partial[((((size_t)ww * GROUPS + gr) * M_TILES + mt) * 16 + mr) * P_ROW + n];
      return sum;
    };
    float square = 0.f;
    if (live) {
      const float inv = (MODE != 1 && scale.squares != nullptr) ? row_inv[m] : 1.f;
      const float first = total(rg) * inv;
      TO* dst = out + (size_t)m * ldo + row;
      if (MODE == 2) *dst = from_float<TO>((first / (1.0f + expf(-first))) * (total(ROW_GROUPS + rg) * inv));
      else if (MODE == 1) {
        const float updated = to_float(*dst) + first;
        *dst = from_float<TO>(updated);
        if (emit.scaled != nullptr) {
          emit.scaled[(size_t)m * emit.ld + row] = __float2bfloat16_rn(updated * emit_w);  // e % BLOCK_ROWS == threadIdx.x % BLOCK_ROWS
          square = updated * updated;
        }
      } else *dst = from_float<TO>(first);
    }
    if (MODE == 1 && emit.squares != nullptr) {
      // the block's rows of one batch row sit in BLOCK_ROWS neighbouring lanes: summed in a fixed order
#pragma unroll
      for (int o = 1; o < BLOCK_ROWS; o <<= 1) square += __shfl_xor_sync(0xffffffffu, square, o);
      if (nb == 0 && m < M) emit.squares[(size_t)blockIdx.x * M + m] = square;
    }
  }
}

template <int M_TILES, int MODE, int GS_STAGES, int ROW_GROUPS, typename TO>
int launch_stream_staged(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                         long long up_offset, const NormEmit& emit, const RowScale& scale, cudaStream_t stream) {
  constexpr int GROUPS = ROW_GROUPS * (MODE == 2 ? 2 : 1);
  constexpr int RING_BYTES = GS_STAGES * GROUPS * GS_ROWS * GS_ROW_BYTES;
  constexpr int PARTIAL_BYTES = GS_WARPS * GROUPS * M_TILES * 16 * (GS_ROWS + 1) * (int)sizeof(float);
  constexpr int SMEM = RING_BYTES > PARTIAL_BYTES ? RING_BYTES : PARTIAL_BYTES;
  auto kernel = gemm_stream_kernel<M_TILES, MODE, GS_STAGES, ROW_GROUPS, TO>;
  static bool allowed = false;
  if (SMEM > 48 * 1024 && !allowed) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return (int)err;
    allowed = true;
  }
  const int blocks = (N + ROW_GROUPS * GS_ROWS - 1) / (ROW_GROUPS * GS_ROWS);
  // the weight is read once a step (cp.async carries no cache hint here): marked as streaming in the L2
  const size_t weight_bytes = ((size_t)(MODE == 2 ? up_offset / K : 0) + (size_t)N) * (size_t)K * sizeof(__nv_bfloat16);
  launch_kernel_streaming(kernel, dim3(blocks), dim3(GS_THREADS), SMEM, stream, w, weight_bytes, (TO*)out,
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, M, N, K, ldx, ldo, up_offset, emit, scale);
  return launch_status();
}

// Three stages: 26 KB a block; registers allow four blocks a multiprocessor.  Rings of 4, 5 and 6
// stages were measured: they help single shapes (the output matrix at one row reaches 6.7 TB/s with
// 5) and lose on others; over a whole decode step of 8 sequences 3 stages is the fastest, except for the
// products that add into the residual stream, where 4 stages with the rotated walk are (alone, 8 rows:
// K 4,096 9.2 -> 8.6 us, K 14,336 26.6 -> 26.1, N 5,120 / K 25,600 85.0 -> 68.4; whole steps 1 % faster).
// Multiprocessors of the current device (148 where there is none to ask: host arithmetic only).
inline int stream_sm_count() {
  static const int count = [] {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0)
      value = 148;
    cudaGetLastError();
    return value;
  }();
  return count;
}

// Groups of 8 weight rows a block for a product of up to 16 rows that adds into the residual stream: one,
// unless its blocks would then not all run at once (four a multiprocessor) and blocks of two groups would
// (three a multiprocessor with their four stages).  640 blocks on 592 places are two rounds, the second
// nearly empty; measured alone at 8 rows, N 5,120: K 8,192 23.4 -> 16.6 us, K 25,600 68.9 -> 48.4 us
// (N 4,096, whose 512 blocks fit, loses with two groups: 26.2 -> 27.1 us at K 14,336).
inline int stream_row_groups_accumulate(int N) {
  const int sms = stream_sm_count();
  if ((N + GS_ROWS - 1) / GS_ROWS <= sms * 4) return 1;
  return (N + 2 * GS_ROWS - 1) / (2 * GS_ROWS) <= sms * 3 ? 2 : 1;
}

template <int M_TILES, int MODE, typename TO>
int launch_stream(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo, long long up_offset,
                  const NormEmit& emit, const RowScale& scale, cudaStream_t stream) {
  // more than 32 batch rows: two row groups a block halve the X traffic per weight byte
  constexpr int RG = M_TILES >= 4 ? 2 : 1;
  // products that add into the residual stream (long K, few blocks a multiprocessor): four stages
  if (MODE == 1 && M_TILES == 1) {
    if (stream_row_groups_accumulate(N) == 2)
      return launch_stream_staged<M_TILES, MODE, 4, 2, TO>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
    return launch_stream_staged<M_TILES, MODE, 4, RG, TO>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
  }
  // a product of up to 16 rows whose blocks of 8 weight rows would not all run at once: 16 rows a block
  // (alone at 8 rows, N 6,144 / K 4,096: 12.9 -> 8.9 us; N 10,240 / K 5,120: 23.0 -> 20.9; N 8,192 / K 8,192:
  // 31.2 -> 28.1; three groups the same, four groups with two stages slower but for the last)
  if (MODE == 0 && M_TILES == 1 && (N + GS_ROWS - 1) / GS_ROWS > stream_sm_count() * 4)
    return launch_stream_staged<M_TILES, MODE, 3, 2, TO>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
  return launch_stream_staged<M_TILES, MODE, 3, RG, TO>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
}

template <int M_TILES>
int dispatch_stream(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo, int out_dtype,
                    int mode, long long up_offset, const NormEmit& emit, const RowScale& scale, cudaStream_t stream) {
  if (mode == 1) return launch_stream<M_TILES, 1, float>(out, x, w, M, N, K, ldx, ldo, 0, emit, scale, stream);
  if (mode == 2) {
    if (out_dtype == XRT_BF16)
      return launch_stream<M_TILES, 2, __nv_bfloat16>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
    return launch_stream<M_TILES, 2, float>(out, x, w, M, N, K, ldx, ldo, up_offset, emit, scale, stream);
  }
  if (out_dtype == XRT_BF16)
    return launch_stream<M_TILES, 0, __nv_bfloat16>(out, x, w, M, N, K, ldx, ldo, 0, emit, scale, stream);
  return launch_stream<M_TILES, 0, float>(out, x, w, M, N, K, ldx, ldo, 0, emit, scale, stream);
}

}  // namespace xrt

// How many floats a batch row `squares` holds one of: the blocks of the launch (M at most 16).
XRT_EXPORT int xrt_gemm_stream_norm_blocks(int M, int N) {
  if (M <= 0 || N <= 0 || M > 16) return XRT_ERR_UNSUPPORTED;
  const int rows = xrt::GS_ROWS * xrt::stream_row_groups_accumulate(N);
  return (N + rows - 1) / rows;
}

// x: bfloat16 [M, K] with row stride ldx (a multiple of 8); w: bfloat16 [N, K] contiguous, K a
// multiple of 8; out: [M, N] with row stride ldo.  mode 0 stores, 1 adds into a float32 out, 2 computes
// silu(x . W[n]) * (x . W[n + up_rows]) for n < N.  M is at most 64.
// With mode 1 and `scaled` not null the product also prepares the norm that follows it (see
// the file's head): scaled = bfloat16 [M, ld_scaled] receives (new residual) * norm_weight ([N], in
// norm_dtype), squares = float32 [xrt_gemm_stream_norm_blocks(M, N), M] the blocks' sums of squares.
// Only for M <= 16 (one group of weight rows a block).
// in_squares not null (modes 0 and 2): x is the result of such a product, residual * norm weight, and
// in_squares = float32 [in_parts, M] the parts of its rows' sums of squares: every row of the result is
// multiplied by 1 / sqrt(sum of the row's parts / K + eps).
XRT_EXPORT int xrt_gemm_stream_normed(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                      int out_dtype, int mode, int up_rows, void* scaled, int ld_scaled,
                                      const void* norm_weight, int norm_dtype, float* squares, const float* in_squares,
                                      int in_parts, float eps, cudaStream_t stream) {
  if (in_squares != nullptr && (in_parts <= 0 || mode == 1)) return XRT_ERR_ARGUMENT;
  xrt::RowScale scale;
  scale.squares = in_squares; scale.parts = in_parts; scale.width = K; scale.eps = eps;
  if (M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || mode < 0 || mode > 2) return XRT_ERR_ARGUMENT;
  if (mode == 1 && out_dtype != XRT_F32) return XRT_ERR_ARGUMENT;
  if (out_dtype != XRT_F32 && out_dtype != XRT_BF16) return XRT_ERR_UNSUPPORTED;
  if (K % 8 != 0 || ldx % 8 != 0 || M > 64) return XRT_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return XRT_ERR_UNSUPPORTED;
  xrt::NormEmit emit;
  if (scaled != nullptr) {
    if (mode != 1 || norm_weight == nullptr || squares == nullptr || ld_scaled < N) return XRT_ERR_ARGUMENT;
    if (M > 16 || (norm_dtype != XRT_F32 && norm_dtype != XRT_BF16)) return XRT_ERR_UNSUPPORTED;
    emit.scaled = (__nv_bfloat16*)scaled; emit.weight = norm_weight; emit.squares = squares;
    emit.ld = ld_scaled; emit.weight_dtype = norm_dtype;
  }
  if (M == 0) return XRT_OK;
  const long long up_offset = (long long)up_rows * K;
  if (M <= 16) return xrt::dispatch_stream<1>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, emit, scale, stream);
  if (M <= 32) return xrt::dispatch_stream<2>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, emit, scale, stream);
  return xrt::dispatch_stream<4>(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_offset, emit, scale, stream);
}

// The same with an x that is what it is.
XRT_EXPORT int xrt_gemm_stream_norm(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                                    int out_dtype, int mode, int up_rows, void* scaled, int ld_scaled,
                                    const void* norm_weight, int norm_dtype, float* squares, cudaStream_t stream) {
  return xrt_gemm_stream_normed(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_rows, scaled, ld_scaled, norm_weight,
                                norm_dtype, squares, nullptr, 0, 0.f, stream);
}

// The same without a norm to prepare.
XRT_EXPORT int xrt_gemm_stream(void* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldo,
                               int out_dtype, int mode, int up_rows, cudaStream_t stream) {
  return xrt_gemm_stream_norm(out, x, w, M, N, K, ldx, ldo, out_dtype, mode, up_rows, nullptr, 0, nullptr, XRT_F32, nullptr,
                              stream);
}
