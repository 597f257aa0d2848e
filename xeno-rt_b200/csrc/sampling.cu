// Sampling on the device, one thread block per row of 32-bit logits.
//
// What the reference's sampler computes (crates/xrt-runtime/src/sampler.rs):
//   repetition penalty p > 1 on every id seen in the history: l > 0 ? l / p : l * p      :77-91, 110-125
//   temperature <= 1e-5: argmax, the first maximum wins                                    :63, 83-98
//   else: keep the top_k largest adjusted logits (0 = all)                                 :107-145
//         probabilities exp((l - max) / T), normalised                                     :148-164
//         keep the shortest prefix, by falling probability, whose sum reaches top_p        :166-183
//         draw r in [0, 1) and walk the cumulative sum                                     :186-195
// The reference sorts the candidates; here nothing is sorted.  A radix select over order-preserving
// keys finds the top_k threshold (by count) and the top_p threshold (by probability mass), equal
// values at a threshold are kept in index order (the reference's heap also keeps the earlier of
// equal values), and the draw walks the kept set in index order.  The kept set and its
// probabilities are those of the reference; which id a given r lands on is this library's own
// convention, as is the generator: u = top 32 bits of
// splitmix64(key[slot] + (counter[slot] + 1) * 0x9E3779B97F4A7C15), counter[slot] += 1 a draw.
// Probability mass is summed as 64-bit integers (probability * 2^32), so sums do not depend on
// the order in which threads add and a seed gives the same tokens on every run.
#include "common.cuh"

namespace xrt {

constexpr int SAMPLE_THREADS = 1024;
constexpr int HIST_COPIES = SAMPLE_THREADS / 64;  // private histograms of the radix select

__device__ __forceinline__ uint64_t sm64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// larger float <=> larger key; NaN sorts lowest
__device__ __forceinline__ uint32_t order_key(float v) {
  if (v != v) return 0u;
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct RowView {
  const float* logits;
  const uint32_t* seen;  // bitmap of ids in the history, or null
  float penalty;
  __device__ __forceinline__ float adjusted(int i) const {
    float l = logits[i];
    if (seen != nullptr && ((seen[i >> 5] >> (i & 31)) & 1u)) l = l > 0.f ? l / penalty : l * penalty;
    return l;
  }
};

__device__ __forceinline__ uint64_t shfl_up64(uint64_t v, int delta) {
  const uint32_t lo = __shfl_up_sync(0xffffffffu, (uint32_t)v, delta);
  const uint32_t hi = __shfl_up_sync(0xffffffffu, (uint32_t)(v >> 32), delta);
  return ((uint64_t)hi << 32) | lo;
}

// Exclusive prefix sum of one value a thread over the block, in thread order; *total gets the sum.
__device__ uint64_t block_exclusive_scan(uint64_t v, uint64_t* warp_totals, uint64_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint64_t up = shfl_up64(inc, d);
    if (lane >= d) inc += up;
  }
  __syncthreads();
  if (lane == 31) warp_totals[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint64_t w = lane < (blockDim.x >> 5) ? warp_totals[lane] : 0;
    uint64_t winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint64_t up = shfl_up64(winc, d);
      if (lane >= d) winc += up;
    }
    warp_totals[lane] = winc - w;          // exclusive offsets of the warps
    if (lane == 31) warp_totals[32] = winc;  // grand total
  }
  __syncthreads();
  *total = warp_totals[32];
  return warp_totals[warp] + inc - v;
}

// The first index, in index order, at which the running sum of weight(i) exceeds `target`;
// -1 if the whole sum does not.  Each thread owns a contiguous segment of indices.
template <typename F>
__device__ int ordered_pick(F weight, int n, uint64_t target, uint64_t* scan_scratch, int* result) {
  const int seg = (n + blockDim.x - 1) / blockDim.x;
  const int lo = min(n, (int)threadIdx.x * seg), hi = min(n, lo + seg);
  uint64_t local = 0;
#pragma unroll 4
  for (int i = lo; i < hi; ++i) local += weight(i);
  if (threadIdx.x == 0) *result = -1;
  uint64_t total;
  const uint64_t before = block_exclusive_scan(local, scan_scratch, &total);
  if (before <= target && target < before + local) {
    uint64_t c = before;
    for (int i = lo; i < hi; ++i) {
      c += weight(i);
      if (c > target) { *result = i; break; }
    }
  }
  __syncthreads();
  const int found = *result;
  __syncthreads();  // the next call resets *result
  return found;
}

// Radix select from the top: the largest key K such that the weight of {key >= K} reaches `want`.
// Returns the key; *inside gets want minus the weight of {key > K} (what the keys equal to K still
// have to supply, >= 1 if want >= 1) and *at_key the weight of {key == K}.  If the whole weight is
// below `want`, returns 0 with *inside = 0.
template <typename A, typename F>
__device__ uint32_t radix_select(A adjusted, F weight, int n, uint64_t want, unsigned long long* hist,
                                 uint64_t* inside, uint64_t* at_key, uint32_t* shared_prefix) {
  uint32_t prefix = 0, mask = 0;
  uint64_t remaining = want;
  for (int pass = 3; pass >= 0; --pass) {
    const int shift = pass * 8;
    // HIST_COPIES private histograms (a pair of warps shares one): logits crowd into a few bins
    // of the leading byte, and a thousand threads adding to the same shared-memory word serialise
    unsigned long long* mine = hist + 258 + (threadIdx.x >> 6) * 256;
    for (int b = threadIdx.x; b < HIST_COPIES * 256; b += blockDim.x) hist[258 + b] = 0ull;
    __syncthreads();
    auto count = [&](int i, float a) {
      const uint32_t k = order_key(a);
      if ((k & mask) == prefix) {
        const uint64_t w = weight(i, a);
        if (w) atomicAdd(&mine[(k >> shift) & 255u], (unsigned long long)w);
      }
    };
    {
      // four loads in flight a thread; the histogram updates follow them
      int i = threadIdx.x;
      for (; i + 3 * (int)blockDim.x < n; i += 4 * blockDim.x) {
        float a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = adjusted(i + u * blockDim.x);
#pragma unroll
        for (int u = 0; u < 4; ++u) count(i + u * blockDim.x, a[u]);
      }
      for (; i < n; i += blockDim.x) count(i, adjusted(i));
    }
    __syncthreads();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
      unsigned long long sum = 0ull;
#pragma unroll
      for (int c = 0; c < HIST_COPIES; ++c) sum += hist[258 + c * 256 + b];
      hist[b] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint64_t above = 0;
      int bin = 255;
      for (; bin >= 0; --bin) {
        if (above + hist[bin] >= remaining) break;
        above += hist[bin];
      }
      if (bin < 0) {  // not enough weight in all: keep everything
        shared_prefix[0] = 0u; shared_prefix[1] = 1u;
        hist[256] = 0ull; hist[257] = 0ull;
      } else {
        shared_prefix[0] = prefix | ((uint32_t)bin << shift); shared_prefix[1] = 0u;
        hist[256] = remaining - above; hist[257] = hist[bin];
      }
    }
    __syncthreads();
    if (shared_prefix[1]) { *inside = 0; *at_key = 0; __syncthreads(); return 0u; }
    prefix = shared_prefix[0];
    mask |= 255u << shift;
    remaining = hist[256];
    *at_key = hist[257];
    __syncthreads();
  }
  *inside = remaining;
  return prefix;
}

constexpr int SAMPLE_CANDIDATES = 4096;                      // room for the candidates of a small top_k
constexpr int SAMPLE_DYNAMIC_BYTES = SAMPLE_CANDIDATES * 8;  // their ids and values; first the 4,096-bin histogram

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int* __restrict__ out_ids, const float* __restrict__ logits, int vocab,
              const int* __restrict__ row_slot, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ penalty, const uint32_t* __restrict__ seen, int seen_words,
              const unsigned long long* __restrict__ rng_key, unsigned int* __restrict__ rng_counter) {
  __shared__ unsigned long long hist[258 + HIST_COPIES * 256];  // merged bins, two result words, private copies
  __shared__ uint64_t scan_scratch[33];
  __shared__ float red_val[32];
  __shared__ int red_idx[32];
  __shared__ uint32_t shared_prefix[2];
  __shared__ int pick_result;
  __shared__ float bcast_max;
  __shared__ int bcast_arg;
  __shared__ int cut_bin, cut_count;
  extern __shared__ __align__(16) unsigned char dynamic[];
  int* cand_id = reinterpret_cast<int*>(dynamic);
  float* cand_val = reinterpret_cast<float*>(dynamic + SAMPLE_CANDIDATES * 4);
  unsigned int* fine_hist = reinterpret_cast<unsigned int*>(dynamic);  // 4,096 bins, before the candidates are written

  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int slot = row_slot[row];
  if (slot < 0) { if (threadIdx.x == 0) out_ids[row] = -1; return; }
  RowView view;
  view.logits = logits + (size_t)row * vocab;
  view.penalty = penalty[row];
  view.seen = (seen != nullptr && view.penalty > 1.0f) ? seen + (size_t)slot * seen_words : nullptr;
  const float temp = temperature[row];
  const int k = top_k[row];

  // A small top_k first gathers its candidates: one pass counts the adjusted logits into 4,096 bins
  // of the order key's top 12 bits, the bin that holds the k-th largest is found, and every element
  // of that bin or above (k plus what shares the bin) is copied to shared memory IN INDEX ORDER
  // (a thread owns a contiguous run of ids; its offset comes from a scan of the counts).  All later
  // steps run over these few candidates instead of the vocabulary: the kept set, its masses and the
  // draw are the same, since they only ever look at elements at or above the top_k threshold.
  int n = vocab;  // elements the later steps walk: the vocabulary, or the candidates
  bool compact = false;
  if (temp > 1e-5f && k > 0 && k < vocab) {
    for (int b = threadIdx.x; b < 4096; b += blockDim.x) fine_hist[b] = 0u;
    __syncthreads();
    {
      int i = threadIdx.x;
      for (; i + 7 * (int)blockDim.x < vocab; i += 8 * blockDim.x) {
        float a[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) a[u] = view.adjusted(i + u * blockDim.x);
#pragma unroll
        for (int u = 0; u < 8; ++u) atomicAdd(&fine_hist[order_key(a[u]) >> 20], 1u);
      }
      for (; i < vocab; i += blockDim.x) atomicAdd(&fine_hist[order_key(view.adjusted(i)) >> 20], 1u);
    }
    __syncthreads();
    {
      // thread t looks at bins 4095 - 4t .. 4092 - 4t (from the top); a scan tells how many lie above them
      uint64_t local = 0;
      if (threadIdx.x == 0) { cut_bin = 0; cut_count = vocab; }
#pragma unroll
      for (int j = 0; j < 4; ++j) local += fine_hist[4095 - 4 * (int)threadIdx.x - j];
      uint64_t total;
      const uint64_t before = block_exclusive_scan(local, scan_scratch, &total);
      if (before < (uint64_t)k && (uint64_t)k <= before + local) {
        uint64_t above = before;
        for (int j = 0; j < 4; ++j) {
          const int bin = 4095 - 4 * (int)threadIdx.x - j;
          above += fine_hist[bin];
          if (above >= (uint64_t)k) { cut_bin = bin; cut_count = (int)above; break; }
        }
      }
      __syncthreads();
    }
    if (cut_count <= SAMPLE_CANDIDATES) {
      const uint32_t cut = (uint32_t)cut_bin;
      const int total_kept = cut_count;
      const int seg = (vocab + blockDim.x - 1) / blockDim.x;
      const int lo = min(vocab, (int)threadIdx.x * seg), hi = min(vocab, lo + seg);
      uint64_t mine = 0;
      for (int i = lo; i < hi; ++i) mine += (order_key(view.adjusted(i)) >> 20) >= cut;
      uint64_t total;
      uint64_t at = block_exclusive_scan(mine, scan_scratch, &total);  // also: every thread is done with the histogram
      for (int i = lo; i < hi && mine > 0; ++i) {
        const float a = view.adjusted(i);
        if ((order_key(a) >> 20) >= cut) { cand_id[at] = i; cand_val[at] = a; ++at; }
      }
      __syncthreads();
      compact = true;
      n = total_kept;
    } else {
      __syncthreads();
    }
  }
  auto adjusted = [&](int j) { return compact ? cand_val[j] : view.adjusted(j); };
  auto id_of = [&](int j) { return compact ? cand_id[j] : j; };

  // maximum and its first index
  float best = -INFINITY; int best_i = 0x7fffffff;
  {
    // eight loads in flight a thread: a row is read once and the pass is bound by load latency
    constexpr int UNROLL = 8;
    int i = threadIdx.x;
    for (; i + (UNROLL - 1) * (int)blockDim.x < n; i += UNROLL * blockDim.x) {
      float a[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) a[u] = adjusted(i + u * blockDim.x);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (a[u] > best) { best = a[u]; best_i = i + u * blockDim.x; }  // indices rise: the first maximum is kept
    }
    for (; i < n; i += blockDim.x) {
      const float a = adjusted(i);
      if (a > best) { best = a; best_i = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { red_val[threadIdx.x >> 5] = best; red_idx[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = red_val[0]; int bi = red_idx[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (red_val[w] > b || (red_val[w] == b && red_idx[w] < bi)) { b = red_val[w]; bi = red_idx[w]; }
    bcast_max = b; bcast_arg = bi == 0x7fffffff ? 0 : bi;
  }
  __syncthreads();
  const float row_max = bcast_max;
  const int row_arg = id_of(bcast_arg);

  unsigned int counter = 0;
  if (threadIdx.x == 0) { counter = rng_counter[slot]; rng_counter[slot] = counter + 1; }
  if (temp <= 1e-5f) { if (threadIdx.x == 0) out_ids[row] = row_arg; return; }

  auto key_of = [&](int i) { return order_key(adjusted(i)); };
  // this thread's share of the sum of weight(i, adjusted(i)) over the elements, four loads in flight
  auto strided_sum = [&](auto weight) {
    uint64_t local = 0;
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < n; i += 4 * blockDim.x) {
      float a[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) a[u] = adjusted(i + u * blockDim.x);
#pragma unroll
      for (int u = 0; u < 4; ++u) local += weight(i + u * blockDim.x, a[u]);
    }
    for (; i < n; i += blockDim.x) local += weight(i, adjusted(i));
    return local;
  };

  // top-k: threshold key and the last index kept among equal keys
  uint32_t k_key = 0u; int k_last = n;  // kept: key > k_key, or key == k_key and i <= k_last
  if (k > 0 && k < n) {
    uint64_t inside, at_key;
    auto one = [&](int, float) { return (uint64_t)1; };
    k_key = radix_select(adjusted, one, n, (uint64_t)k, hist, &inside, &at_key, shared_prefix);
    if (at_key > inside) {
      auto tie = [&](int i) { return (uint64_t)(key_of(i) == k_key); };
      k_last = ordered_pick(tie, n, inside - 1, scan_scratch, &pick_result);
    }
  }
  const float inv_temp = 1.0f / temp;
  auto mass_of = [&](int i, float a) -> uint64_t {
    const uint32_t key = order_key(a);
    if (key < k_key || (key == k_key && i > k_last)) return 0ull;
    return (uint64_t)(expf((a - row_max) * inv_temp) * 4294967296.0f);
  };
  auto mass = [&](int i) -> uint64_t { return mass_of(i, adjusted(i)); };

  // top-p: threshold by probability mass
  uint32_t p_key = 0u; int p_last = n;
  const float p = top_p[row];
  if (p < 1.0f) {
    const uint64_t local = strided_sum(mass_of);
    uint64_t total;
    block_exclusive_scan(local, scan_scratch, &total);
    uint64_t want = (uint64_t)ceil((double)p * (double)total);
    if (want < 1) want = 1;
    uint64_t inside, at_key;
    p_key = radix_select(adjusted, mass_of, n, want, hist, &inside, &at_key, shared_prefix);
    if (at_key > inside) {
      // equal keys have equal mass: how many of them the remaining mass needs
      auto tie_mass = [&](int i) { return key_of(i) == p_key ? mass(i) : 0ull; };
      p_last = ordered_pick(tie_mass, n, inside - 1, scan_scratch, &pick_result);
    }
  }
  auto kept_mass_of = [&](int i, float a) -> uint64_t {
    const uint32_t key = order_key(a);
    if (key < p_key || (key == p_key && i > p_last)) return 0ull;
    return mass_of(i, a);
  };
  auto kept_mass = [&](int i) -> uint64_t { return kept_mass_of(i, adjusted(i)); };

  const uint64_t local = strided_sum(kept_mass_of);
  uint64_t total;
  block_exclusive_scan(local, scan_scratch, &total);
  __shared__ unsigned int shared_u;
  if (threadIdx.x == 0)
    shared_u = (unsigned int)(sm64(rng_key[slot] + ((uint64_t)counter + 1ull) * 0x9E3779B97F4A7C15ull) >> 32);
  __syncthreads();
  const uint64_t target = __umul64hi((uint64_t)shared_u << 32, total);  // floor(u / 2^32 * total)
  const int pick = total > 0 ? ordered_pick(kept_mass, n, target, scan_scratch, &pick_result) : -1;
  if (threadIdx.x == 0) out_ids[row] = pick >= 0 ? id_of(pick) : row_arg;
}

// Marks token ids as seen in their slot's bitmap (the history the repetition penalty looks at).
__global__ void mark_seen_kernel(uint32_t* __restrict__ seen, int seen_words, const int* __restrict__ slots,
                                 const int* __restrict__ ids, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int slot = slots[i], id = ids[i];
  if (slot < 0 || id < 0 || id >= vocab) return;
  atomicOr(&seen[(size_t)slot * seen_words + (id >> 5)], 1u << (id & 31));
}

}  // namespace xrt

// logits: [n_rows, vocab] 32-bit.  Per row: its slot (< 0 = padding, id -1), temperature, top_k
// (0 = all), top_p (>= 1 = all), repetition penalty (<= 1 = none).  seen: [slots, seen_words]
// bitmaps or null.  rng_key / rng_counter: per slot.
XRT_EXPORT int xrt_sample(int* out_ids, const float* logits, int n_rows, int vocab, const int* row_slot,
                          const float* temperature, const int* top_k, const float* top_p, const float* penalty,
                          const unsigned int* seen, int seen_words, const unsigned long long* rng_key,
                          unsigned int* rng_counter, cudaStream_t stream) {
  if (n_rows < 0 || vocab <= 0) return XRT_ERR_ARGUMENT;
  if (seen != nullptr && seen_words * 32 < vocab) return XRT_ERR_ARGUMENT;
  if (n_rows == 0) return XRT_OK;
  static bool allowed = false;
  if (!allowed) {  // static and dynamic shared memory together pass 48 KB
    cudaError_t err = cudaFuncSetAttribute(xrt::sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           xrt::SAMPLE_DYNAMIC_BYTES);
    if (err != cudaSuccess) return (int)err;
    allowed = true;
  }
  xrt::launch_kernel(xrt::sample_kernel, dim3(n_rows), dim3(xrt::SAMPLE_THREADS), xrt::SAMPLE_DYNAMIC_BYTES, stream, out_ids, logits, vocab,
                     row_slot, temperature, top_k, top_p, penalty, (const uint32_t*)seen, seen_words, rng_key, rng_counter);
  return xrt::launch_status();
}

XRT_EXPORT int xrt_mark_seen(unsigned int* seen, int seen_words, const int* slots, const int* ids, int n,
                             int vocab, cudaStream_t stream) {
  if (n < 0 || vocab <= 0 || seen_words * 32 < vocab) return XRT_ERR_ARGUMENT;
  if (n == 0) return XRT_OK;
  xrt::mark_seen_kernel<<<(n + 255) / 256, 256, 0, stream>>>(seen, seen_words, slots, ids, n, vocab);
  return xrt::launch_status();
}
