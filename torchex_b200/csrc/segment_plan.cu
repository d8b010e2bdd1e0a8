// Segment-offset builder: ids[n] -> (sid, perm, offsets) for the reduce kernels.
//
//   * texb_ids_inspect: one pass giving sortedness, id range and run count.
//   * sorted ids: offsets come from neighbour comparison (each entry written
//     exactly once, gaps in the id space become empty segments); no sort runs.
//   * unsorted ids: a stable least-significant-digit radix sort on the id with
//     the row index as payload.  Every digit pass is a per-tile histogram, an
//     exclusive scan over (digit, tile) and a stable scatter, i.e. three plain
//     launches with no inter-CTA waiting.  Rows of one segment therefore stay in
//     increasing row order, which makes the reduce result independent of run
//     order.
//
// Replaces ScatterData.__init__ / GetPreSumFunction
// (torchex/operator_py/scatter_op.py:7-21, 114-135) and the getPreSum kernel
// (torchex/src/scatter/scatter_kernel.cu:85-100), which only handle ids that
// are already sorted and dense.

#include <climits>

#include "common.cuh"

namespace texb {
namespace {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;
constexpr int kSortTile = kSortThreads * kSortItems;    // keys per CTA
constexpr int kWarpTile = 32 * kSortItems;              // keys per warp
constexpr int kSortWarps = kSortThreads / 32;

template <typename IdT>
__device__ __forceinline__ int32_t clamp_id(IdT v) {
  if (sizeof(IdT) == 8) {
    if (v > IdT(INT_MAX)) return INT_MAX;
    if (v < IdT(INT_MIN)) return INT_MIN;
  }
  return int32_t(v);
}

// ---- inspect --------------------------------------------------------------------

__global__ void init_inspect_stats_kernel(int32_t* stats) {
  if (threadIdx.x == 0) {
    stats[0] = 1;
    stats[1] = INT_MAX;
    stats[2] = INT_MIN;
    stats[3] = 0;
  }
}

template <typename IdT>
__global__ void inspect_ids_kernel(const IdT* __restrict__ ids, int64_t n, int32_t* stats) {
  int unsorted = 0, runs = 0;
  int32_t lo = INT_MAX, hi = INT_MIN;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n;
       i += int64_t(gridDim.x) * blockDim.x) {
    const IdT a = ids[i];
    const int32_t a32 = clamp_id<IdT>(a);
    lo = min(lo, a32);
    hi = max(hi, a32);
    if (i + 1 < n) {
      const IdT b = ids[i + 1];
      unsorted |= (a > b);
      runs += (a != b);
    } else {
      runs += 1;  // the last run
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    unsorted |= __shfl_xor_sync(0xffffffffu, unsorted, o);
    runs += __shfl_xor_sync(0xffffffffu, runs, o);
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  // One set of atomics per CTA: every atomic of the grid lands on the same four
  // words, and ten thousand of them (one set per warp) took longer than the read.
  __shared__ int s_unsorted, s_runs, s_lo, s_hi;
  if (threadIdx.x == 0) {
    s_unsorted = 0;
    s_runs = 0;
    s_lo = INT_MAX;
    s_hi = INT_MIN;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    if (unsorted) atomicOr(&s_unsorted, 1);
    if (runs) atomicAdd(&s_runs, runs);
    atomicMin(&s_lo, lo);
    atomicMax(&s_hi, hi);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_unsorted) atomicAnd(&stats[0], 0);
    if (s_lo != INT_MAX) atomicMin(&stats[1], s_lo);
    if (s_hi != INT_MIN) atomicMax(&stats[2], s_hi);
    if (s_runs) atomicAdd(&stats[3], s_runs);
  }
}

// ---- offsets from sorted ids -----------------------------------------------------

// Thread i in [0, n] owns the boundary before sorted position i and writes
// offsets[s] = i for every s in (id[i-1], id[i]], with id[-1] = -1 and id[n] = m.
template <typename IdT>
__global__ void offsets_from_sorted_kernel(const IdT* __restrict__ ids, int32_t* __restrict__ sid_out,
                                           int32_t* __restrict__ offsets, int n, int m,
                                           int32_t* plan_stats) {
  const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i > n) return;
  int64_t a = (i == 0) ? -1 : int64_t(ids[i - 1]);
  int64_t b = (i == n) ? int64_t(m) : int64_t(ids[i]);
  if (i < n) {
    if (plan_stats && (b < 0 || b >= m)) atomicAdd(&plan_stats[2], 1);
    if (sid_out) sid_out[i] = clamp_id<IdT>(ids[i]);
  }
  if (a < -1) a = -1;
  if (b > m) b = m;
  for (int64_t s = a + 1; s <= b; ++s) offsets[s] = int32_t(i);
}

__global__ void plan_stats_kernel(const int32_t* __restrict__ offsets, int m, int32_t* plan_stats) {
  int mx = 0, empty = 0;
  for (int64_t s = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; s < m;
       s += int64_t(gridDim.x) * blockDim.x) {
    const int c = offsets[s + 1] - offsets[s];
    mx = max(mx, c);
    empty += (c == 0);
  }
  for (int o = 16; o > 0; o >>= 1) {
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    empty += __shfl_xor_sync(0xffffffffu, empty, o);
  }
  __shared__ int s_mx, s_empty;
  if (threadIdx.x == 0) {
    s_mx = 0;
    s_empty = 0;
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    if (mx) atomicMax(&s_mx, mx);
    if (empty) atomicAdd(&s_empty, empty);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_mx) atomicMax(&plan_stats[0], s_mx);
    if (s_empty) atomicAdd(&plan_stats[1], s_empty);
  }
}

// ---- balance table ------------------------------------------------------------------
// cost(p) = 4 p + end_cost_x4 * (number of segments that end before p), taken
// as sid[p] - sid[0] (exact for dense ids, an over-estimate across gaps, always
// non-decreasing).  table[k] is the first position whose cost reaches k / K of
// the total, so consecutive entries cut the rows into K pieces of equal cost.
//
// Cuts that fall inside a segment are then moved forward to the start of the next
// segment when that is near: at most kSnapFar positions away if the plan's largest
// segment has at most kSnapFar rows (then EVERY cut lands on a segment start, no
// segment is ever split between two groups of lanes, and the reduce needs neither
// its stitching nor its fix-up launch: TEXB_PLAN_NO_SPLIT), else at most kSnapNear
// positions (fewer split segments at no visible cost in balance).  Moving cuts
// forward keeps the table non-decreasing.
constexpr int kSnapFar = 128;
constexpr int kSnapNear = 8;

__global__ void balance_table_kernel(const int32_t* __restrict__ sid, int n, int end_cost_x4,
                                     int32_t* __restrict__ table, int K,
                                     const int32_t* __restrict__ plan_stats) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k > K) return;
  if (k == 0) { table[0] = 0; return; }
  if (k == K) { table[K] = n; return; }
  const long long first = sid[0];
  const long long total = 4LL * n + (long long)end_cost_x4 * (sid[n - 1] - first + 1);
  // smallest target that piece k must reach, without overflow: total < 2^34 * 1024
  const long long target = (long long)(((__int128)total * k) / K);
  int lo = 0, hi = n;  // cost(lo) < target <= cost(hi), with cost(n) = total
  if (4LL * 0 + (long long)end_cost_x4 * 0 >= target) { table[k] = 0; return; }
  while (hi - lo > 1) {
    const int mid = lo + ((hi - lo) >> 1);
    const long long c = 4LL * mid + (long long)end_cost_x4 * (__ldg(sid + mid) - first);
    if (c < target) lo = mid; else hi = mid;
  }
  // hi in [1, n]: move it to the next segment start if it lies inside a segment
  if (hi < n) {
    const int s_here = __ldg(sid + hi);
    if (__ldg(sid + hi - 1) == s_here) {
      const int window = (plan_stats != nullptr && plan_stats[0] <= kSnapFar) ? kSnapFar : kSnapNear;
      const int far = min(hi + window, n);  // the segment ends at or before `far`, or the cut stays
      if (far == n || __ldg(sid + far) != s_here) {
        int a = hi, b = far;  // sid[a] == s_here; b == n or sid[b] != s_here: first position past the segment
        while (b - a > 1) {
          const int mid = a + ((b - a) >> 1);
          if (__ldg(sid + mid) == s_here) a = mid; else b = mid;
        }
        hi = b;
      }
    }
  }
  table[k] = hi;
}

// ---- radix sort passes -------------------------------------------------------------

template <typename IdT>
__device__ __forceinline__ uint32_t load_key(const void* keys, int64_t idx) {
  return uint32_t(clamp_id<IdT>(static_cast<const IdT*>(keys)[idx]));
}

// ghist[d * num_tiles + tile] = number of keys of this tile whose digit is d.
template <typename IdT>
__global__ void __launch_bounds__(kSortThreads)
radix_histogram_kernel(const void* __restrict__ keys, int n, int shift, uint32_t* __restrict__ ghist,
                       int num_tiles) {
  __shared__ uint32_t s_hist[kRadix];
  for (int d = threadIdx.x; d < kRadix; d += kSortThreads) s_hist[d] = 0u;
  __syncthreads();
  const int64_t tile0 = int64_t(blockIdx.x) * kSortTile;
#pragma unroll 4
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t idx = tile0 + k * kSortThreads + threadIdx.x;
    if (idx < n) atomicAdd(&s_hist[(load_key<IdT>(keys, idx) >> shift) & (kRadix - 1)], 1u);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kRadix; d += kSortThreads)
    ghist[int64_t(d) * num_tiles + blockIdx.x] = s_hist[d];
}

// In-place exclusive scan over `count` words by a single CTA of 1024 threads.
// The array is walked in slabs of 4096 words with coalesced accesses (thread t
// owns words 4t .. 4t+3 of the slab); the running total carries between slabs.
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(uint32_t* data, int64_t count) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t carry = 0u;
  for (int64_t base = 0; base < count; base += 4096) {
    const int64_t i0 = base + int64_t(threadIdx.x) * 4;
    uint32_t v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (i0 + k < count) ? data[i0 + k] : 0u;
    const uint32_t sum = v[0] + v[1] + v[2] + v[3];
    uint32_t incl = sum;
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = s_warp[lane];
      uint32_t wi = w;
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += t;
      }
      s_warp[lane] = wi - w;  // exclusive base of each warp
      if (lane == 31) s_total = wi;
    }
    __syncthreads();
    uint32_t run = carry + s_warp[warp] + (incl - sum);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (i0 + k < count) data[i0 + k] = run;
      run += v[k];
    }
    carry += s_total;
    __syncthreads();  // s_warp / s_total are rewritten by the next slab
  }
}

// Positions of one digit pass.  The keys of digit d and tile t go to
//   (keys of smaller digits) + (keys of digit d in earlier tiles) + rank within the tile.
// CTA d turns row d of ghist (one count per tile) into its exclusive prefix, in place,
// and leaves the row's total in totals[d]; the scatter kernel adds the prefix of the
// 256 totals itself.  256 CTAs of a few hundred counts each instead of one CTA walking
// every count of the pass (34 us per pass at 1 M keys).
__global__ void __launch_bounds__(kSortThreads)
digit_prefix_kernel(uint32_t* __restrict__ ghist, uint32_t* __restrict__ totals, int num_tiles) {
  __shared__ uint32_t s_warp[kSortWarps];
  __shared__ uint32_t s_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t* row = ghist + int64_t(blockIdx.x) * num_tiles;
  uint32_t carry = 0u;
  for (int base = 0; base < num_tiles; base += kSortThreads) {
    const int t = base + threadIdx.x;
    const uint32_t v = (t < num_tiles) ? row[t] : 0u;
    uint32_t incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = (lane < kSortWarps) ? s_warp[lane] : 0u;
      uint32_t wi = w;
      for (int o = 1; o < kSortWarps; o <<= 1) {
        const uint32_t u = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += u;
      }
      if (lane < kSortWarps) s_warp[lane] = wi - w;  // exclusive base of each warp
      if (lane == kSortWarps - 1) s_total = wi;
    }
    __syncthreads();
    if (t < num_tiles) row[t] = carry + s_warp[warp] + (incl - v);
    carry += s_total;
    __syncthreads();  // s_warp / s_total are rewritten by the next slab
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

// Stable scatter of one digit pass.  Within a warp, item k of lane l is key
// tile0 + warp * kWarpTile + k * 32 + l, so (warp, k, lane) order is key order.
template <typename IdT, bool FIRST>
__global__ void __launch_bounds__(kSortThreads)
radix_scatter_kernel(const void* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
                     int32_t* __restrict__ keys_out, int32_t* __restrict__ vals_out, int n, int shift,
                     const uint32_t* __restrict__ ghist, const uint32_t* __restrict__ totals,
                     int num_tiles) {
  static_assert(kRadix == kSortThreads, "one digit per thread in the prefix of the digit totals");
  __shared__ uint32_t s_wcount[kSortWarps][kRadix];
  __shared__ uint32_t s_gbase[kRadix];
  __shared__ uint32_t s_wsum[kSortWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kSortWarps * kRadix; i += kSortThreads) (&s_wcount[0][0])[i] = 0u;
  // exclusive prefix of the 256 digit totals (thread d owns digit d), kept for the end
  const uint32_t my_total = totals[threadIdx.x];
  uint32_t digit_incl = my_total;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t u = __shfl_up_sync(0xffffffffu, digit_incl, o);
    if (lane >= o) digit_incl += u;
  }
  if (lane == 31) s_wsum[warp] = digit_incl;
  __syncthreads();

  const int64_t w0 = int64_t(blockIdx.x) * kSortTile + int64_t(warp) * kWarpTile;
  uint32_t key[kSortItems];
  uint32_t rank[kSortItems];
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t idx = w0 + k * 32 + lane;
    const bool valid = idx < n;
    key[k] = valid ? load_key<IdT>(keys_in, idx) : 0u;
    const uint32_t d = (key[k] >> shift) & (kRadix - 1);
    const uint32_t tag = valid ? d : uint32_t(kRadix);  // out-of-range lanes group together
    const uint32_t peers = __match_any_sync(0xffffffffu, tag);
    const int leader = __ffs(peers) - 1;
    uint32_t before = 0u;
    if (valid && lane == leader) {
      before = s_wcount[warp][d];
      s_wcount[warp][d] = before + __popc(peers);
    }
    before = __shfl_sync(0xffffffffu, before, leader);
    rank[k] = before + __popc(peers & lt_mask);
    __syncwarp();
  }
  __syncthreads();
  for (int d = threadIdx.x; d < kRadix; d += kSortThreads) {
    uint32_t run = 0u;
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      const uint32_t c = s_wcount[w][d];
      s_wcount[w][d] = run;
      run += c;
    }
    uint32_t digit_base = digit_incl - my_total;  // d == threadIdx.x
    for (int w = 0; w < warp; ++w) digit_base += s_wsum[w];
    s_gbase[d] = digit_base + ghist[int64_t(d) * num_tiles + blockIdx.x];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t idx = w0 + k * 32 + lane;
    if (idx < n) {
      const uint32_t d = (key[k] >> shift) & (kRadix - 1);
      const uint32_t pos = s_gbase[d] + s_wcount[warp][d] + rank[k];
      keys_out[pos] = int32_t(key[k]);
      vals_out[pos] = FIRST ? int32_t(idx) : vals_in[idx];
    }
  }
}

int bit_width(int64_t v) {
  int b = 0;
  while (v > 0) { ++b; v >>= 1; }
  return b;
}

int num_sort_passes(int64_t m) {
  int bits = bit_width(m > 1 ? m - 1 : 1);
  return (bits + kRadixBits - 1) / kRadixBits;
}

struct SortWorkspace {
  int32_t* tmp_keys;
  int32_t* tmp_vals;
  uint32_t* ghist;
  size_t bytes;
};

SortWorkspace carve_sort_workspace(void* ws, int64_t n) {
  SortWorkspace s;
  const size_t arr = align_up(size_t(n) * sizeof(int32_t), 256);
  const int64_t tiles = ceil_div(n, kSortTile);
  const size_t hist = align_up((size_t(tiles) + 1) * kRadix * sizeof(uint32_t), 256);  // counts + digit totals
  uintptr_t base = align_up(reinterpret_cast<uintptr_t>(ws), 256);
  s.tmp_keys = reinterpret_cast<int32_t*>(base);
  s.tmp_vals = reinterpret_cast<int32_t*>(base + arr);
  s.ghist = reinterpret_cast<uint32_t*>(base + 2 * arr);
  s.bytes = 2 * arr + hist + 256;
  return s;
}

template <typename IdT>
int run_sort(const void* ids, int64_t n, int64_t m, int32_t* sid_out, int32_t* perm_out,
             const SortWorkspace& sw, cudaStream_t stream) {
  const int passes = num_sort_passes(m);
  const int tiles = int(ceil_div(n, kSortTile));
  const void* src_k = ids;
  const int32_t* src_v = nullptr;
  for (int p = 0; p < passes; ++p) {
    const bool to_out = ((passes - 1 - p) % 2) == 0;
    int32_t* dst_k = to_out ? sid_out : sw.tmp_keys;
    int32_t* dst_v = to_out ? perm_out : sw.tmp_vals;
    const int shift = p * kRadixBits;
    if (p == 0) {
      radix_histogram_kernel<IdT><<<tiles, kSortThreads, 0, stream>>>(src_k, int(n), shift, sw.ghist, tiles);
    } else {
      radix_histogram_kernel<int32_t><<<tiles, kSortThreads, 0, stream>>>(src_k, int(n), shift, sw.ghist, tiles);
    }
    uint32_t* totals = sw.ghist + int64_t(tiles) * kRadix;
    digit_prefix_kernel<<<kRadix, kSortThreads, 0, stream>>>(sw.ghist, totals, tiles);
    if (p == 0) {
      radix_scatter_kernel<IdT, true><<<tiles, kSortThreads, 0, stream>>>(
          src_k, src_v, dst_k, dst_v, int(n), shift, sw.ghist, totals, tiles);
    } else {
      radix_scatter_kernel<int32_t, false><<<tiles, kSortThreads, 0, stream>>>(
          src_k, src_v, dst_k, dst_v, int(n), shift, sw.ghist, totals, tiles);
    }
    int st = check_launch("radix sort pass");
    if (st != TEXB_OK) return st;
    src_k = dst_k;
    src_v = dst_v;
  }
  return TEXB_OK;
}

template <typename IdT>
int run_offsets(const void* sorted_ids, int32_t* sid_out, int32_t* offsets, int64_t n, int64_t m,
                int32_t* plan_stats, cudaStream_t stream) {
  const int64_t threads = n + 1;
  offsets_from_sorted_kernel<IdT><<<unsigned(ceil_div(threads, 256)), 256, 0, stream>>>(
      static_cast<const IdT*>(sorted_ids), sid_out, offsets, int(n), int(m), plan_stats);
  int st = check_launch("offsets_from_sorted_kernel");
  if (st != TEXB_OK) return st;
  if (m > 0) {
    int64_t blocks = ceil_div(m, 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    plan_stats_kernel<<<unsigned(blocks), 256, 0, stream>>>(offsets, int(m), plan_stats);
    st = check_launch("plan_stats_kernel");
  }
  return st;
}

}  // namespace

int ids_inspect_impl(const void* ids, int id_bytes, int64_t n, int32_t* stats_dev,
                     cudaStream_t stream) {
  if (id_bytes != 4 && id_bytes != 8)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "id_bytes must be 4 or 8, got %d", id_bytes);
  if (n < 0 || !stats_dev || (n > 0 && !ids))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "ids_inspect: bad pointer or size");
  init_inspect_stats_kernel<<<1, 32, 0, stream>>>(stats_dev);
  if (n > 0) {
    int64_t blocks = ceil_div(n, 256 * 4);
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (id_bytes == 4)
      inspect_ids_kernel<int32_t><<<unsigned(blocks), 256, 0, stream>>>(
          static_cast<const int32_t*>(ids), n, stats_dev);
    else
      inspect_ids_kernel<int64_t><<<unsigned(blocks), 256, 0, stream>>>(
          static_cast<const int64_t*>(ids), n, stats_dev);
  }
  return check_launch("inspect_ids_kernel");
}

size_t plan_workspace_bytes_impl(int64_t n, int64_t m, int sorted) {
  (void)m;
  if (sorted || n <= 0) return 256;
  return carve_sort_workspace(nullptr, n).bytes;
}

int plan_build_impl(const void* ids, int id_bytes, int64_t n, int64_t m, int sorted,
                    int32_t* sid_out, int32_t* perm_out, int32_t* offsets_out,
                    int32_t* plan_stats_dev, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream) {
  if (id_bytes != 4 && id_bytes != 8)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "id_bytes must be 4 or 8, got %d", id_bytes);
  if (n < 0 || m < 0) return fail(TEXB_ERR_INVALID_ARGUMENT, "plan_build: negative size");
  if (n > INT_MAX - 65536 || m > INT_MAX - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "plan_build: n and num_segments must be below 2^31 - 65536");
  if (!offsets_out || !plan_stats_dev || (n > 0 && (!ids || !sid_out)))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "plan_build: NULL pointer");
  if (!sorted && n > 0 && !perm_out)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "plan_build: perm_out is required for unsorted ids");
  if (!sorted && n > 0 && static_cast<const void*>(sid_out) == ids)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "plan_build: sid_out may not alias unsorted ids");
  cudaError_t e = cudaMemsetAsync(plan_stats_dev, 0, 4 * sizeof(int32_t), stream);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));

  if (sorted || n == 0) {
    int32_t* sid_dst = (static_cast<const void*>(sid_out) == ids) ? nullptr : sid_out;
    if (id_bytes == 4)
      return run_offsets<int32_t>(ids, sid_dst, offsets_out, n, m, plan_stats_dev, stream);
    return run_offsets<int64_t>(ids, sid_dst, offsets_out, n, m, plan_stats_dev, stream);
  }

  SortWorkspace sw = carve_sort_workspace(workspace, n);
  const size_t pad = reinterpret_cast<uintptr_t>(sw.tmp_keys) - reinterpret_cast<uintptr_t>(workspace);
  if (!workspace || workspace_bytes + 256 < sw.bytes + pad)
    return fail(TEXB_ERR_WORKSPACE, "plan workspace: need %zu bytes, got %zu", sw.bytes,
                workspace_bytes);
  int st = (id_bytes == 4) ? run_sort<int32_t>(ids, n, m, sid_out, perm_out, sw, stream)
                           : run_sort<int64_t>(ids, n, m, sid_out, perm_out, sw, stream);
  if (st != TEXB_OK) return st;
  // sid_out now holds the sorted ids; offsets come from their run boundaries.
  return run_offsets<int32_t>(sid_out, nullptr, offsets_out, n, m, plan_stats_dev, stream);
}

namespace {

// ---- dense ids from arbitrary keys (the torch.unique step) ----------------------------
// Sorted keys -> run starts -> dense ids.  Tile = kSortTile consecutive sorted
// positions; thread t of a tile owns 16 consecutive positions.

__global__ void __launch_bounds__(kSortThreads)
unique_tile_count_kernel(const int32_t* __restrict__ keys, int n, uint32_t* __restrict__ tile_counts) {
  __shared__ uint32_t s_warp[kSortWarps];
  const int64_t p0 = int64_t(blockIdx.x) * kSortTile + int64_t(threadIdx.x) * kSortItems;
  uint32_t c = 0;
#pragma unroll 4
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t p = p0 + k;
    if (p < n) c += (p == 0) || (keys[p] != keys[p - 1]);
  }
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t t = 0;
    for (int w = 0; w < kSortWarps; ++w) t += s_warp[w];
    tile_counts[blockIdx.x] = t;
  }
}

// After the exclusive scan of tile_counts: total number of distinct keys.
__global__ void unique_total_kernel(const uint32_t* __restrict__ tile_base, const int32_t* __restrict__ keys,
                                    int n, int num_tiles, int32_t* stats) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  // base of the last tile + its own count (recounted: the scan overwrote it)
  uint32_t c = 0;
  for (int64_t p = int64_t(num_tiles - 1) * kSortTile; p < n; ++p) c += (p == 0) || (keys[p] != keys[p - 1]);
  stats[0] = int32_t(tile_base[num_tiles - 1] + c);
}

__global__ void __launch_bounds__(kSortThreads)
unique_fill_kernel(const int32_t* __restrict__ keys, const int32_t* __restrict__ perm, int n, int m,
                   const uint32_t* __restrict__ tile_base, int32_t* __restrict__ sid,
                   int32_t* __restrict__ offsets, int32_t* __restrict__ unq_inv,
                   int32_t* __restrict__ unique_keys) {
  __shared__ uint32_t s_warp[kSortWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t p0 = int64_t(blockIdx.x) * kSortTile + int64_t(threadIdx.x) * kSortItems;
  uint32_t flags = 0;
#pragma unroll 4
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t p = p0 + k;
    if (p < n && ((p == 0) || (keys[p] != keys[p - 1]))) flags |= 1u << k;
  }
  const uint32_t mine = __popc(flags);
  uint32_t incl = mine;
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  uint32_t before = tile_base[blockIdx.x] + incl - mine;
  for (int w = 0; w < warp; ++w) before += s_warp[w];
  // `before` = number of run starts in front of this thread's first position
  int32_t id = int32_t(before) - 1;
  for (int k = 0; k < kSortItems; ++k) {
    const int64_t p = p0 + k;
    if (p >= n) break;
    if (flags & (1u << k)) {
      ++id;
      if (id < m) {
        offsets[id] = int32_t(p);
        unique_keys[id] = keys[p];
      }
    }
    sid[p] = id;
    const int row = perm ? perm[p] : int(p);
    if (row >= 0 && row < n) unq_inv[row] = id;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) offsets[m] = n;
}

__global__ void narrow_keys_kernel(const int64_t* __restrict__ in, int32_t* __restrict__ out, int64_t n) {
  const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i < n) out[i] = clamp_id<int64_t>(in[i]);
}

struct UniqueWorkspace {
  SortWorkspace sort;
  uint32_t* tile_counts;
  size_t bytes;
};

UniqueWorkspace carve_unique_workspace(void* ws, int64_t n) {
  UniqueWorkspace u;
  u.sort = carve_sort_workspace(ws, n);
  const size_t tiles = size_t(ceil_div(n > 0 ? n : 1, kSortTile));
  uintptr_t base = reinterpret_cast<uintptr_t>(u.sort.tmp_keys) + align_up(u.sort.bytes, 256);
  u.tile_counts = reinterpret_cast<uint32_t*>(base);
  u.bytes = align_up(u.sort.bytes, 256) + align_up(tiles * sizeof(uint32_t), 256) + 256;
  return u;
}

}  // namespace

size_t unique_workspace_bytes_impl(int64_t n) { return n > 0 ? carve_unique_workspace(nullptr, n).bytes : 512; }

int unique_count_impl(const void* keys, int key_bytes, int64_t n, int64_t key_bound, int sorted,
                      int32_t* sorted_keys, int32_t* perm, int32_t* stats_dev, void* workspace,
                      size_t workspace_bytes, cudaStream_t stream) {
  if (key_bytes != 4 && key_bytes != 8)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "key_bytes must be 4 or 8, got %d", key_bytes);
  if (n < 0 || key_bound < 0 || !stats_dev || (n > 0 && (!keys || !sorted_keys)))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unique_count: bad pointer or size");
  if (n > INT_MAX - 65536 || key_bound > INT_MAX)
    return fail(TEXB_ERR_UNSUPPORTED, "unique_count: n and the keys must be below 2^31");
  if (!sorted && n > 0 && !perm)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unique_count: perm is required for unsorted keys");
  cudaError_t e = cudaMemsetAsync(stats_dev, 0, 4 * sizeof(int32_t), stream);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  if (n == 0) return TEXB_OK;
  UniqueWorkspace uw = carve_unique_workspace(workspace, n);
  const size_t pad = reinterpret_cast<uintptr_t>(uw.sort.tmp_keys) - reinterpret_cast<uintptr_t>(workspace);
  if (!workspace || workspace_bytes + 256 < uw.bytes + pad)
    return fail(TEXB_ERR_WORKSPACE, "unique workspace: need %zu bytes, got %zu", uw.bytes, workspace_bytes);
  if (sorted) {
    if (key_bytes == 8) {
      narrow_keys_kernel<<<unsigned(ceil_div(n, 256)), 256, 0, stream>>>(static_cast<const int64_t*>(keys),
                                                                        sorted_keys, n);
    } else if (static_cast<const void*>(sorted_keys) != keys) {
      e = cudaMemcpyAsync(sorted_keys, keys, size_t(n) * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemcpyAsync: %s", cudaGetErrorString(e));
    }
  } else {
    if (static_cast<const void*>(sorted_keys) == keys)
      return fail(TEXB_ERR_INVALID_ARGUMENT, "unique_count: sorted_keys may not alias unsorted keys");
    int st = (key_bytes == 4) ? run_sort<int32_t>(keys, n, key_bound, sorted_keys, perm, uw.sort, stream)
                              : run_sort<int64_t>(keys, n, key_bound, sorted_keys, perm, uw.sort, stream);
    if (st != TEXB_OK) return st;
  }
  const int tiles = int(ceil_div(n, kSortTile));
  unique_tile_count_kernel<<<tiles, kSortThreads, 0, stream>>>(sorted_keys, int(n), uw.tile_counts);
  exclusive_scan_kernel<<<1, 1024, 0, stream>>>(uw.tile_counts, tiles);
  unique_total_kernel<<<1, 32, 0, stream>>>(uw.tile_counts, sorted_keys, int(n), tiles, stats_dev);
  return check_launch("unique count kernels");
}

int unique_fill_impl(const int32_t* sorted_keys, const int32_t* perm, int64_t n, int64_t m, int32_t* sid,
                     int32_t* offsets, int32_t* unq_inv, int32_t* unique_keys, int32_t* plan_stats_dev,
                     void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (n < 0 || m < 0 || !offsets || !plan_stats_dev ||
      (n > 0 && (!sorted_keys || !sid || !unq_inv || !unique_keys)))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unique_fill: bad pointer or size");
  if (n > INT_MAX - 65536) return fail(TEXB_ERR_UNSUPPORTED, "unique_fill: n must be below 2^31 - 65536");
  cudaError_t e = cudaMemsetAsync(plan_stats_dev, 0, 4 * sizeof(int32_t), stream);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  if (n == 0) {
    e = cudaMemsetAsync(offsets, 0, size_t(m + 1) * sizeof(int32_t), stream);
    if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return TEXB_OK;
  }
  UniqueWorkspace uw = carve_unique_workspace(workspace, n);
  const size_t pad = reinterpret_cast<uintptr_t>(uw.sort.tmp_keys) - reinterpret_cast<uintptr_t>(workspace);
  if (!workspace || workspace_bytes + 256 < uw.bytes + pad)
    return fail(TEXB_ERR_WORKSPACE, "unique workspace: need %zu bytes, got %zu", uw.bytes, workspace_bytes);
  const int tiles = int(ceil_div(n, kSortTile));
  unique_fill_kernel<<<tiles, kSortThreads, 0, stream>>>(sorted_keys, perm, int(n), int(m), uw.tile_counts, sid,
                                                         offsets, unq_inv, unique_keys);
  int st = check_launch("unique_fill_kernel");
  if (st != TEXB_OK || m == 0) return st;
  int64_t blocks = ceil_div(m, 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  plan_stats_kernel<<<unsigned(blocks), 256, 0, stream>>>(offsets, int(m), plan_stats_dev);
  return check_launch("plan_stats_kernel");
}

int plan_balance_impl(const int32_t* sid, int64_t n, int32_t* table, int table_len, const int32_t* plan_stats,
                      cudaStream_t stream) {
  if (n < 0 || !table || table_len < 2 || (n > 0 && !sid))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "plan_balance: bad pointer or size");
  if (n > INT_MAX - 65536) return fail(TEXB_ERR_UNSUPPORTED, "plan_balance: n must be below 2^31 - 65536");
  const int K = table_len - 1;
  if (n == 0) {
    cudaError_t e = cudaMemsetAsync(table, 0, size_t(table_len) * sizeof(int32_t), stream);
    if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return TEXB_OK;
  }
  balance_table_kernel<<<unsigned(ceil_div(table_len, 256)), 256, 0, stream>>>(
      sid, int(n), tuning().end_cost_x4, table, K, plan_stats);
  return check_launch("balance_table_kernel");
}

// Plan entries found outside their range by segment_rank_kernel (a segment id outside
// [0, num_segments), a perm entry outside [0, n)): the entry is skipped and counted
// (sticky; part of texb_device_status) instead of being used as an address.
__device__ int g_plan_bad_indices = 0;

// rank[row of position p] = p - offsets[sid[p]]: the index of every point inside
// its segment, in increasing row order (the plan's sort is stable).
__global__ void segment_rank_kernel(const int32_t* __restrict__ sid, const int32_t* __restrict__ perm,
                                    const int32_t* __restrict__ offsets, int n, int m,
                                    int64_t* __restrict__ rank) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  const int row = perm ? perm[p] : p;
  const int s = sid[p];
  if (unsigned(row) >= unsigned(n) || unsigned(s) >= unsigned(m)) {
    atomicAdd(&g_plan_bad_indices, 1);
    return;
  }
  rank[row] = int64_t(p - offsets[s]);
}

int segment_rank_impl(const int32_t* sid, const int32_t* perm, const int32_t* offsets, int64_t n,
                      int64_t num_segments, int64_t* rank_out, cudaStream_t stream) {
  if (n < 0 || num_segments < 0 || (n > 0 && (!sid || !offsets || !rank_out)))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "segment_rank: bad pointer or size");
  if (n > INT_MAX - 65536 || num_segments > INT_MAX - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "segment_rank: n and num_segments must be below 2^31 - 65536");
  if (n == 0) return TEXB_OK;
  segment_rank_kernel<<<unsigned(ceil_div(n, 256)), 256, 0, stream>>>(sid, perm, offsets, int(n),
                                                                      int(num_segments), rank_out);
  return check_launch("segment_rank_kernel");
}

int plan_bad_indices_impl(int* count) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_plan_bad_indices, sizeof(int));
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  *count = v;
  return TEXB_OK;
}

int get_pre_sum_impl(const int32_t* unq_inv, int32_t* pre_sum, int64_t num_total, int64_t num_unq,
                     cudaStream_t stream) {
  if (num_total < 0 || num_unq < 0 || !pre_sum || (num_total > 0 && !unq_inv))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "get_pre_sum: bad pointer or size");
  if (num_total > INT_MAX - 65536 || num_unq > INT_MAX - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "get_pre_sum: sizes must be below 2^31 - 65536");
  offsets_from_sorted_kernel<int32_t><<<unsigned(ceil_div(num_total + 1, 256)), 256, 0, stream>>>(
      unq_inv, nullptr, pre_sum, int(num_total), int(num_unq), nullptr);
  return check_launch("offsets_from_sorted_kernel");
}

}  // namespace texb
