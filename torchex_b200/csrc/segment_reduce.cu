// Forward segment reduction (sum / mean / max+argmax) for sm_100a.
//
// Work is split by ROWS of the segment-sorted order, never by segments, so a
// 100 000-row segment and 100 000 one-row segments cost the same:
//
//   * a CTA owns `rows_per_cta` consecutive sorted positions; inside it every
//     "group" of LPR lanes (LPR * VEC channels wide, one 128-bit load per lane
//     when VEC == 4) owns a consecutive sub-range and walks it row by row with
//     several row loads in flight, keeping one running accumulator per channel;
//   * a segment that starts and ends inside a group's sub-range is written
//     straight to `out`; a run that touches the edge of the sub-range is left
//     in shared memory, and one group then stitches the CTA's edge runs in
//     position order (segments that live inside one CTA finish here);
//   * runs that cross a CTA edge go to a small workspace (two records per CTA)
//     and the fix-up kernel stitches those chains, again in position order.
//
// The combination order depends only on the geometry, so results are
// bit-reproducible, and no floating-point atomic is used anywhere.
//
// Replaces scatter_sum / scatter_max and their launchers in
// torchex/src/scatter/scatter_kernel.cu:102-192, whose block shape is sized
// from the largest segment and whose lanes run along rows (4-byte loads at a
// stride of C * 4 bytes).

#include <cfloat>
#include <cstdio>

#include "common.cuh"

namespace texb {
namespace {

constexpr unsigned kValid = 1u;
constexpr unsigned kOpenLeft = 2u;   // segment began before this range
constexpr unsigned kOpenRight = 4u;  // segment continues after this range

template <int VEC>
struct Acc {
  float a[VEC];     // running sum, or running maximum
  uint32_t b[VEC];  // bits of the compensation term, or row index of the maximum
};

// ---- operators --------------------------------------------------------------

struct OpSumComp {  // sum with an error-free two-sum; value = a + b
  static constexpr bool kIsMax = false;
  template <int VEC>
  static __device__ __forceinline__ void init(Acc<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.a[k] = 0.f; x.b[k] = 0u; }
  }
  static __device__ __forceinline__ void two_sum(float s, float v, float& t, float& e) {
    t = s + v;
    float bp = t - s;
    e = (s - (t - bp)) + (v - bp);
  }
  template <int VEC>
  static __device__ __forceinline__ void add(Acc<VEC>& x, const float (&v)[VEC], int) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float t, e;
      two_sum(x.a[k], v[k], t, e);
      x.b[k] = __float_as_uint(__uint_as_float(x.b[k]) + e);
      x.a[k] = t;
    }
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(Acc<VEC>& x, const Acc<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      float t, e;
      two_sum(x.a[k], y.a[k], t, e);
      x.b[k] = __float_as_uint((__uint_as_float(x.b[k]) + __uint_as_float(y.b[k])) + e);
      x.a[k] = t;
    }
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const Acc<VEC>& x, int k) {
    return x.a[k] + __uint_as_float(x.b[k]);
  }
};

struct OpSumPlain {  // plain fp32 running sum
  static constexpr bool kIsMax = false;
  template <int VEC>
  static __device__ __forceinline__ void init(Acc<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.a[k] = 0.f; x.b[k] = 0u; }
  }
  template <int VEC>
  static __device__ __forceinline__ void add(Acc<VEC>& x, const float (&v)[VEC], int) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.a[k] += v[k];
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(Acc<VEC>& x, const Acc<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.a[k] += y.a[k];
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const Acc<VEC>& x, int k) {
    return x.a[k];
  }
};

struct OpMax {  // maximum + row index; ties -> lowest row; NaN never wins
  static constexpr bool kIsMax = true;
  template <int VEC>
  static __device__ __forceinline__ void init(Acc<VEC>& x) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { x.a[k] = -FLT_MAX; x.b[k] = 0xffffffffu; }
  }
  template <int VEC>
  static __device__ __forceinline__ void add(Acc<VEC>& x, const float (&v)[VEC], int row) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      bool take = (v[k] > x.a[k]) || (v[k] == x.a[k] && uint32_t(row) < x.b[k]);
      if (take) { x.a[k] = v[k]; x.b[k] = uint32_t(row); }
    }
  }
  template <int VEC>
  static __device__ __forceinline__ void merge(Acc<VEC>& x, const Acc<VEC>& y) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      bool take = (y.a[k] > x.a[k]) || (y.a[k] == x.a[k] && y.b[k] < x.b[k]);
      if (take) { x.a[k] = y.a[k]; x.b[k] = y.b[k]; }
    }
  }
  template <int VEC>
  static __device__ __forceinline__ float value(const Acc<VEC>& x, int k) {
    return x.a[k];
  }
};

// ---- small device helpers -----------------------------------------------------

template <int VEC>
__device__ __forceinline__ void load_row(const float* __restrict__ p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = __ldg(p + k);
  }
}

template <int VEC>
__device__ __forceinline__ void store_words(uint32_t* p, const uint32_t (&v)[VEC]) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<uint4*>(p) = make_uint4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) p[k] = v[k];
  }
}

template <int VEC>
__device__ __forceinline__ void load_words(const uint32_t* p, uint32_t (&v)[VEC]) {
  if constexpr (VEC == 4) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = p[k];
  }
}

// Accumulator <-> two arrays of VEC 32-bit words (shared or global memory).
template <int VEC>
__device__ __forceinline__ void store_acc(uint32_t* pa, uint32_t* pb, const Acc<VEC>& x) {
  uint32_t wa[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) wa[k] = __float_as_uint(x.a[k]);
  store_words<VEC>(pa, wa);
  store_words<VEC>(pb, x.b);
}

template <int VEC>
__device__ __forceinline__ void load_acc(const uint32_t* pa, const uint32_t* pb, Acc<VEC>& x) {
  uint32_t wa[VEC];
  load_words<VEC>(pa, wa);
  load_words<VEC>(pb, x.b);
#pragma unroll
  for (int k = 0; k < VEC; ++k) x.a[k] = __uint_as_float(wa[k]);
}

// Writes one finished segment row.  `ch` is this lane's first channel.
template <class Op, int VEC>
__device__ __forceinline__ void store_out(float* __restrict__ out, int32_t* __restrict__ arg,
                                          int64_t seg, int C, int ch, bool lane_on,
                                          const Acc<VEC>& x, int cnt, bool mean) {
  if (!lane_on) return;
  float r[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) r[k] = Op::template value<VEC>(x, k);
  if (!Op::kIsMax && mean) {
    float c = float(cnt);
#pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = __fdiv_rn(r[k], c);
  }
  float* po = out + seg * C + ch;
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(po) = make_float4(r[0], r[1], r[2], r[3]);
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) po[k] = r[k];
  }
  if constexpr (Op::kIsMax) {
    int32_t* pa = arg + seg * C + ch;
    if constexpr (VEC == 4) {
      *reinterpret_cast<int4*>(pa) = make_int4(int(x.b[0]), int(x.b[1]), int(x.b[2]), int(x.b[3]));
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) pa[k] = int(x.b[k]);
    }
  }
}

// Workspace: for CTA b and channel slab y there are two records,
// rec = (y * num_ctas + b) * 2 + {0: head, 1: tail}.  A record is CPS words of
// `a`, CPS words of `b` (CPS = LPR * VEC channels per slab) and an int4 of
// meta {sid, row count, flags, 0}.
struct Workspace {
  uint32_t* vec;  // [num_slabs * num_ctas * 2][2 * CPS]
  int4* meta;     // [num_slabs * num_ctas * 2]
};

// ---- main kernel --------------------------------------------------------------

template <class Op, int VEC, int LPR, bool HAS_PERM>
__global__ void __launch_bounds__(kCtaThreads)
segment_reduce_kernel(const float* __restrict__ feats, const int32_t* __restrict__ sid,
                      const int32_t* __restrict__ perm, float* __restrict__ out,
                      int32_t* __restrict__ arg, Workspace ws, int n, int C,
                      int rows_per_cta, int rows_per_group, bool mean) {
  constexpr int GPC = kCtaThreads / LPR;           // groups per CTA
  constexpr int CPS = LPR * VEC;                   // channels per slab
  constexpr int U = (LPR >= 8) ? 8 : LPR;          // row loads in flight per group
  constexpr int SLOTS = 2 * GPC;

  __shared__ __align__(16) uint32_t s_vec[SLOTS * 2 * CPS];
  __shared__ int s_sid[SLOTS];
  __shared__ int s_cnt[SLOTS];
  __shared__ unsigned s_flag[SLOTS];

  const int lane_g = threadIdx.x & (LPR - 1);
  const int group = threadIdx.x / LPR;
  const unsigned gmask =
      (LPR == 32) ? 0xffffffffu
                  : (((1u << LPR) - 1u) << ((threadIdx.x & 31) & ~(LPR - 1)));
  const int ch = blockIdx.y * CPS + lane_g * VEC;  // first channel of this lane
  const bool lane_on = ch < C;                     // VEC == 4 implies C % 4 == 0

  const int c0 = blockIdx.x * rows_per_cta;
  const int c1 = min(c0 + rows_per_cta, n);
  const int g0 = c0 + group * rows_per_group;
  const int g1 = min(g0 + rows_per_group, c1);

  if (lane_g == 0) {
    s_flag[2 * group] = 0u;
    s_flag[2 * group + 1] = 0u;
  }

  if (g0 < g1) {
    int cur_sid = __ldg(sid + g0);
    const bool first_open_left = (g0 > 0) && (__ldg(sid + g0 - 1) == cur_sid);
    bool is_first = true;
    int cnt = 0;
    Acc<VEC> acc;
    Op::template init<VEC>(acc);

    // Ends the current run.  open_right is only ever true for the last run.
    auto close_run = [&](bool open_right) {
      const bool open_left = is_first && first_open_left;
      if (!open_left && !open_right) {
        store_out<Op, VEC>(out, arg, cur_sid, C, ch, lane_on, acc, cnt, mean);
      } else {
        const int slot = 2 * group + (open_right ? 1 : 0);
        uint32_t* pa = s_vec + slot * 2 * CPS + lane_g * VEC;
        store_acc<VEC>(pa, pa + CPS, acc);
        if (lane_g == 0) {
          s_sid[slot] = cur_sid;
          s_cnt[slot] = cnt;
          s_flag[slot] = kValid | (open_left ? kOpenLeft : 0u) | (open_right ? kOpenRight : 0u);
        }
      }
    };

    for (int base = g0; base < g1; base += LPR) {
      const int p = base + lane_g;
      int my_sid = -1, my_row = 0;
      if (p < g1) {
        my_sid = __ldg(sid + p);
        my_row = HAS_PERM ? __ldg(perm + p) : p;
      }
#pragma unroll 1
      for (int j = 0; j < LPR; j += U) {
        if (base + j >= g1) break;
        float v[U][VEC];
        int s[U], r[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
          s[k] = __shfl_sync(gmask, my_sid, j + k, LPR);
          r[k] = __shfl_sync(gmask, my_row, j + k, LPR);
          if (s[k] >= 0 && lane_on) {
            load_row<VEC>(feats + int64_t(r[k]) * C + ch, v[k]);
          } else {
#pragma unroll
            for (int q = 0; q < VEC; ++q) v[k][q] = 0.f;
          }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
          if (s[k] >= 0) {
            if (s[k] != cur_sid) {
              close_run(false);
              cur_sid = s[k];
              is_first = false;
              cnt = 0;
              Op::template init<VEC>(acc);
            }
            Op::template add<VEC>(acc, v[k], r[k]);
            ++cnt;
          }
        }
      }
    }
    const bool open_right = (g1 < n) && (__ldg(sid + g1) == cur_sid);
    close_run(open_right);
  }
  __syncthreads();

  // Stitch the edge runs of this CTA in position order (group 0 only).
  if (group == 0) {
    const int64_t rec = (int64_t(blockIdx.y) * gridDim.x + blockIdx.x) * 2;
    bool have = false, cur_open_left = false;
    int cur_sid = 0, cur_cnt = 0;
    unsigned head_flag = 0u;
    Acc<VEC> cur;
    Op::template init<VEC>(cur);
    for (int slot = 0; slot < SLOTS; ++slot) {
      const unsigned f = s_flag[slot];
      if (!(f & kValid)) continue;
      Acc<VEC> x;
      const uint32_t* pa = s_vec + slot * 2 * CPS + lane_g * VEC;
      load_acc<VEC>(pa, pa + CPS, x);
      if (!have) {
        cur = x;
        cur_sid = s_sid[slot];
        cur_cnt = s_cnt[slot];
        cur_open_left = (f & kOpenLeft) != 0u;
        have = true;
      } else {
        Op::template merge<VEC>(cur, x);
        cur_cnt += s_cnt[slot];
      }
      if (!(f & kOpenRight)) {
        if (!cur_open_left) {
          store_out<Op, VEC>(out, arg, cur_sid, C, ch, lane_on, cur, cur_cnt, mean);
        } else {
          uint32_t* ga = ws.vec + rec * 2 * CPS + lane_g * VEC;
          store_acc<VEC>(ga, ga + CPS, cur);
          head_flag = kValid | kOpenLeft;
          if (lane_g == 0) ws.meta[rec] = make_int4(cur_sid, cur_cnt, int(head_flag), 0);
        }
        have = false;
      }
    }
    if (head_flag == 0u && lane_g == 0) ws.meta[rec] = make_int4(0, 0, 0, 0);
    if (have) {
      uint32_t* ga = ws.vec + (rec + 1) * 2 * CPS + lane_g * VEC;
      store_acc<VEC>(ga, ga + CPS, cur);
      const unsigned f = kValid | kOpenRight | (cur_open_left ? kOpenLeft : 0u);
      if (lane_g == 0) ws.meta[rec + 1] = make_int4(cur_sid, cur_cnt, int(f), 0);
    } else if (lane_g == 0) {
      ws.meta[rec + 1] = make_int4(0, 0, 0, 0);
    }
  }
}

// ---- fix-up kernel --------------------------------------------------------------
// Block (b, y) finishes the segment whose first piece is CTA b's tail record
// (valid, open to the right, not open to the left).  The pieces that follow are
// the tail records of the CTAs the segment runs through and the head record of
// the CTA where it ends.

template <class Op, int VEC, int LPR>
__global__ void __launch_bounds__(kCtaThreads)
segment_fixup_kernel(Workspace ws, float* __restrict__ out, int32_t* __restrict__ arg,
                     int num_ctas, int C, bool mean) {
  constexpr int GPC = kCtaThreads / LPR;
  constexpr int CPS = LPR * VEC;

  __shared__ __align__(16) uint32_t s_vec[GPC * 2 * CPS];
  __shared__ int s_cnt[GPC];
  __shared__ int s_last;

#if __CUDA_ARCH__ >= 900
  // With programmatic dependent launch this grid may start before the reduce
  // grid has finished; wait for its memory to be visible.  No-op otherwise.
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif

  const int b = blockIdx.x;
  const int64_t rec_base = int64_t(blockIdx.y) * num_ctas;
  const int4 m0 = ws.meta[(rec_base + b) * 2 + 1];
  const unsigned f0 = unsigned(m0.z);
  if (!(f0 & kValid) || !(f0 & kOpenRight) || (f0 & kOpenLeft)) return;  // block-uniform

  // Find the CTA where the segment ends: the first one after b with a head record.
  if (threadIdx.x == 0) s_last = num_ctas;
  __syncthreads();
  for (int base = b + 1; base < num_ctas; base += kCtaThreads) {
    const int idx = base + threadIdx.x;
    if (idx < num_ctas) {
      const int4 mh = ws.meta[(rec_base + idx) * 2];
      if (unsigned(mh.z) & kValid) atomicMin(&s_last, idx);
    }
    __syncthreads();
    if (s_last < num_ctas) break;  // uniform: s_last was read after the barrier
    __syncthreads();
  }
  const int last = s_last;
  if (last >= num_ctas) return;  // inconsistent workspace; leave the row untouched

  const int lane_g = threadIdx.x & (LPR - 1);
  const int group = threadIdx.x / LPR;
  const int ch = blockIdx.y * CPS + lane_g * VEC;
  const bool lane_on = ch < C;

  // Pieces i = 0 .. K-1: tail[b], tail[b+1] .. tail[last-1], head[last].
  const int K = last - b + 1;
  const int per = (K + GPC - 1) / GPC;
  const int i0 = min(group * per, K);
  const int i1 = min(i0 + per, K);
  Acc<VEC> acc;
  Op::template init<VEC>(acc);
  int cnt = 0;
  for (int i = i0; i < i1; ++i) {
    const int64_t rec = (rec_base + b + i) * 2 + ((i == K - 1) ? 0 : 1);
    Acc<VEC> x;
    const uint32_t* ga = ws.vec + rec * 2 * CPS + lane_g * VEC;
    load_acc<VEC>(ga, ga + CPS, x);
    if (i == i0) acc = x; else Op::template merge<VEC>(acc, x);
    cnt += ws.meta[rec].y;
  }
  uint32_t* pa = s_vec + group * 2 * CPS + lane_g * VEC;
  store_acc<VEC>(pa, pa + CPS, acc);
  if (lane_g == 0) s_cnt[group] = cnt;
  __syncthreads();
  if (group == 0) {
    const int used = (K + per - 1) / per;  // groups that held at least one piece
    for (int g = 1; g < used; ++g) {
      Acc<VEC> x;
      const uint32_t* qa = s_vec + g * 2 * CPS + lane_g * VEC;
      load_acc<VEC>(qa, qa + CPS, x);
      Op::template merge<VEC>(acc, x);
      cnt += s_cnt[g];
    }
    store_out<Op, VEC>(out, arg, m0.x, C, ch, lane_on, acc, cnt, mean);
  }
}

// Rows of empty segments: 0 for sum / mean, (-FLT_MAX, -1) for max.
__global__ void fill_empty_kernel(const int32_t* __restrict__ offsets, float* __restrict__ out,
                                  int32_t* __restrict__ arg, int64_t m, int C, bool is_max) {
  const int64_t total = m * C;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t s = i / C;
    if (offsets[s] == offsets[s + 1]) {
      out[i] = is_max ? -FLT_MAX : 0.f;
      if (is_max) arg[i] = -1;
    }
  }
}

// Expands offsets[m + 1] into one segment id per sorted position.
__global__ void expand_offsets_kernel(const int32_t* __restrict__ offsets, int32_t* __restrict__ sid,
                                      int n, int m) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n) return;
  // Largest s with offsets[s] <= p; empty segments sit at equal offsets and the
  // upper-bound search steps over them.
  int lo = 0, hi = m;  // invariant: offsets[lo] <= p < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(offsets + mid) <= p) lo = mid; else hi = mid;
  }
  sid[p] = lo;
}

// ---- host side ----------------------------------------------------------------

struct Geometry {
  int vec, lpr, cps, num_slabs, gpc, rows_per_cta, rows_per_group, num_ctas;
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

Geometry make_geometry(int64_t n, int C, bool allow_vec4) {
  Geometry g;
  g.vec = (allow_vec4 && C % 4 == 0) ? 4 : 1;
  const int lanes = C / g.vec;
  int lpr = 1;
  while (lpr < lanes && lpr < 32) lpr <<= 1;
  if (g.vec == 1) lpr = (lpr <= 1) ? 1 : (lpr <= 4 ? 4 : 32);
  g.lpr = lpr;
  g.cps = g.lpr * g.vec;
  g.num_slabs = (C + g.cps - 1) / g.cps;
  g.gpc = kCtaThreads / g.lpr;
  int rows = tuning().rows_per_cta;
  rows = int(ceil_div(rows, g.gpc)) * g.gpc;
  g.rows_per_cta = rows;
  g.rows_per_group = rows / g.gpc;
  g.num_ctas = int(ceil_div(n, rows));
  return g;
}

size_t reduce_workspace_bytes(int64_t n, int C) {
  // Sized for the scalar layout too (a caller may pass unaligned pointers).
  size_t best = 0;
  for (int v = 0; v < 2; ++v) {
    Geometry g = make_geometry(n, C, v == 1);
    size_t recs = size_t(g.num_slabs) * g.num_ctas * 2;
    size_t bytes = align_up(recs * 2 * g.cps * sizeof(uint32_t), 256) + recs * sizeof(int4);
    if (bytes > best) best = bytes;
  }
  return best + 256;
}

template <class Op, int VEC, int LPR>
int launch_reduce(const Geometry& g, const float* feats, const int32_t* sid, const int32_t* perm,
                  float* out, int32_t* arg, Workspace ws, int n, int C, bool mean,
                  cudaStream_t stream) {
  dim3 grid(g.num_ctas, g.num_slabs);
  if (perm) {
    segment_reduce_kernel<Op, VEC, LPR, true><<<grid, kCtaThreads, 0, stream>>>(
        feats, sid, perm, out, arg, ws, n, C, g.rows_per_cta, g.rows_per_group, mean);
  } else {
    segment_reduce_kernel<Op, VEC, LPR, false><<<grid, kCtaThreads, 0, stream>>>(
        feats, sid, perm, out, arg, ws, n, C, g.rows_per_cta, g.rows_per_group, mean);
  }
  int st = check_launch("segment_reduce_kernel");
  if (st != TEXB_OK) return st;
  if (g.num_ctas > 1) {
    if (tuning().fixup_pdl) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(kCtaThreads);
      cfg.dynamicSmemBytes = 0;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      cudaError_t e = cudaLaunchKernelEx(&cfg, segment_fixup_kernel<Op, VEC, LPR>, ws, out, arg,
                                         g.num_ctas, C, mean);
      if (e != cudaSuccess)
        return fail(TEXB_ERR_CUDA, "segment_fixup_kernel launch: %s", cudaGetErrorString(e));
    } else {
      segment_fixup_kernel<Op, VEC, LPR><<<grid, kCtaThreads, 0, stream>>>(ws, out, arg,
                                                                           g.num_ctas, C, mean);
    }
    st = check_launch("segment_fixup_kernel");
  }
  return st;
}

template <class Op, int VEC>
int dispatch_lpr(const Geometry& g, const float* feats, const int32_t* sid, const int32_t* perm,
                 float* out, int32_t* arg, Workspace ws, int n, int C, bool mean,
                 cudaStream_t stream) {
  switch (g.lpr) {
    case 1: return launch_reduce<Op, VEC, 1>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
    case 4: return launch_reduce<Op, VEC, 4>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
    case 32: return launch_reduce<Op, VEC, 32>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
    default: break;
  }
  if constexpr (VEC == 4) {
    switch (g.lpr) {
      case 2: return launch_reduce<Op, 4, 2>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
      case 8: return launch_reduce<Op, 4, 8>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
      case 16: return launch_reduce<Op, 4, 16>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
      default: break;
    }
  }
  return fail(TEXB_ERR_UNSUPPORTED, "no kernel for %d lanes per row", g.lpr);
}

template <class Op>
int dispatch_vec(const Geometry& g, const float* feats, const int32_t* sid, const int32_t* perm,
                 float* out, int32_t* arg, Workspace ws, int n, int C, bool mean,
                 cudaStream_t stream) {
  if (g.vec == 4) return dispatch_lpr<Op, 4>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
  return dispatch_lpr<Op, 1>(g, feats, sid, perm, out, arg, ws, n, C, mean, stream);
}

}  // namespace

int segment_reduce_impl(int op, const float* feats, const int32_t* sid, const int32_t* perm,
                        const int32_t* offsets, int has_empty, int64_t n, int C, int64_t m,
                        float* out, int32_t* arg, void* workspace, size_t workspace_bytes,
                        cudaStream_t stream) {
  if (op != TEXB_OP_SUM && op != TEXB_OP_MEAN && op != TEXB_OP_MAX)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", op);
  if (n < 0 || m < 0 || C < 1)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "bad sizes n=%lld channel=%d num_segments=%lld",
                (long long)n, C, (long long)m);
  if (n >= (int64_t(1) << 31) || m >= (int64_t(1) << 31))
    return fail(TEXB_ERR_UNSUPPORTED, "n and num_segments must be below 2^31");
  if (m > 0 && !out) return fail(TEXB_ERR_INVALID_ARGUMENT, "out is NULL");
  if (m > 0 && op == TEXB_OP_MAX && !arg) return fail(TEXB_ERR_INVALID_ARGUMENT, "arg is NULL");
  if (n > 0 && (!feats || !sid)) return fail(TEXB_ERR_INVALID_ARGUMENT, "feats or sid is NULL");
  if (has_empty && !offsets)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "offsets is required when has_empty is set");
  if (m == 0) return TEXB_OK;

  if (has_empty || n == 0) {
    int64_t total = m * C;
    int blocks = int(ceil_div(total, 256) < 148 * 16 ? ceil_div(total, 256) : 148 * 16);
    if (n == 0 && !offsets) {
      return fail(TEXB_ERR_INVALID_ARGUMENT, "offsets is required when n == 0");
    }
    fill_empty_kernel<<<blocks, 256, 0, stream>>>(offsets, out, arg, m, C, op == TEXB_OP_MAX);
    int st = check_launch("fill_empty_kernel");
    if (st != TEXB_OK || n == 0) return st;
  }

  const bool vec_ok = aligned16(feats) && aligned16(out) && (op != TEXB_OP_MAX || aligned16(arg));
  Geometry g = make_geometry(n, C, vec_ok);
  const size_t recs = size_t(g.num_slabs) * g.num_ctas * 2;
  const size_t vec_bytes = align_up(recs * 2 * g.cps * sizeof(uint32_t), 256);
  const size_t need = vec_bytes + recs * sizeof(int4);
  uintptr_t base = align_up(reinterpret_cast<uintptr_t>(workspace), 256);
  size_t pad = base - reinterpret_cast<uintptr_t>(workspace);
  if (!workspace || workspace_bytes < need + pad)
    return fail(TEXB_ERR_WORKSPACE, "reduce workspace: need %zu bytes, got %zu", need + pad,
                workspace_bytes);
  Workspace ws;
  ws.vec = reinterpret_cast<uint32_t*>(base);
  ws.meta = reinterpret_cast<int4*>(base + vec_bytes);

  const bool mean = (op == TEXB_OP_MEAN);
  if (op == TEXB_OP_MAX)
    return dispatch_vec<OpMax>(g, feats, sid, perm, out, arg, ws, int(n), C, false, stream);
  if (tuning().compensated)
    return dispatch_vec<OpSumComp>(g, feats, sid, perm, out, arg, ws, int(n), C, mean, stream);
  return dispatch_vec<OpSumPlain>(g, feats, sid, perm, out, arg, ws, int(n), C, mean, stream);
}

int expand_offsets_impl(const int32_t* offsets, int32_t* sid, int64_t n, int64_t m,
                        cudaStream_t stream) {
  if (n == 0) return TEXB_OK;
  expand_offsets_kernel<<<unsigned(ceil_div(n, 256)), 256, 0, stream>>>(offsets, sid, int(n), int(m));
  return check_launch("expand_offsets_kernel");
}

size_t reduce_workspace_bytes_impl(int64_t n, int C) { return reduce_workspace_bytes(n, C); }

}  // namespace texb
