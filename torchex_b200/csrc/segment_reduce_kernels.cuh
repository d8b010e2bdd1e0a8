#pragma once
// Forward segment reduction (sum / mean / max+argmax) for sm_100a.
//
// Work is split by ROWS of the segment-sorted order, never by segments, so a
// 100 000-row segment and 100 000 one-row segments cost the same:
//
//   * a CTA owns a range of consecutive sorted positions (by default the rows are
//     divided over exactly one resident wave of CTAs, cut by the plan's balance
//     table so that every group gets the same estimated cost); inside it
//     every "group" of LPR lanes (LPR * VEC channels wide, one 128-bit access per
//     lane when VEC == 4) owns a consecutive sub-range and walks it row by row,
//     keeping one running accumulator per channel;
//   * a segment that starts and ends inside a group's sub-range is written
//     straight to `out`; a run that touches the edge of the sub-range is kept,
//     and one group then stitches the CTA's edge runs in position order
//     (segments that live inside one CTA finish here);
//   * runs that cross a CTA edge go to a small workspace (two records per CTA)
//     and the fix-up kernel stitches those chains, again in position order.
//
// Two walkers share that skeleton.  The staged kernel (fp32 or bf16 rows of 16 or
// 32 sixteen-byte lanes) streams rows into a ring in shared memory with bulk
// copies (or cp.async), batches ahead of the batch being reduced; the register
// kernel (every other layout) keeps eight row loads in flight in registers.
// Both are programmatic dependent launches, as is the fix-up kernel, so in a
// sequence of reductions each grid is placed while the previous one drains.
//
// Sums carry an error-free compensation term (TwoSum) through every add and
// every merge, so a 175 000-row segment stays within a few ulp of the exact sum.
// The combination order depends only on the geometry, so results are
// bit-reproducible, and no floating-point atomic is used anywhere.
//
// Replaces scatter_sum / scatter_max and their launchers in
// torchex/src/scatter/scatter_kernel.cu:102-192, whose block shape is sized
// from the largest segment and whose lanes run along rows (4-byte loads at a
// stride of C * 4 bytes).

#include <cuda_bf16.h>

#include <cfloat>
#include <atomic>
#include <cstdio>
#include <mutex>

#include "common.cuh"

// Build-time shape of the staged walker's inner loops (override with -D to experiment).
//
// TEXB_SLOW_UNROLL: rows of a batch WITH run ends that are expanded inline per trip.
//   Every expanded row carries its own copy of the code that closes a run (the
//   division for the mean, the stores, the parking of an edge run).  Expanded
//   eight times that code no longer fits the instruction cache: the bf16 kernel
//   ran at an 80-86 % instruction-cache hit rate and 134 / 182 us (sum / mean)
//   on 1 M skewed rows; expanded twice the same kernel takes 105 / 113 us and
//   the fp32 kernels are unchanged to within noise.
// TEXB_FAST_UNROLL: rows of a batch WITHOUT run ends expanded inline (no such code).
// TEXB_PACKED_F32X2: TwoSum on channel pairs with the packed fp32x2 instructions
//   (bit-identical to the scalar form; 1 M skewed rows: bf16 sum 81.5 -> 75.1 us,
//   fp32 sum 97.7 -> 96.0 us, 500 k rows of short segments 59.1 -> 55.7 us).
#ifndef TEXB_SLOW_UNROLL
#define TEXB_SLOW_UNROLL 2
#endif
#ifndef TEXB_FAST_UNROLL
#define TEXB_FAST_UNROLL 8
#endif
#ifndef TEXB_PACKED_F32X2
#define TEXB_PACKED_F32X2 1
#endif

// TEXB_BF16_PACKED_MAX: 1 = the maximum of bf16 rows works on packed bf16 pairs (OpMaxBf16).
#ifndef TEXB_BF16_PACKED_MAX
#define TEXB_BF16_PACKED_MAX 1
#endif

#include <type_traits>

#include "reduce_ops.cuh"

namespace texb {
namespace reduce_detail {


constexpr unsigned kValid = 1u;
constexpr unsigned kOpenLeft = 2u;   // segment began before this range
constexpr unsigned kOpenRight = 4u;  // segment continues after this range

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
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<uint2*>(p) = make_uint2(v[0], v[1]);
  } else if constexpr (VEC == 8) {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(v[4], v[5], v[6], v[7]);
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
  } else if constexpr (VEC == 2) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = t.x; v[1] = t.y;
  } else if constexpr (VEC == 8) {
    const uint4 t = reinterpret_cast<const uint4*>(p)[0], u = reinterpret_cast<const uint4*>(p)[1];
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    v[4] = u.x; v[5] = u.y; v[6] = u.z; v[7] = u.w;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = p[k];
  }
}

// A state in memory: Op::kPlanes arrays ("planes") of `stride` words, this lane's VEC words at p.
template <class Op, int VEC>
__device__ __forceinline__ void store_state(uint32_t* p, int stride,
                                            const typename Op::template State<VEC>& x) {
  uint32_t w[Op::kPlanes][VEC];
  Op::template pack<VEC>(x, w);
#pragma unroll
  for (int pl = 0; pl < Op::kPlanes; ++pl) store_words<VEC>(p + pl * stride, w[pl]);
}

template <class Op, int VEC>
__device__ __forceinline__ void load_state(const uint32_t* p, int stride,
                                           typename Op::template State<VEC>& x) {
  uint32_t w[Op::kPlanes][VEC];
#pragma unroll
  for (int pl = 0; pl < Op::kPlanes; ++pl) load_words<VEC>(p + pl * stride, w[pl]);
  Op::template unpack<VEC>(x, w);
}

// Where results go besides the pointers: the offset added to reported rows and the
// number of output rows, against which every segment id is checked before a store.
struct OutSpec {
  int arg_base;
  int num_segments;
  float* out_sum;  // sum / mean rows of the two-output operator (its maxima go to `out`); else unused
};

// Number of indices found outside their range (a row of `perm` outside [0, n), a
// segment id outside [0, num_segments), a cut of the balance table outside [0, n]).
// Such an index comes from a corrupt plan; the access is skipped and counted here
// (sticky; read with texb_device_status) instead of faulting the GPU.
static __device__ int g_bad_indices = 0;

template <int VEC>
__device__ __forceinline__ void store_row(float* po, const float (&r)[VEC]) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4*>(po) = make_float4(r[0], r[1], r[2], r[3]);
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2*>(po) = make_float2(r[0], r[1]);
  } else if constexpr (VEC == 8) {
    reinterpret_cast<float4*>(po)[0] = make_float4(r[0], r[1], r[2], r[3]);
    reinterpret_cast<float4*>(po)[1] = make_float4(r[4], r[5], r[6], r[7]);
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) po[k] = r[k];
  }
}

// Writes one finished segment row.  `ch` is this lane's first channel.
template <class Op, int VEC>
__device__ __forceinline__ void store_out(float* __restrict__ out, int32_t* __restrict__ arg,
                                       int seg, int C, int ch, bool lane_on,
                                       const typename Op::template State<VEC>& x, int cnt, bool mean,
                                       OutSpec ospec) {
  if (unsigned(seg) >= unsigned(ospec.num_segments)) {
    if (ch == 0) atomicAdd(&g_bad_indices, 1);
    return;
  }
  if (!lane_on) return;
  if constexpr (Op::kHasSum) {  // sum or mean row: to `out`, or beside the maxima of the two-output operator
    float r[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = Op::template sum_value<VEC>(x, k);
    if (mean) divide_by_count<VEC>(r, cnt);
    store_row<VEC>((Op::kIsMax ? ospec.out_sum : out) + int64_t(seg) * C + ch, r);
  }
  if constexpr (Op::kIsMax) {
    float r[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = Op::template value<VEC>(x, k);
    store_row<VEC>(out + int64_t(seg) * C + ch, r);
  }
  if constexpr (Op::kIsMax) {
    int32_t* pa = arg + int64_t(seg) * C + ch;
    int ix[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {  // rows are reported relative to ospec; "no row" stays -1
      const int i = Op::template index<VEC>(x, k);
      ix[k] = i < 0 ? i : i + ospec.arg_base;
    }
    if constexpr (VEC == 4) {
      *reinterpret_cast<int4*>(pa) = make_int4(ix[0], ix[1], ix[2], ix[3]);
    } else if constexpr (VEC == 2) {
      *reinterpret_cast<int2*>(pa) = make_int2(ix[0], ix[1]);
    } else if constexpr (VEC == 8) {
      reinterpret_cast<int4*>(pa)[0] = make_int4(ix[0], ix[1], ix[2], ix[3]);
      reinterpret_cast<int4*>(pa)[1] = make_int4(ix[4], ix[5], ix[6], ix[7]);
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) pa[k] = ix[k];
    }
  }
}

// A segment of exactly one row: sum and mean are the row itself; max goes through
// the operator so that NaN / -inf rows keep the (-FLT_MAX, -1) answer.
template <class Op, int VEC>
__device__ __forceinline__ void store_single(float* __restrict__ out, int32_t* __restrict__ arg, int seg,
                                             int C, int ch, bool lane_on, const float (&v)[VEC], int row, OutSpec ospec) {
  if constexpr (Op::kIsMax) {
    typename Op::template State<VEC> x;
    Op::template init<VEC>(x);
    Op::template add<VEC>(x, v, row);
    store_out<Op, VEC>(out, arg, seg, C, ch, lane_on, x, 1, false, ospec);  // a mean over one row is the row
  } else {
    if (unsigned(seg) >= unsigned(ospec.num_segments)) {
      if (ch == 0) atomicAdd(&g_bad_indices, 1);
      return;
    }
    if (!lane_on) return;
    store_row<VEC>(out + int64_t(seg) * C + ch, v);
  }
}

// Workspace: for CTA b and channel slab y there are two records,
// rec = (y * num_ctas + b) * 2 + {0: head, 1: tail}.  A record is CPS words of
// `a`, CPS words of `b` (CPS = LPR * VEC channels per slab) and an int4 of
// meta {sid, row count, flags, 0}.
struct Workspace {
  uint32_t* vec;  // [num_slabs * num_ctas * 2][planes of the operator * CPS]
  int4* meta;     // [num_slabs * num_ctas * 2]
  // Chains finished inside the reduce kernel (see finish_chain_in_kernel): one word per
  // (slab, CTA) that the CTA sets to `epoch` once its records are visible.  `epoch` is
  // different for every launch of the process, so whatever an earlier call (or fresh
  // memory) left in the array never reads as "ready".  NULL: the fix-up kernel runs instead.
  unsigned long long* ready;
  unsigned long long epoch;
};

// Low word of the nanosecond timer.  The last field of a CTA's tail meta records
// when the CTA finished: a diagnostic for the spread of finishing times.
__device__ __forceinline__ unsigned global_timer_lo() {
  unsigned t;
  asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
  return t;
}

// A reduction that did not wait for the stream at its start waits here, when its own work
// is done: its grid then cannot complete before the grid launched just before it has, so the
// reductions of a sequence complete in order and whatever follows them in the stream sees
// all of their results.  The earlier grid started first, so this wait is normally over
// before it begins.
__device__ __forceinline__ void stream_tail_wait(bool no_wait) {
#if __CUDA_ARCH__ >= 900
  if (no_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}

// Stitches the edge runs a CTA left in shared memory.  The valid slots, taken in
// slot order, form chains: a slot that is open to the right is continued by the
// next valid slot.  A chain is folded in position order by the group that owns
// its first slot, so the chains of a CTA (usually one per pair of neighbouring
// groups) are folded side by side and the result does not depend on who folds.
// A chain that closes inside the CTA is a finished segment and goes to `out`;
// the chain that enters from the left edge becomes the CTA's head record, the
// one that leaves through the right edge its tail record.  Every thread of the
// CTA must call this, after a barrier that follows the last slot write.
template <class Op, int VEC, int LPR>
__device__ __forceinline__ bool stitch_cta(const uint32_t* s_vec, const int* s_sid, const int* s_cnt,
                                           const unsigned* s_flag, float* __restrict__ out,
                                           int32_t* __restrict__ arg, Workspace ws, int C, int ch,
                                           bool lane_on, int lane_g, int group, bool mean, OutSpec ospec,
                                           unsigned t_start = 0u) {
  using State = typename Op::template State<VEC>;
  constexpr int GPC = kCtaThreads / LPR;
  constexpr int CPS = LPR * VEC;
  constexpr int SLOTS = 2 * GPC;
  __shared__ int s_first_valid, s_last_valid;
  __shared__ int s_chain_ends_here;  // a chain entered from the left and closed inside this CTA (read by the caller)
  if (threadIdx.x == 0) {
    s_first_valid = SLOTS;
    s_last_valid = -1;
    s_chain_ends_here = 0;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < SLOTS; t += kCtaThreads) {
    if (s_flag[t] & kValid) {
      atomicMin(&s_first_valid, t);
      atomicMax(&s_last_valid, t);
    }
  }
  __syncthreads();
  const int first = s_first_valid, last = s_last_valid;
  const int64_t rec = (int64_t(blockIdx.y) * gridDim.x + blockIdx.x) * 2;
  if (threadIdx.x == 0) {  // records this CTA does not produce are marked empty
    if (first >= SLOTS || !(s_flag[first] & kOpenLeft)) ws.meta[rec] = make_int4(0, 0, 0, int(t_start));
    if (last < 0 || !(s_flag[last] & kOpenRight)) ws.meta[rec + 1] = make_int4(0, 0, 0, int(global_timer_lo()));
  }
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const int slot = 2 * group + which;
    const unsigned f = s_flag[slot];
    if (!(f & kValid)) continue;
    const bool from_left = (f & kOpenLeft) != 0u;
    if (from_left && slot != first) continue;  // part of a chain that an earlier slot starts
    State cur;
    const uint32_t* pa = s_vec + slot * Op::kPlanes * CPS + lane_g * VEC;
    load_state<Op, VEC>(pa, CPS, cur);
    const int cur_sid = s_sid[slot];
    int cur_cnt = s_cnt[slot];
    unsigned fs = f;
    int at = slot;
    bool leaves = false;  // the chain runs past the CTA's right edge
    while (fs & kOpenRight) {
      int t = at + 1;
      while (t < SLOTS && !(s_flag[t] & kValid)) ++t;
      if (t >= SLOTS) {
        leaves = true;
        break;
      }
      State x;
      const uint32_t* pb = s_vec + t * Op::kPlanes * CPS + lane_g * VEC;
      load_state<Op, VEC>(pb, CPS, x);
      Op::template merge<VEC>(cur, x);
      cur_cnt += s_cnt[t];
      fs = s_flag[t];
      at = t;
    }
    if (!leaves && !from_left) {
      store_out<Op, VEC>(out, arg, cur_sid, C, ch, lane_on, cur, cur_cnt, mean, ospec);
    } else if (!leaves) {
      uint32_t* ga = ws.vec + rec * Op::kPlanes * CPS + lane_g * VEC;
      store_state<Op, VEC>(ga, CPS, cur);
      if (lane_g == 0) {
        ws.meta[rec] = make_int4(cur_sid, cur_cnt, int(kValid | kOpenLeft), int(t_start));
        s_chain_ends_here = 1;
      }
    } else {
      uint32_t* ga = ws.vec + (rec + 1) * Op::kPlanes * CPS + lane_g * VEC;
      store_state<Op, VEC>(ga, CPS, cur);
      const unsigned ft = kValid | kOpenRight | (from_left ? kOpenLeft : 0u);
      if (lane_g == 0) {
        ws.meta[rec + 1] = make_int4(cur_sid, cur_cnt, int(ft), int(global_timer_lo()));
        // one run from edge to edge: it is the tail record, and there is no head record
        if (from_left) ws.meta[rec] = make_int4(0, 0, 0, int(t_start));
      }
    }
  }
  __syncthreads();
  return s_chain_ends_here != 0;  // block-uniform: a chain that entered from the left closed in this CTA
}

// ---- finishing the chains -------------------------------------------------------
// A chain is a segment that runs through several CTAs: its pieces are the tail record
// of the CTA where it starts, the tail records of the CTAs it runs through and the
// head record of the CTA where it ends.  merge_chain folds them in position order with
// all the groups of a CTA (four independent record loads in flight per group) and
// writes the row.  It is called either by the fix-up kernel (one CTA per chain start)
// or, when the workspace carries ready flags, by the reduce kernel itself from the CTA
// in which the chain ends.  Records are read around L1 (ld.global.cg): in the reduce
// kernel they were written by other CTAs of the same grid.

__device__ __forceinline__ uint32_t ld_cg_u32(const uint32_t* p) { return __ldcg(p); }

template <int VEC>
__device__ __forceinline__ void load_words_cg(const uint32_t* p, uint32_t (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const uint4 t = __ldcg(reinterpret_cast<const uint4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else if constexpr (VEC == 2) {
    const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
    v[0] = t.x; v[1] = t.y;
  } else if constexpr (VEC == 8) {
    const uint4 t = __ldcg(reinterpret_cast<const uint4*>(p)), u = __ldcg(reinterpret_cast<const uint4*>(p) + 1);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    v[4] = u.x; v[5] = u.y; v[6] = u.z; v[7] = u.w;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = __ldcg(p + k);
  }
}

template <class Op, int VEC>
__device__ __forceinline__ void load_state_cg(const uint32_t* p, int stride, typename Op::template State<VEC>& x) {
  uint32_t w[Op::kPlanes][VEC];
#pragma unroll
  for (int pl = 0; pl < Op::kPlanes; ++pl) load_words_cg<VEC>(p + pl * stride, w[pl]);
  Op::template unpack<VEC>(x, w);
}

// Chain from CTA `first` (its tail record) to CTA `last` (its head record), first < last.
// s_vec / s_cnt: shared scratch of at least GPC states / GPC counts.  Every thread of the CTA calls this.
template <class Op, int VEC, int LPR>
__device__ __forceinline__ void merge_chain(Workspace ws, int64_t rec_base, int first, int last, int seg,
                                            uint32_t* s_vec, int* s_cnt, float* __restrict__ out,
                                            int32_t* __restrict__ arg, int C, int ch, bool lane_on, int lane_g,
                                            int group, bool mean, OutSpec ospec) {
  using State = typename Op::template State<VEC>;
  constexpr int GPC = kCtaThreads / LPR;
  constexpr int CPS = LPR * VEC;
  // Pieces i = 0 .. K-1: tail[first], tail[first+1] .. tail[last-1], head[last].
  const int K = last - first + 1;
  const int per = (K + GPC - 1) / GPC;
  const int i0 = min(group * per, K);
  const int i1 = min(i0 + per, K);
  State acc;
  Op::template init<VEC>(acc);
  int cnt = 0;
  for (int i = i0; i < i1; i += 4) {  // four independent record loads in flight
    State x[4];
    int c4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int ii = min(i + u, i1 - 1);
      const int64_t rec = (rec_base + first + ii) * 2 + ((ii == K - 1) ? 0 : 1);
      const uint32_t* ga = ws.vec + rec * Op::kPlanes * CPS + lane_g * VEC;
      load_state_cg<Op, VEC>(ga, CPS, x[u]);
      c4[u] = __ldcg(&ws.meta[rec]).y;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i + u < i1) {
        if (i + u == i0) acc = x[u]; else Op::template merge<VEC>(acc, x[u]);
        cnt += c4[u];
      }
    }
  }
  uint32_t* pa = s_vec + group * Op::kPlanes * CPS + lane_g * VEC;
  store_state<Op, VEC>(pa, CPS, acc);
  if (lane_g == 0) s_cnt[group] = cnt;
  __syncthreads();
  if (group == 0) {
    const int used = (K + per - 1) / per;  // groups that held at least one piece
    for (int g = 1; g < used; ++g) {
      State x;
      const uint32_t* qa = s_vec + g * Op::kPlanes * CPS + lane_g * VEC;
      load_state<Op, VEC>(qa, CPS, x);
      Op::template merge<VEC>(acc, x);
      cnt += s_cnt[g];
    }
    store_out<Op, VEC>(out, arg, seg, C, ch, lane_on, acc, cnt, mean, ospec);
  }
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

static __device__ int g_wait_timeouts_chain = 0;  // look-backs that gave up (added to texb_device_status' wait_timeouts)

// Polls of one look-back before it gives up (each poll is a trip to L2, and the lanes
// sleep between polls): far longer than any reduce kernel runs, short enough to return.
constexpr int kChainSpins = 1 << 16;

// Called by every thread of a reduce CTA after stitch_cta, when the workspace carries
// ready flags.  The CTA publishes its records; if a chain ends in this CTA (`ends_here`,
// block-uniform) it then finds where the chain starts by looking back over the CTAs to
// its left -- waiting, with a limit, for each one to publish -- and folds the chain.
// Waits only ever point to CTAs with a lower index, which the hardware dispatches no
// later than this one, so they are resident or finished; should a wait run out anyway,
// the event is counted, the row is left unwritten and the kernel returns.
template <class Op, int VEC, int LPR>
__device__ __forceinline__ void finish_chain_in_kernel(Workspace ws, bool ends_here, uint32_t* s_vec, int* s_cnt,
                                                       float* __restrict__ out, int32_t* __restrict__ arg, int C,
                                                       int ch, bool lane_on, int lane_g, int group, bool mean,
                                                       OutSpec ospec) {
  __shared__ int s_chain_first;
  const int b = blockIdx.x, num_ctas = gridDim.x;
  const int64_t rec_base = int64_t(blockIdx.y) * num_ctas;
  __threadfence();  // this thread's record words are visible device-wide before the flag is
  __syncthreads();
  if (threadIdx.x == 0) {
    st_release_u64(ws.ready + rec_base + b, ws.epoch);
    s_chain_first = -1;
  }
  if (!ends_here) return;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int first = -1;
    bool gave_up = false;
    for (int base = b - 1; base >= 0 && first < 0 && !gave_up; base -= 32) {
      const int j = base - lane;
      int state = (j < 0) ? 2 : 0;  // 0: not published yet, 1: the chain runs through CTA j, 2: it starts there (or cannot go further)
      int it = 0;
      for (; it < kChainSpins; ++it) {
        if (state == 0 && ld_acquire_u64(ws.ready + rec_base + j) == ws.epoch) {
          const unsigned f = unsigned(__ldcg(&ws.meta[(rec_base + j) * 2 + 1]).z);
          state = ((f & kValid) && (f & kOpenRight) && (f & kOpenLeft)) ? 1 : 2;
        }
        const unsigned known = __ballot_sync(0xffffffffu, state != 0);
        const unsigned starts = __ballot_sync(0xffffffffu, state == 2);
        if (starts) {
          const int p = __ffs(starts) - 1;  // nearest CTA where the chain can start
          const unsigned upto = (p == 31) ? 0xffffffffu : ((2u << p) - 1u);
          if ((known & upto) == upto) {     // and everything nearer is known to be run through
            first = base - p;
            break;
          }
        } else if (known == 0xffffffffu) {
          break;  // all 32 are run through: look further back
        }
        __nanosleep(100);
      }
      if (it >= kChainSpins) gave_up = true;
    }
    if (lane == 0) {
      if (gave_up) atomicAdd(&g_wait_timeouts_chain, 1);
      s_chain_first = gave_up ? -1 : first;
    }
  }
  __syncthreads();
  const int first = s_chain_first;
  if (first < 0 || first >= b) return;  // gave up, or an inconsistent workspace: leave the row untouched
  const unsigned f0 = unsigned(__ldcg(&ws.meta[(rec_base + first) * 2 + 1]).z);
  if (!(f0 & kValid) || !(f0 & kOpenRight) || (f0 & kOpenLeft)) return;  // block-uniform
  const int seg = __ldcg(&ws.meta[(rec_base + b) * 2]).x;
  merge_chain<Op, VEC, LPR>(ws, rec_base, first, b, seg, s_vec, s_cnt, out, arg, C, ch, lane_on, lane_g, group, mean,
                            ospec);
}

// Range of sorted positions walked by one group.  With a balance table (K + 1
// increasing positions that cut the rows into K pieces of equal estimated cost,
// built with the plan) group gi of G takes pieces [gi K / G, (gi + 1) K / G);
// without one the rows are cut evenly: rows_per_cta per CTA, rows_per_group per group.
struct Split {
  const int32_t* balance;  // NULL: even split
  int balance_k;
  int stream_hint;         // 1: feature rows are copied with an L2 evict-first policy
  int plan_settled;        // 1: the plan arrays may be read before the stream's earlier work is visible
  int no_wait;             // 1: a later reduction of a back-to-back sequence: nothing is waited for at the start
  int rows_per_cta, rows_per_group, num_ctas;
};

__device__ __forceinline__ void group_range(const Split& sp, int n, int group, int gpc, int& g0, int& g1) {
  if (sp.balance) {
    const long long gi = (long long)blockIdx.x * gpc + group;
    const long long G = (long long)gridDim.x * gpc;
    g0 = __ldg(sp.balance + int(gi * sp.balance_k / G));
    g1 = __ldg(sp.balance + int((gi + 1) * sp.balance_k / G));
  } else {
    const int c0 = blockIdx.x * sp.rows_per_cta;
    const int c1 = min(c0 + sp.rows_per_cta, n);
    g0 = min(c0 + group * sp.rows_per_group, c1);
    g1 = min(g0 + sp.rows_per_group, c1);
  }
  // cuts of a corrupt balance table are pulled back into [0, n], in order
  const int lo = min(max(g0, 0), n), hi = min(max(g1, lo), n);
  if ((lo != g0 || hi != g1) && (threadIdx.x & 31) == 0) atomicAdd(&g_bad_indices, 1);
  g0 = lo;
  g1 = hi;
}

// ---- register kernel ------------------------------------------------------------

template <class Op, int VEC, int LPR, bool HAS_PERM>
__global__ void __launch_bounds__(kCtaThreads)
segment_reduce_kernel(const float* __restrict__ feats, const int32_t* __restrict__ sid,
                      const int32_t* __restrict__ perm, float* __restrict__ out,
                      int32_t* __restrict__ arg, Workspace ws, int n, int C,
                      Split sp, bool mean, OutSpec ospec) {
  using State = typename Op::template State<VEC>;
  constexpr int GPC = kCtaThreads / LPR;           // groups per CTA
  constexpr int CPS = LPR * VEC;                   // channels per slab
  constexpr int U = (LPR >= 8) ? 8 : LPR;          // row loads in flight per group
  constexpr int SLOTS = 2 * GPC;

  __shared__ __align__(16) uint32_t s_vec[SLOTS * Op::kPlanes * CPS];
  __shared__ int s_sid[SLOTS];
  __shared__ int s_cnt[SLOTS];
  __shared__ unsigned s_flag[SLOTS];

#if __CUDA_ARCH__ >= 900
  // Let the dependent fix-up grid be scheduled now (it parks at its own
  // griddepcontrol.wait until this grid has finished); a no-op for a plain launch.
  // This grid may itself be a dependent launch of whatever kernel precedes it in
  // the stream (typically the fix-up of the previous reduction): its CTAs are then
  // placed while that kernel drains, and the wait below holds them until all of
  // its memory operations are visible, before anything is read.
  // A later reduction of a back-to-back sequence (sp.no_wait) does not wait: everything it
  // reads was complete before the first reduction of the sequence let its dependents start,
  // and it writes only buffers of its own.  It waits at its END instead (see stream_tail_wait).
  if (!sp.no_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
  const int lane_g = threadIdx.x & (LPR - 1);
  const int group = threadIdx.x / LPR;
  const unsigned gmask =
      (LPR == 32) ? 0xffffffffu
                  : (((1u << LPR) - 1u) << ((threadIdx.x & 31) & ~(LPR - 1)));
  const int ch = blockIdx.y * CPS + lane_g * VEC;  // first channel of this lane
  const bool lane_on = ch < C;                     // VEC == 4 implies C % 4 == 0

  int g0, g1;
  group_range(sp, n, group, GPC, g0, g1);

  if (lane_g == 0) {
    s_flag[2 * group] = 0u;
    s_flag[2 * group + 1] = 0u;
  }

  if (g0 < g1) {
    int cur_sid = __ldg(sid + g0);
    const bool first_open_left = (g0 > 0) && (__ldg(sid + g0 - 1) == cur_sid);
    bool is_first = true;
    int cnt = 0;
    State acc;
    Op::template init<VEC>(acc);

    // Ends the current run.  open_right is only ever true for the last run.
    auto close_run = [&](bool open_right) {
      const bool open_left = is_first && first_open_left;
      if (!open_left && !open_right) {
        store_out<Op, VEC>(out, arg, cur_sid, C, ch, lane_on, acc, cnt, mean, ospec);
      } else {
        const int slot = 2 * group + (open_right ? 1 : 0);
        uint32_t* pa = s_vec + slot * Op::kPlanes * CPS + lane_g * VEC;
        store_state<Op, VEC>(pa, CPS, acc);
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
        if (HAS_PERM && unsigned(my_row) >= unsigned(n)) {  // corrupt plan: read row 0 instead, and say so
          my_row = 0;
          atomicAdd(&g_bad_indices, 1);
        }
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
  const bool ends_here = stitch_cta<Op, VEC, LPR>(s_vec, s_sid, s_cnt, s_flag, out, arg, ws, C, ch, lane_on, lane_g,
                                                  group, mean, ospec);
  if (ws.ready)
    finish_chain_in_kernel<Op, VEC, LPR>(ws, ends_here, s_vec, s_cnt, out, arg, C, ch, lane_on, lane_g, group, mean,
                                         ospec);
  stream_tail_wait(sp.no_wait != 0);
}

// ---- staged kernel --------------------------------------------------------------
// Rows of 64..128 fp32 channels per slab (LPR 16 or 32, 128-bit lanes).  Rows are
// not loaded into registers: every lane streams its own 16 bytes of each row into
// a private ring in shared memory with cp.async (L2 -> shared, bypassing L1 and
// the register file), two batches of eight rows ahead of the batch being reduced.
// A lane only ever reads back bytes it copied itself, so the ring needs no
// barrier: cp.async.wait_group on the lane's own copy groups is the only
// synchronisation.  Run ends come from one ballot per 32-position tile; a batch
// without a run end takes a branch-free path of eight shared-memory loads and
// accumulations.

__device__ __forceinline__ void cp_async_16(unsigned smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Bulk (TMA) copy of one row slab, global -> this CTA's shared memory, signalling
// an mbarrier with the byte count.  One destination CTA only; the source is always this
// GPU's own memory.  Source, destination and size are multiples of 16 bytes.
// `policy` is an L2 eviction policy.  Feature rows are read exactly once, so an
// evict-first policy is the textbook choice and is available as a knob; measured
// on the three-reduction step it loses to the normal policy (0.319 vs 0.300 ms),
// so the normal policy is the default.
__device__ __forceinline__ void bulk_copy_g2s(unsigned smem_dst, const void* gmem_src, unsigned bytes,
                                              unsigned bar, unsigned long long policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ unsigned long long l2_policy(bool evict_first) {
  unsigned long long p;
  if (evict_first) {
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  } else {
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  }
  return p;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// TEXB_WAIT_HINT_NS: upper bound, in nanoseconds, that one mbarrier.try_wait may keep the
//   warp suspended before it reports "not yet" (0: the hardware's own default limit).
// TEXB_WAIT_SLEEP_NS: nanoseconds a warp sleeps between two unsuccessful polls (0: none).
// A waiting warp that polls less often leaves its issue slots to the warps that compute.
#ifndef TEXB_WAIT_HINT_NS
#define TEXB_WAIT_HINT_NS 0
#endif
#ifndef TEXB_WAIT_SLEEP_NS
#define TEXB_WAIT_SLEEP_NS 0
#endif

__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
#if TEXB_WAIT_HINT_NS > 0
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(unsigned(TEXB_WAIT_HINT_NS)) : "memory");
#else
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#endif
  return ok != 0u;
}

// Number of bounded waits that gave up (sticky; read with texb_device_status).
static __device__ int g_wait_timeouts = 0;

// Waits for a phase of an mbarrier, at most kWaitSpins polls (each poll itself
// blocks for a bounded, hardware-defined time).  On expiry the event is counted
// and the caller carries on with whatever the ring holds: the result is wrong
// but the kernel returns and the context stays usable.
constexpr int kWaitSpins = 1 << 20;
__device__ __forceinline__ void mbar_wait_bounded(unsigned bar, unsigned parity) {
  for (int it = 0; it < kWaitSpins; ++it) {
    if (mbar_try_wait(bar, parity)) return;
#if TEXB_WAIT_SLEEP_NS > 0
    __nanosleep(TEXB_WAIT_SLEEP_NS);
#endif
  }
  atomicAdd(&g_wait_timeouts, 1);
}

constexpr int kStageBatch = 8;    // rows per copy batch
constexpr int kStageTile = 32;    // positions per metadata tile
// A lane owns LB bytes of every row: 16 (4 fp32 or 8 bf16 channels) or 8 (4 bf16
// channels, so that a 128-channel bf16 row spans a whole warp like its fp32 twin).
// Batches in the ring: fp32 rows three (two in flight, one being reduced); bf16
// rows with 16-byte lanes carry eight channels per lane, which doubles the shared
// memory of the edge-run slots, so their ring has two batches to keep two CTAs per
// SM; bf16 rows with 8-byte lanes are half as wide, and three batches (48 KB) let
// three CTAs share an SM (measured: 82 us against 92 us with four batches and two CTAs).
// The two-output operator's edge-run slots are twice as large (four planes), so
// its fp32 ring has two batches, again to keep two CTAs per SM.
template <class In, int LB, int PLANES>
constexpr int kStageDepthFor = (LB == 8) ? (PLANES == 2 ? 3 : 4) : (sizeof(In) == 4) ? (PLANES == 2 ? 3 : 2) : 2;
template <int LB> constexpr int kStageSlotBytesFor = kCtaThreads * LB;  // one row slot for the whole CTA
template <class In, int LB, int PLANES>
constexpr int kStageRingBytesFor = kStageBatch * kStageDepthFor<In, LB, PLANES> * kStageSlotBytesFor<LB>;

template <int LB> struct LaneWord;
template <> struct LaneWord<16> { using type = float4; };
template <> struct LaneWord<8> { using type = float2; };

// The bytes a lane owns of a row, as fp32 channels.
template <class In, int VEC>
__device__ __forceinline__ void unpack_lane(const float4& t4, float (&v)[VEC]) {
  if constexpr (sizeof(In) == 4) {
    v[0] = t4.x; v[1] = t4.y; v[2] = t4.z; v[3] = t4.w;
  } else {
    const unsigned w[4] = {__float_as_uint(t4.x), __float_as_uint(t4.y), __float_as_uint(t4.z), __float_as_uint(t4.w)};
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // a bf16 is the upper half of the fp32 with the same value
      v[2 * k] = __uint_as_float(w[k] << 16);
      v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}
template <class In, int VEC>
__device__ __forceinline__ void unpack_lane(const float2& t2, float (&v)[VEC]) {
  if constexpr (sizeof(In) == 4) {  // 8-byte lanes: two fp32 channels
    static_assert(VEC == 2, "8-byte lanes hold two fp32 channels");
    v[0] = t2.x; v[1] = t2.y;
  } else {                          // or four bf16 channels
    static_assert(VEC == 4, "8-byte lanes hold four bf16 channels");
    const unsigned w[2] = {__float_as_uint(t2.x), __float_as_uint(t2.y)};
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      v[2 * k] = __uint_as_float(w[k] << 16);
      v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}

// Adds one row (the bytes this lane owns of it) to the running state.  An operator that
// works on packed bf16 pairs takes them as they are; the others get fp32 channels.
template <class Op, class In, int VEC, class State>
__device__ __forceinline__ void accumulate_lane(State& acc, const float4& t4, int row) {
  if constexpr (Op::kRawBf16 && sizeof(In) == 2) {
    static_assert(VEC == 8, "16-byte lanes hold eight bf16 channels");
    const uint32_t w[4] = {__float_as_uint(t4.x), __float_as_uint(t4.y), __float_as_uint(t4.z), __float_as_uint(t4.w)};
    Op::template add_raw<VEC>(acc, w, row);
  } else {
    float v[VEC];
    unpack_lane<In, VEC>(t4, v);
    Op::template add<VEC>(acc, v, row);
  }
}
template <class Op, class In, int VEC, class State>
__device__ __forceinline__ void accumulate_lane(State& acc, const float2& t2, int row) {
  if constexpr (Op::kRawBf16 && sizeof(In) == 2) {
    static_assert(VEC == 4, "8-byte lanes hold four bf16 channels");
    const uint32_t w[2] = {__float_as_uint(t2.x), __float_as_uint(t2.y)};
    Op::template add_raw<VEC>(acc, w, row);
  } else {
    float v[VEC];
    unpack_lane<In, VEC>(t2, v);
    Op::template add<VEC>(acc, v, row);
  }
}

// Resident CTAs per SM the staged kernel is compiled for: three where the ring and
// the edge-run slots leave room (bf16 rows on 8-byte lanes, single-output operators),
// otherwise two.  (8-byte lanes: bf16 rows of up to 128 channels, fp32 rows of up to 64.)
template <class Op, class In, int LB>
constexpr int kStagedCtasPerSm = (LB == 8 && Op::kPlanes == 2) ? 3 : 2;

template <class Op, class In, int LB, int LPR, bool HAS_PERM, bool BULK>
__global__ void __launch_bounds__(kCtaThreads, kStagedCtasPerSm<Op, In, LB>)
segment_reduce_staged_kernel(const In* __restrict__ feats, const int32_t* __restrict__ sid,
                             const int32_t* __restrict__ perm, float* __restrict__ out,
                             int32_t* __restrict__ arg, Workspace ws, int n, int C,
                             Split sp, bool mean, OutSpec ospec) {
  constexpr int VEC = LB / sizeof(In);  // channels in the bytes a lane owns: 4 fp32, 8 or 4 bf16
  using State = typename Op::template State<VEC>;
  using Word = typename LaneWord<LB>::type;
  constexpr int GPC = kCtaThreads / LPR;
  constexpr int CPS = LPR * VEC;
  constexpr int SLOTS = 2 * GPC;
  constexpr int B = kStageBatch, S = kStageDepthFor<In, LB, Op::kPlanes>, T = kStageTile;
  constexpr int kStageSlotBytes = kStageSlotBytesFor<LB>;
  static_assert(BULK || LB == 16, "the cp.async ring copies 16 bytes per lane");
  constexpr int NREG = T / LPR;  // tile positions held per lane
  static_assert(LPR == 16 || LPR == 32, "staged kernel handles 16 or 32 lanes per row");
  static_assert(S >= 2 && (S - 1) * B <= T && T % B == 0 && LPR % B == 0, "the copy front must stay within two tiles");

  extern __shared__ __align__(16) unsigned char s_dyn[];  // the ring
  __shared__ __align__(16) uint32_t s_vec[SLOTS * Op::kPlanes * CPS];  // edge runs of the groups
  __shared__ int s_sid[SLOTS];
  __shared__ int s_cnt[SLOTS];
  __shared__ unsigned s_flag[SLOTS];
  __shared__ __align__(8) unsigned long long s_bar[BULK ? GPC * S : 1];  // one mbarrier per (group, stage)

  // This grid may be a programmatic dependent launch of whatever kernel precedes it in
  // the stream (typically the fix-up of the previous reduction): its CTAs are then
  // placed while that kernel drains, and memory written by earlier work of the stream
  // is only guaranteed to be visible after griddepcontrol.wait.  By default the wait
  // therefore comes first, before anything is read.  When the caller states that the
  // plan is settled (its arrays were complete and the host had synchronised with the
  // stream before this launch), the prologue that reads only the plan (sid, perm,
  // balance) and writes only this CTA's shared memory runs ahead of the wait, under
  // the tail of the previous kernel; the features are read and global memory is
  // written after it either way.  A no-op for a plain launch.
  bool waited = false;
  const bool no_wait = sp.no_wait != 0;
  auto wait_for_stream = [&waited, no_wait] {
    if (waited) return;
    waited = true;
#if __CUDA_ARCH__ >= 900
    // A later reduction of a back-to-back sequence does not wait here (see stream_tail_wait).
    if (!no_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
    // Let the dependent grid be scheduled now (a fix-up parks at its own wait until this
    // grid has finished; the next reduction of a sequence starts as this grid's CTAs retire).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
  };
  if (!sp.plan_settled || no_wait) wait_for_stream();
  const unsigned t_start = global_timer_lo();
  const int lane_g = threadIdx.x & (LPR - 1);
  const int group = threadIdx.x / LPR;
  const int lane_base = (threadIdx.x & 31) & ~(LPR - 1);  // first lane of the group
  const unsigned gmask = (LPR == 32) ? 0xffffffffu : (((1u << LPR) - 1u) << lane_base);
  const int ch = blockIdx.y * CPS + lane_g * VEC;
  const bool lane_on = ch < C;

  int g0, g1;
  group_range(sp, n, group, GPC, g0, g1);

  if (lane_g == 0) {
    s_flag[2 * group] = 0u;
    s_flag[2 * group + 1] = 0u;
  }
  if constexpr (BULK) {
    if (lane_g == 0) {
#pragma unroll
      for (int st = 0; st < S; ++st)
        mbar_init(unsigned(__cvta_generic_to_shared(&s_bar[group * S + st])), 1u);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }

  if (g0 < g1) {
    const int L = g1 - g0;
    const int nb = (L + B - 1) / B;
    // Inactive lanes (channel tail of the last slab) copy channel 0 instead of
    // branching around every access; their results are never stored.
    const In* lane_src = feats + (lane_on ? ch : 0);
    // cp.async layout: slot s of the CTA at s * kStageSlotBytes, lane t at + 16 t.
    // Bulk layout: each group owns S * B consecutive row slabs of kRowBytes.
    constexpr int kRowBytes = LPR * LB;
    constexpr int kSlotFloat4 = BULK ? LPR : kCtaThreads;  // stride between slots, in lane words
    const int row_bytes = min(CPS, C - blockIdx.y * CPS) * int(sizeof(In));  // the last slab may be narrower
    const unsigned ring_addr = BULK
        ? unsigned(__cvta_generic_to_shared(s_dyn)) + unsigned(group * S * B) * kRowBytes
        : unsigned(__cvta_generic_to_shared(s_dyn)) + threadIdx.x * 16;
    const Word* ring = BULK
        ? reinterpret_cast<const Word*>(s_dyn) + group * S * B * LPR + lane_g
        : reinterpret_cast<const Word*>(s_dyn) + threadIdx.x;
    const unsigned bar0 = unsigned(__cvta_generic_to_shared(&s_bar[BULK ? group * S : 0]));
    const In* slab_src = feats + blockIdx.y * CPS;
    const unsigned long long stream_policy = BULK ? l2_policy(sp.stream_hint != 0) : 0ull;

    // Tile metadata: lane_g holds positions t * T + r * LPR + lane_g (r < NREG).
    int cur_sid_r[NREG], cur_row_r[NREG], nxt_sid_r[NREG], nxt_row_r[NREG];
    unsigned cur_mask = 0u, nxt_mask = 0u;  // bit j: position j of the tile ends a run
    auto load_tile = [&](int t, int (&m_sid)[NREG], int (&m_row)[NREG], unsigned& m_mask) {
      m_mask = 0u;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int p = g0 + t * T + r * LPR + lane_g;
        const bool in = p < g1;
        m_sid[r] = in ? __ldg(sid + p) : -1;
        const int nxt = (in && p + 1 < n) ? __ldg(sid + p + 1) : -2;
        m_row[r] = HAS_PERM ? (in ? __ldg(perm + p) : 0) : p;
        if (HAS_PERM && unsigned(m_row[r]) >= unsigned(n)) {  // corrupt plan: read row 0 instead, and say so
          m_row[r] = 0;
          atomicAdd(&g_bad_indices, 1);
        }
        const unsigned bal = __ballot_sync(gmask, in && (m_sid[r] != nxt));
        m_mask |= ((bal >> lane_base) & ((LPR == 32) ? 0xffffffffu : ((1u << LPR) - 1u))) << (r * LPR);
      }
    };
    // Register of a tile array that holds positions j0 .. j0 + B - 1 (B divides LPR).
    auto tile_reg = [&](const int (&m)[NREG], int j0) {
      int v = m[0];
#pragma unroll
      for (int r = 1; r < NREG; ++r)
        if (j0 / LPR == r) v = m[r];
      return v;
    };
    int cur_t = 0;
    load_tile(0, cur_sid_r, cur_row_r, cur_mask);
    load_tile(1, nxt_sid_r, nxt_row_r, nxt_mask);

    // Copies batch bb (rows bb*B .. bb*B+B-1 of this group's range) into ring stage `stage`.
    auto issue = [&](int bb, int stage) {
      if constexpr (BULK) {
        // Lanes j0 .. j0 + nv - 1 of the tile hold the rows of this batch: each
        // issues the copy of its own row; all copies report to the stage's mbarrier.
        if (bb < nb) {
          const int q0 = bb * B;
          const int j0 = q0 & (T - 1);
          const int nv = min(B, L - q0);
          const int k = lane_g - (j0 & (LPR - 1));
          __syncwarp(gmask);  // every lane has finished reading the stage being refilled
          if (k >= 0 && k < nv) {
            int row = g0 + q0 + k;
            if constexpr (HAS_PERM) row = (q0 / T == cur_t) ? tile_reg(cur_row_r, j0) : tile_reg(nxt_row_r, j0);
            const unsigned bar = bar0 + stage * 8;
            if (k == 0) mbar_arrive_expect_tx(bar, unsigned(nv * row_bytes));
            bulk_copy_g2s(ring_addr + unsigned(stage * B + k) * kRowBytes, slab_src + int64_t(row) * C,
                          unsigned(row_bytes), bar, stream_policy);
          }
        }
      } else {
        if (bb < nb) {
          const int q0 = bb * B;
          const int j0 = q0 & (T - 1);
          const unsigned dst = ring_addr + unsigned(stage * B) * kStageSlotBytes;
          int rows_reg = 0;
          if constexpr (HAS_PERM) rows_reg = (q0 / T == cur_t) ? tile_reg(cur_row_r, j0) : tile_reg(nxt_row_r, j0);
          if (q0 + B <= L) {
#pragma unroll
            for (int k = 0; k < B; ++k) {
              int row = g0 + q0 + k;
              if constexpr (HAS_PERM) row = __shfl_sync(gmask, rows_reg, (j0 & (LPR - 1)) + k, LPR);
              cp_async_16(dst + k * kStageSlotBytes, lane_src + int64_t(row) * C);
            }
          } else {
#pragma unroll
            for (int k = 0; k < B; ++k) {
              if (q0 + k < L) {
                int row = g0 + q0 + k;
                if constexpr (HAS_PERM) row = __shfl_sync(gmask, rows_reg, (j0 & (LPR - 1)) + k, LPR);
                cp_async_16(dst + k * kStageSlotBytes, lane_src + int64_t(row) * C);
              }
            }
          }
        }
        cp_async_commit();
      }
    };

    const bool first_open_left = (g0 > 0) && (__ldg(sid + g0 - 1) == __ldg(sid + g0));
    bool is_first = true;
    int run_start = 0;  // first row (index in this group's range) of the current run
    State acc;
    Op::template init<VEC>(acc);

    // Ends the current run: a complete segment goes to `out`, a run open at an
    // edge of this range is parked in the group's shared-memory slot.
    auto close_run = [&](int sid_now, int cnt, bool open_right) {
      const bool open_left = is_first && first_open_left;
      if (!open_left && !open_right) {
        store_out<Op, VEC>(out, arg, sid_now, C, ch, lane_on, acc, cnt, mean, ospec);
      } else {
        const int slot = 2 * group + (open_right ? 1 : 0);
        uint32_t* pa = s_vec + slot * Op::kPlanes * CPS + lane_g * VEC;
        store_state<Op, VEC>(pa, CPS, acc);
        if (lane_g == 0) {
          s_sid[slot] = sid_now;
          s_cnt[slot] = cnt;
          s_flag[slot] = kValid | (open_left ? kOpenLeft : 0u) | (open_right ? kOpenRight : 0u);
        }
      }
    };
    // One row of a batch that holds run ends.  `single`: the row is a whole segment.
    auto row_step = [&](int q, const Word& t4, int row, bool end_k, bool single, int sids_reg, int lane_k) {
      if (single) {
        float v[VEC];
        unpack_lane<In, VEC>(t4, v);
        const int sid_now = __shfl_sync(gmask, sids_reg, lane_k, LPR);
        store_single<Op, VEC>(out, arg, sid_now, C, ch, lane_on, v, row, ospec);
        is_first = false;
        run_start = q + 1;
      } else {
        accumulate_lane<Op, In, VEC>(acc, t4, row);
        if (end_k) {
          const int sid_now = __shfl_sync(gmask, sids_reg, lane_k, LPR);
          close_run(sid_now, q - run_start + 1, false);
          is_first = false;
          run_start = q + 1;
          Op::template init<VEC>(acc);
        }
      }
    };
    // 1 when the previous row closed a run, i.e. the next row starts a segment
    // (at the start of the range: unless the first run continues from the left).
    unsigned carry = first_open_left ? 0u : 1u;

    wait_for_stream();
#pragma unroll
    for (int bb = 0; bb < S - 1; ++bb) issue(bb, bb);
    int stage_c = 0;        // ring stage of the batch being reduced
    int stage_p = S - 1;    // ring stage the next copy batch goes to

#pragma unroll 1
    for (int b = 0; b < nb; ++b) {
      const int q0 = b * B;
      const int j0 = q0 & (T - 1);
      if (b > 0 && j0 == 0) {  // the reduce front enters the next tile
        ++cur_t;
#pragma unroll
        for (int r = 0; r < NREG; ++r) { cur_sid_r[r] = nxt_sid_r[r]; cur_row_r[r] = nxt_row_r[r]; }
        cur_mask = nxt_mask;
        load_tile(cur_t + 1, nxt_sid_r, nxt_row_r, nxt_mask);
      }
      issue(b + S - 1, stage_p);
      stage_p = (stage_p + 1 == S) ? 0 : stage_p + 1;
      if constexpr (BULK) {
        mbar_wait_bounded(bar0 + stage_c * 8, unsigned(b / S) & 1u);  // batch b has landed
      } else {
        cp_async_wait<S - 1>();  // batch b has landed (groups complete in order)
      }

      const Word* src = ring + stage_c * B * kSlotFloat4;
      stage_c = (stage_c + 1 == S) ? 0 : stage_c + 1;
      const unsigned ends = (cur_mask >> j0) & ((1u << B) - 1u);
      int rows_reg = 0;
      if constexpr (Op::kIsMax && HAS_PERM) rows_reg = tile_reg(cur_row_r, j0);

      if (q0 + B <= L) {
        if (ends == 0u) {
          // eight rows of one run: no bookkeeping
          constexpr int FU = TEXB_FAST_UNROLL;
#pragma unroll FU
          for (int k = 0; k < B; ++k) {
            const Word t4 = src[k * kSlotFloat4];
            int row = g0 + q0 + k;
            if constexpr (Op::kIsMax && HAS_PERM) row = __shfl_sync(gmask, rows_reg, (j0 & (LPR - 1)) + k, LPR);
            accumulate_lane<Op, In, VEC>(acc, t4, row);
          }
          carry = 0u;
        } else {
          // a full batch with run ends: the rows are in registers before any run is closed
          const int sids_reg = tile_reg(cur_sid_r, j0);
          const unsigned singles = ends & ((ends << 1) | carry);  // rows that start and end a run
          carry = (ends >> (B - 1)) & 1u;
          constexpr int U = TEXB_SLOW_UNROLL;
#pragma unroll 1
          for (int k0 = 0; k0 < B; k0 += U) {
            Word t4[U];
#pragma unroll
            for (int u = 0; u < U; ++u) t4[u] = src[(k0 + u) * kSlotFloat4];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int k = k0 + u;
              int row = g0 + q0 + k;
              if constexpr (Op::kIsMax && HAS_PERM) row = __shfl_sync(gmask, rows_reg, (j0 & (LPR - 1)) + k, LPR);
              row_step(q0 + k, t4[u], row, ((ends >> k) & 1u) != 0u, ((singles >> k) & 1u) != 0u, sids_reg,
                       (j0 & (LPR - 1)) + k);
            }
          }
        }
      } else {
        // the ragged last batch of the range
        const int nv = L - q0;
        const int sids_reg = tile_reg(cur_sid_r, j0);
        const unsigned singles = ends & ((ends << 1) | carry);
#pragma unroll 1
        for (int k = 0; k < nv; ++k) {
          const Word t4 = src[k * kSlotFloat4];
          int row = g0 + q0 + k;
          if constexpr (Op::kIsMax && HAS_PERM) row = __shfl_sync(gmask, rows_reg, (j0 & (LPR - 1)) + k, LPR);
          row_step(q0 + k, t4, row, ((ends >> k) & 1u) != 0u, ((singles >> k) & 1u) != 0u, sids_reg,
                   (j0 & (LPR - 1)) + k);
        }
      }
    }
    if (run_start < L) {  // the last run continues past this range
      const int jl = (L - 1) & (T - 1);
      const int sid_now = __shfl_sync(gmask, tile_reg(cur_sid_r, jl & ~(B - 1)), jl & (LPR - 1), LPR);
      close_run(sid_now, L - run_start, true);
    }
  } else {
    wait_for_stream();
  }
  if constexpr (!BULK) cp_async_wait<0>();
  __syncthreads();
  const bool ends_here = stitch_cta<Op, VEC, LPR>(s_vec, s_sid, s_cnt, s_flag, out, arg, ws, C, ch, lane_on, lane_g,
                                                  group, mean, ospec, t_start);
  if (ws.ready)
    finish_chain_in_kernel<Op, VEC, LPR>(ws, ends_here, s_vec, s_cnt, out, arg, C, ch, lane_on, lane_g, group, mean,
                                         ospec);
  stream_tail_wait(sp.no_wait != 0);
}

// ---- fix-up kernel --------------------------------------------------------------
// Block (b, y) finishes the segment whose first piece is CTA b's tail record
// (valid, open to the right, not open to the left).  The pieces that follow are
// the tail records of the CTAs the segment runs through and the head record of
// the CTA where it ends.

template <class Op, int VEC, int LPR>
__global__ void __launch_bounds__(kCtaThreads)
segment_fixup_kernel(Workspace ws, float* __restrict__ out, int32_t* __restrict__ arg,
                     int num_ctas, int C, bool mean, OutSpec ospec) {
  constexpr int GPC = kCtaThreads / LPR;
  constexpr int CPS = LPR * VEC;

  __shared__ __align__(16) uint32_t s_vec[GPC * Op::kPlanes * CPS];
  __shared__ int s_cnt[GPC];
  __shared__ int s_last;

#if __CUDA_ARCH__ >= 900
  // With programmatic dependent launch this grid may start before the reduce
  // grid has finished; wait for its memory to be visible.  No-op otherwise.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif

  const int b = blockIdx.x;
  const int64_t rec_base = int64_t(blockIdx.y) * num_ctas;
  // The first window of head records is fetched together with this CTA's own tail
  // record, so a chain start pays one trip to L2 before it knows where it ends.
  const int4 m0 = ws.meta[(rec_base + b) * 2 + 1];
  const int first = b + 1 + threadIdx.x;
  int4 mh = make_int4(0, 0, 0, 0);
  if (first < num_ctas) mh = ws.meta[(rec_base + first) * 2];
  const unsigned f0 = unsigned(m0.z);
  if (!(f0 & kValid) || !(f0 & kOpenRight) || (f0 & kOpenLeft)) return;  // block-uniform

  // Find the CTA where the segment ends: the first one after b with a head record.
  if (threadIdx.x == 0) s_last = num_ctas;
  __syncthreads();
  for (int base = b + 1; base < num_ctas; base += kCtaThreads) {
    const int idx = base + threadIdx.x;
    if (base != b + 1 && idx < num_ctas) mh = ws.meta[(rec_base + idx) * 2];
    if (idx < num_ctas && (unsigned(mh.z) & kValid)) atomicMin(&s_last, idx);
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
  merge_chain<Op, VEC, LPR>(ws, rec_base, b, last, m0.x, s_vec, s_cnt, out, arg, C, ch, lane_on, lane_g, group, mean,
                            ospec);
}

// ---- host side ----------------------------------------------------------------

struct Layout {
  int in_bytes;  // 4: fp32 features, 2: bf16 features (staged kernel only)
  int lane_bytes;  // bytes of a row one lane owns: vec * in_bytes
  int vec, lpr, cps, num_slabs, gpc;
  int staged;  // 0: register kernel, 1: cp.async ring, 2: bulk-copy (TMA) ring; 128-bit lanes, 16 or 32 lanes per row
};

inline int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#ifndef TEXB_SMALL_BYTES
#define TEXB_SMALL_BYTES (8 << 20)
#endif

// `force_vec` (workspace sizing only) names the channels per lane instead of choosing them.
inline Layout make_layout(int C, bool allow_vec4, int in_bytes = 4, int64_t n = -1, int force_vec = 0) {
  Layout g;
  g.in_bytes = in_bytes;
  g.vec = (allow_vec4 && C % 4 == 0) ? 4 : 1;
  // A few megabytes of narrow rows are bound by latency, not bandwidth: with
  // 128-bit lanes a row of 16 channels is 4 lanes, a CTA holds 64 groups that
  // each fetch ids, rows and features in dependent steps of 4 positions, and one
  // group then stitches 128 edge runs.  One lane per channel makes a group a
  // warp: 32 positions per step and 16 edge runs per CTA.
  if (in_bytes == 4 && C <= 32 && n >= 0 && n * C * 4 <= int64_t(TEXB_SMALL_BYTES)) g.vec = 1;
  // fp32 rows of 36..64 channels: 8-byte lanes, so that a row spans a whole warp
  // (with 16-byte lanes two groups share a warp and each waits while the other
  // closes its runs); needs the bulk-copy ring.
  if (in_bytes == 4 && g.vec == 4 && C > 32 && C <= 64 && tuning().staged == 2) g.vec = 2;
  // bf16 (the caller has checked C % 8 == 0 and the alignment): rows of up to 128
  // channels take 8-byte lanes so that one row spans a warp; wider rows 16-byte lanes.
  if (in_bytes == 2) g.vec = (C <= 128) ? 4 : 8;
  if (force_vec) g.vec = force_vec;
  g.lane_bytes = g.vec * in_bytes;
  const int lanes = C / g.vec;
  int lpr = 1;
  while (lpr < lanes && lpr < 32) lpr <<= 1;
  if (g.vec == 1) lpr = (lpr <= 1) ? 1 : (lpr <= 4 ? 4 : 32);
  g.lpr = lpr;
  g.cps = g.lpr * g.vec;
  g.num_slabs = (C + g.cps - 1) / g.cps;
  g.gpc = kCtaThreads / g.lpr;
  g.staged = ((g.vec >= 4 && g.lpr >= 16) || g.vec == 2) ? tuning().staged : 0;
  if (in_bytes == 2 && g.staged == 0) g.staged = 2;  // bf16 rows exist only in the staged kernel
  return g;
}

// rows_per_cta == 0 (default): the rows are divided evenly over one wave of
// CTAs, `ctas_per_sm` per SM (what the kernel's occupancy allows), so that no
// SM is left with a partial second wave; at least 16 rows per group.
inline Split make_split(int64_t n, const Layout& g, int ctas_per_sm) {
  Split s;
  s.balance = nullptr;
  s.balance_k = 0;
  s.stream_hint = tuning().l2_stream_hint;
  s.plan_settled = 0;
  s.no_wait = 0;
  int64_t rows = tuning().rows_per_cta;
  if (rows <= 0) {
    const int64_t resident = int64_t(sm_count()) * ctas_per_sm;
    rows = ceil_div(n > 0 ? n : 1, resident);
    if (rows < 16 * g.gpc) rows = 16 * g.gpc;
  }
  rows = ceil_div(rows, g.gpc) * g.gpc;
  s.rows_per_cta = int(rows);
  s.rows_per_group = int(rows / g.gpc);
  s.num_ctas = int(ceil_div(n, rows));
  return s;
}

constexpr int kMaxCtasPerSm = 8;  // 256-thread CTAs: the hardware limit of 2048 threads per SM

inline size_t records_vec_bytes(const Layout& g, int num_ctas, int planes) {
  return align_up(size_t(g.num_slabs) * num_ctas * 2 * planes * g.cps * sizeof(uint32_t), 256);
}
inline size_t records_meta_bytes(const Layout& g, int num_ctas) {
  return size_t(g.num_slabs) * num_ctas * 2 * sizeof(int4);
}
inline size_t records_ready_bytes(const Layout& g, int num_ctas) {
  return size_t(g.num_slabs) * num_ctas * sizeof(unsigned long long);
}

// Upper bound over both lane layouts (a caller may pass unaligned pointers) and
// over every occupancy the launch may find.
inline size_t reduce_workspace_bytes(int64_t n, int C, int planes = 2) {
  size_t best = 0;
  // every lane layout a launch may pick for this channel count: fp32 with 1, 4 or 2
  // channels per lane, bf16 with 4 or 8
  const int cand[5][2] = {{4, 1}, {4, 4}, {4, 2}, {2, 4}, {2, 8}};
  for (int v = 0; v < 5; ++v) {
    const int in_bytes = cand[v][0], vec = cand[v][1];
    if (in_bytes == 4 && vec == 4 && C % 4 != 0) continue;
    if (in_bytes == 4 && vec == 2 && (C % 4 != 0 || C <= 32 || C > 64)) continue;
    if (in_bytes == 2 && (C % 8 != 0 || (vec == 4 && C > 128))) continue;
    const Layout g = make_layout(C, true, in_bytes, -1, vec);
    const Split s = make_split(n, g, kMaxCtasPerSm);
    const size_t bytes = records_vec_bytes(g, s.num_ctas, planes) + records_meta_bytes(g, s.num_ctas) +
                         records_ready_bytes(g, s.num_ctas);
    if (bytes > best) best = bytes;
  }
  return best + 512;
}

// One number per launch, never repeated in the life of the process and shared by every
// kernel instantiation (they may use the same workspace one after the other).
inline unsigned long long next_launch_epoch() {
  static std::atomic<unsigned long long> epoch{0x5eed000000000000ull};
  return epoch.fetch_add(1) + 1;
}

struct Call {
  const void* feats;
  const int32_t* sid;
  const int32_t* perm;
  float* out;
  float* out_sum;  // second output of the two-output operator, else NULL
  int32_t* arg;
  void* workspace;
  size_t workspace_bytes;
  int n, C;
  bool mean;
  cudaStream_t stream;
  const int32_t* balance;
  int balance_k;
  int arg_base;
  int m;
  bool plan_settled;
  bool no_split;  // every cut of the balance table is a segment start: no records, nothing to fix up
  bool single_launch;  // finish chains inside the reduce kernel whatever the knob says (sequences of reductions)
  bool no_wait;        // a later reduction of such a sequence
};

// Resident CTAs per SM of one kernel instantiation (asked once per process).
template <class Kernel>
int resident_ctas(Kernel kernel, size_t dyn_smem) {
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kCtaThreads, dyn_smem) != cudaSuccess ||
      blocks < 1) {
    (void)cudaGetLastError();
    blocks = 1;
  }
  return blocks < kMaxCtasPerSm ? blocks : kMaxCtasPerSm;
}

template <class Op, class In, int VEC, int LPR, class Kernel>
int launch_pair(Kernel kernel, size_t dyn_smem, int ctas_per_sm, const Layout& g, const Call& c) {
  Split s = make_split(c.n, g, ctas_per_sm);
  if (c.balance && c.balance_k > 0 && tuning().balanced) {
    s.balance = c.balance;
    s.balance_k = c.balance_k;
  }
  s.plan_settled = c.plan_settled ? 1 : 0;
  s.no_wait = c.no_wait ? 1 : 0;
  const size_t vec_bytes = records_vec_bytes(g, s.num_ctas, Op::kPlanes);
  const size_t meta_bytes = records_meta_bytes(g, s.num_ctas);
  const size_t need = vec_bytes + meta_bytes + records_ready_bytes(g, s.num_ctas);
  const uintptr_t base = align_up(reinterpret_cast<uintptr_t>(c.workspace), 256);
  const size_t pad = base - reinterpret_cast<uintptr_t>(c.workspace);
  if (!c.workspace || c.workspace_bytes < need + pad)
    return fail(TEXB_ERR_WORKSPACE, "reduce workspace: need %zu bytes, got %zu", need + pad,
                c.workspace_bytes);
  Workspace ws;
  ws.vec = reinterpret_cast<uint32_t*>(base);
  ws.meta = reinterpret_cast<int4*>(base + vec_bytes);
  // Chains are finished by the reduce kernel itself ("chain_inline" knob, the default) or by
  // the fix-up kernel that follows it.
  // (The packed bf16 maximum always finishes its chains in the kernel: with a fix-up launch behind it a
  // reduction of the skewed 1 M x 128 workload takes 81.6 us, without 63.4 us -- measured, not understood;
  // its kernels alone take 64.9 + 7.4 us under ncu.)
  const bool inline_chains =
      (tuning().chain_inline != 0 || c.single_launch || c.no_wait || Op::kRawBf16) && s.num_ctas > 1;
  ws.ready = inline_chains ? reinterpret_cast<unsigned long long*>(base + vec_bytes + meta_bytes) : nullptr;
  ws.epoch = inline_chains ? next_launch_epoch() : 0ull;

  const dim3 grid(s.num_ctas, g.num_slabs);
  if (tuning().fixup_pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kCtaThreads);
    cfg.dynamicSmemBytes = dyn_smem;
    cfg.stream = c.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<const In*>(c.feats), c.sid, c.perm, c.out,
                                       c.arg, ws, c.n, c.C, s, c.mean, OutSpec{c.arg_base, c.m, c.out_sum});
    if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "segment reduce launch: %s", cudaGetErrorString(e));
  } else {
    kernel<<<grid, kCtaThreads, dyn_smem, c.stream>>>(static_cast<const In*>(c.feats), c.sid, c.perm, c.out,
                                                      c.arg, ws, c.n, c.C, s, c.mean, OutSpec{c.arg_base, c.m, c.out_sum});
  }
  int st = check_launch("segment reduce kernel");
  if (st != TEXB_OK || s.num_ctas <= 1 || inline_chains) return st;
  if (c.no_split && s.balance != nullptr) return st;  // no segment crosses a group: the fix-up would find nothing

  if (tuning().fixup_pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kCtaThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = c.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, segment_fixup_kernel<Op, VEC, LPR>, ws, c.out, c.arg,
                                       s.num_ctas, c.C, c.mean, OutSpec{c.arg_base, c.m, c.out_sum});
    if (e != cudaSuccess)
      return fail(TEXB_ERR_CUDA, "segment_fixup_kernel launch: %s", cudaGetErrorString(e));
  } else {
    segment_fixup_kernel<Op, VEC, LPR><<<grid, kCtaThreads, 0, c.stream>>>(ws, c.out, c.arg, s.num_ctas,
                                                                           c.C, c.mean, OutSpec{c.arg_base, c.m, c.out_sum});
  }
  return check_launch("segment_fixup_kernel");
}

// Staged walkers (cp.async or bulk-copy ring) for one input type.
template <class Op, class In, int LB, int LPR, bool HAS_PERM>
int launch_staged(const Layout& g, const Call& c) {
  constexpr int VEC = LB / sizeof(In);
  constexpr int kRing = kStageRingBytesFor<In, LB, Op::kPlanes>;
  // The shared-memory attribute is per device: set it on every call (a host-side table write).
  auto staged_launch = [&](auto kernel, int* resident) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing);
    if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    if (*resident == 0) *resident = resident_ctas(kernel, kRing);
    return launch_pair<Op, In, VEC, LPR>(kernel, kRing, *resident, g, c);
  };
  if constexpr (LB == 16) {
    if (g.staged != 2) {
      static int resident = 0;
      return staged_launch(segment_reduce_staged_kernel<Op, In, LB, LPR, HAS_PERM, false>, &resident);
    }
  }
  static int resident = 0;
  return staged_launch(segment_reduce_staged_kernel<Op, In, LB, LPR, HAS_PERM, true>, &resident);
}

template <class Op, int VEC, int LPR, bool HAS_PERM>
int launch_reduce(const Layout& g, const Call& c) {
  if constexpr (VEC == 4 && (LPR == 16 || LPR == 32)) {
    if (g.staged) return launch_staged<Op, float, 16, LPR, HAS_PERM>(g, c);
  }
  auto kernel = segment_reduce_kernel<Op, VEC, LPR, HAS_PERM>;
  static const int resident = resident_ctas(kernel, 0);
  return launch_pair<Op, float, VEC, LPR>(kernel, 0, resident, g, c);
}

template <class Op, int VEC, int LPR>
int dispatch_perm(const Layout& g, const Call& c) {
  if (c.perm) return launch_reduce<Op, VEC, LPR, true>(g, c);
  return launch_reduce<Op, VEC, LPR, false>(g, c);
}

template <class Op>
int dispatch_layout(const Layout& g, const Call& c) {
  if (g.in_bytes == 2) {
    using H = __nv_bfloat16;
    // the maximum of bf16 rows is taken on packed pairs
    using BOp = std::conditional_t<std::is_same_v<Op, OpMax> && TEXB_BF16_PACKED_MAX != 0, OpMaxBf16, Op>;
    if (g.lane_bytes == 8 && g.lpr == 32)
      return c.perm ? launch_staged<BOp, H, 8, 32, true>(g, c) : launch_staged<BOp, H, 8, 32, false>(g, c);
    if constexpr (Op::kPlanes == 2) {  // the two-output operator's edge-run slots would not fit beside 16-byte bf16 lanes
      if (g.lane_bytes == 16 && g.lpr == 32)
        return c.perm ? launch_staged<BOp, H, 16, 32, true>(g, c) : launch_staged<BOp, H, 16, 32, false>(g, c);
    } else if (g.lane_bytes == 16) {
      return fail(TEXB_ERR_UNSUPPORTED, "the two-output reduction takes bf16 rows of up to 128 channels (got %d); "
                  "convert wider rows to fp32", c.C);
    }
    return fail(TEXB_ERR_UNSUPPORTED, "bf16 features need at least 128 channels (got %d lanes per row)", g.lpr);
  }
  if (g.vec == 2)  // make_layout chooses this only for the bulk-copy ring and 32 lanes per row
    return c.perm ? launch_staged<Op, float, 8, 32, true>(g, c) : launch_staged<Op, float, 8, 32, false>(g, c);
  if (g.vec == 4) {
    switch (g.lpr) {
      case 1: return dispatch_perm<Op, 4, 1>(g, c);
      case 2: return dispatch_perm<Op, 4, 2>(g, c);
      case 4: return dispatch_perm<Op, 4, 4>(g, c);
      case 8: return dispatch_perm<Op, 4, 8>(g, c);
      case 16: return dispatch_perm<Op, 4, 16>(g, c);
      case 32: return dispatch_perm<Op, 4, 32>(g, c);
      default: break;
    }
  } else {
    switch (g.lpr) {
      case 1: return dispatch_perm<Op, 1, 1>(g, c);
      case 4: return dispatch_perm<Op, 1, 4>(g, c);
      case 32: return dispatch_perm<Op, 1, 32>(g, c);
      default: break;
    }
  }
  return fail(TEXB_ERR_UNSUPPORTED, "no kernel for %d lanes per row", g.lpr);
}


// Sticky counters of this translation unit's kernels (each unit that instantiates the
// kernels has its own copy; texb_device_status adds them up).
inline int read_unit_counters(int* wait_timeouts, int* bad_indices) {
  int v = 0, v_chain = 0, w = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_wait_timeouts, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&v_chain, g_wait_timeouts_chain, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&w, g_bad_indices, sizeof(int));
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  *wait_timeouts += v + v_chain;
  *bad_indices += w;
  return TEXB_OK;
}

}  // namespace reduce_detail

// One translation unit per operator instantiates the kernels (they compile side by side).
#define TEXB_DECLARE_REDUCE_UNIT(tag)                                                        \
  int reduce_dispatch_##tag(const reduce_detail::Layout& g, const reduce_detail::Call& c);  \
  int reduce_counters_##tag(int* wait_timeouts, int* bad_indices);
#define TEXB_DEFINE_REDUCE_UNIT(tag, Op)                                                      \
  int reduce_dispatch_##tag(const reduce_detail::Layout& g, const reduce_detail::Call& c) {  \
    return reduce_detail::dispatch_layout<Op>(g, c);                                          \
  }                                                                                           \
  int reduce_counters_##tag(int* wait_timeouts, int* bad_indices) {                           \
    return reduce_detail::read_unit_counters(wait_timeouts, bad_indices);                     \
  }
TEXB_DECLARE_REDUCE_UNIT(sum)
TEXB_DECLARE_REDUCE_UNIT(sum_plain)
TEXB_DECLARE_REDUCE_UNIT(max)
TEXB_DECLARE_REDUCE_UNIT(sum_max)

}  // namespace texb
