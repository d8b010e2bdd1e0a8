// Backward of the scatter operators: one fused row-broadcast pass per call.
//
//   sum : g_in[i, :] = g[sid_i, :]
//   mean: g_in[i, :] = g[sid_i, :] / count(sid_i)
//   max : g_in[i, c] = (arg[sid_i, c] == i) ? g[sid_i, c] : 0
//   mean + max (the two-output forward): the sum of the mean and max expressions,
//         from g (gradient of the means) and g2 (gradient of the maxima)
//
// Lanes run along the channel axis (128-bit accesses when the layout allows),
// a group of lanes handles eight consecutive entries of `ids` per step, and g_in
// is written with streaming stores so that g / arg stay resident in cache.  With
// a permutation the walk is in segment-sorted order (ids = the plan's sid, row =
// perm[i]): consecutive entries then belong to the same segment, so the rows of
// g and arg are fetched once from L2 and afterwards hit in L1, instead of one
// random 512-byte L2 read per point.  No memset, no atomics.
//
// Replaces the ATen expressions in ScatterSumFunction.backward,
// ScatterMeanFunction.backward and ScatterMaxFunction.backward
// (torchex/operator_py/scatter_op.py:47-50, 73-78, 105-111).

#include "common.cuh"

namespace texb {
namespace {

constexpr int kModeSum = 0, kModeMean = 1, kModeMax = 2, kModeMeanMax = 3;
constexpr int kRowsPerStep = 4;

template <int VEC>
struct Pack { float v[VEC]; };

template <int VEC>
__device__ __forceinline__ Pack<VEC> load_f(const float* p) {
  Pack<VEC> r;
  if constexpr (VEC == 4) {
    float4 t = __ldg(reinterpret_cast<const float4*>(p));
    r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
  } else {
    r.v[0] = __ldg(p);
  }
  return r;
}

template <int VEC>
struct PackI { int v[VEC]; };

template <int VEC>
__device__ __forceinline__ PackI<VEC> load_i(const int32_t* p) {
  PackI<VEC> r;
  if constexpr (VEC == 4) {
    int4 t = __ldg(reinterpret_cast<const int4*>(p));
    r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
  } else {
    r.v[0] = __ldg(p);
  }
  return r;
}

template <int VEC>
__device__ __forceinline__ void store_stream(float* p, const Pack<VEC>& r) {
  if constexpr (VEC == 4) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
  } else {
    __stcs(p, r.v[0]);
  }
}

// Entries handled per step and per group of lanes; a group walks
// kStepsPerGroup consecutive steps and fetches the ids / rows / counts of the
// next step while it works on the current one.
constexpr int kStepsPerGroup = 8;

struct StepMeta {
  int s[kRowsPerStep];    // segment of each entry, -1: write a zero row
  int row[kRowsPerStep];  // row of g_in each entry writes, -1: nothing
  int den[kRowsPerStep];  // row count of the segment (mean only)
};

template <int MODE>
__device__ __forceinline__ void load_meta(StepMeta& mt, int64_t e0, const int32_t* __restrict__ ids,
                                          const int32_t* __restrict__ perm,
                                          const int32_t* __restrict__ offsets, int64_t n, int64_t m) {
#pragma unroll
  for (int k = 0; k < kRowsPerStep; ++k) {
    const int64_t i = e0 + k;
    const bool in = i < n;
    const int v = in ? __ldg(ids + i) : -1;
    mt.s[k] = (v >= 0 && v < m) ? v : -1;  // ids outside the range get a zero row
    int r = in ? int(i) : -1;
    if (perm != nullptr && in) {
      const int pr = __ldg(perm + i);
      r = (pr >= 0 && pr < n) ? pr : -1;  // a bad permutation entry writes nothing
    }
    mt.row[k] = r;
  }
  if constexpr (MODE == kModeMean || MODE == kModeMeanMax) {
#pragma unroll
    for (int k = 0; k < kRowsPerStep; ++k) {
      mt.den[k] = 1;
      if (mt.s[k] >= 0) mt.den[k] = __ldg(offsets + mt.s[k] + 1) - __ldg(offsets + mt.s[k]);
    }
  }
}

template <int MODE, int VEC, int LPR>
__global__ void __launch_bounds__(kCtaThreads, 4)
broadcast_back_kernel(const float* __restrict__ g, const float* __restrict__ g2, const int32_t* __restrict__ arg,
                      const int32_t* __restrict__ ids, const int32_t* __restrict__ perm,
                      const int32_t* __restrict__ offsets, float* __restrict__ g_in, int64_t n, int C,
                      int64_t m) {
  constexpr int GPC = kCtaThreads / LPR;
  const int lane_g = threadIdx.x & (LPR - 1);
  const int group = threadIdx.x / LPR;
  const int64_t e_begin = (int64_t(blockIdx.x) * GPC + group) * (kRowsPerStep * kStepsPerGroup);
  if (e_begin >= n) return;
  const int64_t e_end = min(e_begin + int64_t(kRowsPerStep * kStepsPerGroup), n);

  StepMeta cur, nxt;
  load_meta<MODE>(cur, e_begin, ids, perm, offsets, n, m);
  for (int64_t e0 = e_begin; e0 < e_end; e0 += kRowsPerStep) {
    const bool more = e0 + kRowsPerStep < e_end;
    if (more) load_meta<MODE>(nxt, e0 + kRowsPerStep, ids, perm, offsets, n, m);
    for (int ch = lane_g * VEC; ch < C; ch += LPR * VEC) {
      Pack<VEC> val[kRowsPerStep];
      Pack<VEC> quotient;  // g / count of the entry before: neighbours mostly share their segment
#pragma unroll
      for (int k = 0; k < kRowsPerStep; ++k) {
        if (cur.s[k] >= 0) {
          val[k] = load_f<VEC>(g + int64_t(cur.s[k]) * C + ch);
          if constexpr (MODE == kModeMax) {
            PackI<VEC> a = load_i<VEC>(arg + int64_t(cur.s[k]) * C + ch);
#pragma unroll
            for (int q = 0; q < VEC; ++q)
              if (a.v[q] != cur.row[k]) val[k].v[q] = 0.f;
          }
          if constexpr (MODE == kModeMean || MODE == kModeMeanMax) {
            // the walk is in sorted order, so the division is done once per run of equal
            // segments in a step and copied for the entries that follow
            if (k > 0 && cur.s[k] == cur.s[k > 0 ? k - 1 : 0]) {
              val[k] = quotient;
            } else {
              divide_by_count<VEC>(val[k].v, cur.den[k]);
              quotient = val[k];
            }
          }
          if constexpr (MODE == kModeMeanMax) {
            const Pack<VEC> gm = load_f<VEC>(g2 + int64_t(cur.s[k]) * C + ch);
            const PackI<VEC> a = load_i<VEC>(arg + int64_t(cur.s[k]) * C + ch);
#pragma unroll
            for (int q = 0; q < VEC; ++q)
              if (a.v[q] == cur.row[k]) val[k].v[q] += gm.v[q];
          }
        } else {
#pragma unroll
          for (int q = 0; q < VEC; ++q) val[k].v[q] = 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < kRowsPerStep; ++k) {
        if (cur.row[k] >= 0) store_stream<VEC>(g_in + int64_t(cur.row[k]) * C + ch, val[k]);
      }
    }
    if (more) cur = nxt;
  }
}

template <int MODE, int VEC>
int launch_lpr(int lpr, const float* g, const float* g2, const int32_t* arg, const int32_t* ids, const int32_t* perm,
               const int32_t* offsets, float* g_in, int64_t n, int C, int64_t m,
               cudaStream_t stream) {
  const int gpc = kCtaThreads / lpr;
  const unsigned blocks = unsigned(ceil_div(n, int64_t(gpc) * kRowsPerStep * kStepsPerGroup));
#define TEXB_LAUNCH(L)                                                                   \
  broadcast_back_kernel<MODE, VEC, L><<<blocks, kCtaThreads, 0, stream>>>(g, g2, arg, ids, \
                                                                         perm, offsets, g_in, n, C, m)
  switch (lpr) {
    case 1: TEXB_LAUNCH(1); break;
    case 2: TEXB_LAUNCH(2); break;
    case 4: TEXB_LAUNCH(4); break;
    case 8: TEXB_LAUNCH(8); break;
    case 16: TEXB_LAUNCH(16); break;
    default: TEXB_LAUNCH(32); break;
  }
#undef TEXB_LAUNCH
  return check_launch("broadcast_back_kernel");
}

template <int MODE>
int launch_back(const float* g, const float* g2, const int32_t* arg, const int32_t* ids, const int32_t* perm,
                const int32_t* offsets, float* g_in, int64_t n, int C, int64_t m, cudaStream_t stream) {
  if (n < 0 || m < 0 || C < 1) return fail(TEXB_ERR_INVALID_ARGUMENT, "backward: bad sizes");
  if (n == 0) return TEXB_OK;
  constexpr bool kArg = MODE == kModeMax || MODE == kModeMeanMax;
  constexpr bool kDen = MODE == kModeMean || MODE == kModeMeanMax;
  if (!g_in || !ids || (m > 0 && !g) || (kArg && m > 0 && !arg) || (kDen && !offsets) ||
      (MODE == kModeMeanMax && m > 0 && !g2))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "backward: NULL pointer");
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec4 = (C % 4 == 0) && al(g) && al(g_in) && (!kArg || al(arg)) && (MODE != kModeMeanMax || al(g2));
  const int vec = vec4 ? 4 : 1;
  int lpr = 1;
  while (lpr < C / vec && lpr < 32) lpr <<= 1;
  if (vec4) return launch_lpr<MODE, 4>(lpr, g, g2, arg, ids, perm, offsets, g_in, n, C, m, stream);
  return launch_lpr<MODE, 1>(lpr, g, g2, arg, ids, perm, offsets, g_in, n, C, m, stream);
}

}  // namespace

int sum_backward_impl(const float* g, const int32_t* ids, const int32_t* perm, float* g_in, int64_t n,
                      int C, int64_t m, cudaStream_t stream) {
  return launch_back<kModeSum>(g, nullptr, nullptr, ids, perm, nullptr, g_in, n, C, m, stream);
}
int mean_backward_impl(const float* g, const int32_t* ids, const int32_t* perm, const int32_t* offsets,
                       float* g_in, int64_t n, int C, int64_t m, cudaStream_t stream) {
  return launch_back<kModeMean>(g, nullptr, nullptr, ids, perm, offsets, g_in, n, C, m, stream);
}
int max_backward_impl(const float* g, const int32_t* arg, const int32_t* ids, const int32_t* perm,
                      float* g_in, int64_t n, int C, int64_t m, cudaStream_t stream) {
  return launch_back<kModeMax>(g, nullptr, arg, ids, perm, nullptr, g_in, n, C, m, stream);
}
int mean_max_backward_impl(const float* g_mean, const float* g_max, const int32_t* arg, const int32_t* ids,
                           const int32_t* perm, const int32_t* offsets, float* g_in, int64_t n, int C,
                           int64_t m, cudaStream_t stream) {
  return launch_back<kModeMeanMax>(g_mean, g_max, arg, ids, perm, offsets, g_in, n, C, m, stream);
}

}  // namespace texb
