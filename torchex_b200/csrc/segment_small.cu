// One-launch segment reduction for inputs of a few megabytes made of short segments.
//
// The row-tiled kernels of segment_reduce.cu are built for bandwidth: a launch
// pair (reduce + fix-up), a workspace and a balance table.  On a 1 MB input that
// machinery is all latency: two launches and three or four dependent trips to
// memory per group.  Here one warp owns one segment: it reads the two offsets,
// then the rows (32 / LPR of them side by side, sixteen in flight), folds the
// partial states of its sub-groups with shuffles and writes the output row.  No
// workspace, no fix-up, no fill of empty rows (a warp that finds an empty range
// writes the empty answer itself), no dependence on the plan's sid / balance
// arrays -- offsets (TorchEx's preSum) and, for unsorted ids, the permutation
// are enough, which is exactly what the reference-shaped entry points receive.
//
// The result is right for any input; it is fast when no segment is long, because a
// segment is walked by a single warp.  Callers choose it with
// texb_segment_reduce_small_ok (size of the features, largest segment).
//
// Same arithmetic as the row-tiled kernels: compensated (TwoSum) sums, the mean's
// IEEE division, maxima with the lowest row on ties, NaN and -inf never winning.
// Replaces scatter_sum / scatter_max of torchex/src/scatter/scatter_kernel.cu:102-171
// on the small shapes where that kernel's single launch used to win.

#include "reduce_ops.cuh"

namespace texb {
namespace {

// Rows (perm entries) outside [0, n) and offsets outside [0, n] found by the small
// kernel: skipped or clamped, and counted (sticky; part of texb_device_status).
__device__ int g_small_bad_indices = 0;

constexpr int kSmallInFlight = 16;  // rows a warp keeps in flight

template <int VEC>
__device__ __forceinline__ void small_load_row(const float* __restrict__ p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = __ldg(p);
  }
}

// Folds the state of the sub-group `delta` lanes away into this one.  The two hold
// interleaved rows of the same segment, so for the maximum the tie rule is spelled
// out on the row numbers instead of relying on the order of arrival.
template <class Op, int VEC>
__device__ __forceinline__ void fold_from_lane(typename Op::template State<VEC>& x, int delta) {
  uint32_t w[Op::kPlanes][VEC];
  Op::template pack<VEC>(x, w);
#pragma unroll
  for (int pl = 0; pl < Op::kPlanes; ++pl)
#pragma unroll
    for (int k = 0; k < VEC; ++k) w[pl][k] = __shfl_xor_sync(0xffffffffu, w[pl][k], delta);
  typename Op::template State<VEC> y;
  Op::template unpack<VEC>(y, w);
  if constexpr (Op::kIsMax) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      // "no row" is -1: as unsigned it is larger than every row, so it never wins a tie
      if (y.v[k] > x.v[k] || (y.v[k] == x.v[k] && unsigned(y.i[k]) < unsigned(x.i[k]))) {
        x.v[k] = y.v[k];
        x.i[k] = y.i[k];
      }
    }
  } else {
    // both lanes of a pair must end with the same bits: merge in lane order
    const bool low = ((threadIdx.x & 31) & delta) == 0;
    if (low) {
      Op::template merge<VEC>(x, y);
    } else {
      Op::template merge<VEC>(y, x);
      x = y;
    }
  }
}

template <class Op, int VEC, int LPR, bool HAS_PERM>
__global__ void __launch_bounds__(kCtaThreads)
segment_small_kernel(const float* __restrict__ feats, const int32_t* __restrict__ offsets,
                     const int32_t* __restrict__ perm, float* __restrict__ out, int32_t* __restrict__ arg,
                     int n, int C, int m, bool mean, int arg_base) {
  using State = typename Op::template State<VEC>;
  constexpr int R = 32 / LPR;                                      // rows side by side in a warp
  constexpr int U = (R >= kSmallInFlight) ? 1 : kSmallInFlight / R;  // steps in flight
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR, lane_g = lane % LPR;
  const int warps = (gridDim.x * kCtaThreads) >> 5;
  for (int s = (blockIdx.x * kCtaThreads + threadIdx.x) >> 5; s < m; s += warps) {
    int o0 = __ldg(offsets + s), o1 = __ldg(offsets + s + 1);
    const int lo = min(max(o0, 0), n), hi = min(max(o1, lo), n);
    if ((lo != o0 || hi != o1) && lane == 0) atomicAdd(&g_small_bad_indices, 1);
    o0 = lo;
    o1 = hi;
    for (int ch0 = 0; ch0 < C; ch0 += LPR * VEC) {  // channel slabs of LPR * VEC
      const int ch = ch0 + lane_g * VEC;
      const bool lane_on = ch < C;  // VEC == 4 implies C % 4 == 0
      State acc;
      Op::template init<VEC>(acc);
      for (int base = o0; base < o1; base += R * U) {
        int row[U];
        float v[U][VEC];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int p = base + u * R + sub;
          row[u] = -1;
          if (p < o1) {
            row[u] = HAS_PERM ? __ldg(perm + p) : p;
            if (HAS_PERM && unsigned(row[u]) >= unsigned(n)) {  // corrupt plan: skip the row, and say so
              row[u] = -1;
              if (lane_g == 0) atomicAdd(&g_small_bad_indices, 1);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (row[u] >= 0 && lane_on) {
            small_load_row<VEC>(feats + int64_t(row[u]) * C + ch, v[u]);
          } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[u][k] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (row[u] >= 0) Op::template add<VEC>(acc, v[u], row[u]);
      }
#pragma unroll
      for (int delta = LPR; delta < 32; delta <<= 1) fold_from_lane<Op, VEC>(acc, delta);
      if (sub == 0 && lane_on) {
        float r[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) r[k] = Op::template value<VEC>(acc, k);
        if constexpr (!Op::kIsMax) {
          if (mean && o1 - o0 > 1) divide_by_count<VEC>(r, o1 - o0);
        }
        float* po = out + int64_t(s) * C + ch;
        if constexpr (VEC == 4) {
          *reinterpret_cast<float4*>(po) = make_float4(r[0], r[1], r[2], r[3]);
        } else {
          po[0] = r[0];
        }
        if constexpr (Op::kIsMax) {
          int ix[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {  // "no row" stays -1
            const int i = Op::template index<VEC>(acc, k);
            ix[k] = i < 0 ? i : i + arg_base;
          }
          int32_t* pa = arg + int64_t(s) * C + ch;
          if constexpr (VEC == 4) {
            *reinterpret_cast<int4*>(pa) = make_int4(ix[0], ix[1], ix[2], ix[3]);
          } else {
            pa[0] = ix[0];
          }
        }
      }
    }
  }
}

template <class Op, int VEC, int LPR>
int launch_small(const float* feats, const int32_t* offsets, const int32_t* perm, float* out, int32_t* arg,
                 int n, int C, int m, bool mean, int arg_base, cudaStream_t stream) {
  int64_t ctas = ceil_div(int64_t(m) * 32, kCtaThreads);
  const int64_t cap = 148 * 8;  // one resident wave of 256-thread CTAs
  if (ctas > cap) ctas = cap;
  if (perm)
    segment_small_kernel<Op, VEC, LPR, true><<<unsigned(ctas), kCtaThreads, 0, stream>>>(
        feats, offsets, perm, out, arg, n, C, m, mean, arg_base);
  else
    segment_small_kernel<Op, VEC, LPR, false><<<unsigned(ctas), kCtaThreads, 0, stream>>>(
        feats, offsets, perm, out, arg, n, C, m, mean, arg_base);
  return check_launch("segment_small_kernel");
}

template <class Op, int VEC>
int dispatch_small(int lpr, const float* feats, const int32_t* offsets, const int32_t* perm, float* out,
                   int32_t* arg, int n, int C, int m, bool mean, int arg_base, cudaStream_t stream) {
  switch (lpr) {
    case 1: return launch_small<Op, VEC, 1>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
    case 2: return launch_small<Op, VEC, 2>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
    case 4: return launch_small<Op, VEC, 4>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
    case 8: return launch_small<Op, VEC, 8>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
    case 16: return launch_small<Op, VEC, 16>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
    default: return launch_small<Op, VEC, 32>(feats, offsets, perm, out, arg, n, C, m, mean, arg_base, stream);
  }
}

}  // namespace

#ifndef TEXB_SMALL_PATH_BYTES
#define TEXB_SMALL_PATH_BYTES (8 << 20)
#endif
#ifndef TEXB_SMALL_PATH_MAX_CNT
#define TEXB_SMALL_PATH_MAX_CNT 128
#endif

bool segment_small_ok_impl(int64_t n, int C, int64_t max_cnt) {
  return n >= 0 && C >= 1 && max_cnt >= 0 && max_cnt <= TEXB_SMALL_PATH_MAX_CNT &&
         n * int64_t(C) * 4 <= int64_t(TEXB_SMALL_PATH_BYTES);
}

int segment_small_impl(int op, const float* feats, const int32_t* offsets, const int32_t* perm, int64_t n,
                       int C, int64_t m, float* out, int32_t* arg, int32_t arg_base, cudaStream_t stream) {
  if (op != TEXB_OP_SUM && op != TEXB_OP_MEAN && op != TEXB_OP_MAX)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", op);
  if (n < 0 || m < 0 || C < 1)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "bad sizes n=%lld channel=%d num_segments=%lld", (long long)n, C,
                (long long)m);
  if (n >= (int64_t(1) << 31) - 65536 || m >= (int64_t(1) << 31) - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "n and num_segments must be below 2^31 - 65536");
  if (m == 0) return TEXB_OK;
  if (!out || !offsets) return fail(TEXB_ERR_INVALID_ARGUMENT, "out or offsets is NULL");
  if (op == TEXB_OP_MAX && !arg) return fail(TEXB_ERR_INVALID_ARGUMENT, "arg is NULL");
  if (n > 0 && !feats) return fail(TEXB_ERR_INVALID_ARGUMENT, "feats is NULL");
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec4 = C % 4 == 0 && al(feats) && al(out) && (op != TEXB_OP_MAX || al(arg));
  const int vec = vec4 ? 4 : 1;
  int lpr = 1;
  while (lpr < C / vec && lpr < 32) lpr <<= 1;
  const bool mean = op == TEXB_OP_MEAN;
  if (op == TEXB_OP_MAX) {
    if (vec4) return dispatch_small<OpMax, 4>(lpr, feats, offsets, perm, out, arg, int(n), C, int(m), false, arg_base, stream);
    return dispatch_small<OpMax, 1>(lpr, feats, offsets, perm, out, arg, int(n), C, int(m), false, arg_base, stream);
  }
  if (vec4) return dispatch_small<OpSumComp, 4>(lpr, feats, offsets, perm, out, arg, int(n), C, int(m), mean, arg_base, stream);
  return dispatch_small<OpSumComp, 1>(lpr, feats, offsets, perm, out, arg, int(n), C, int(m), mean, arg_base, stream);
}

int small_bad_indices_impl(int* count) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_small_bad_indices, sizeof(int));
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  *count = v;
  return TEXB_OK;
}

}  // namespace texb
