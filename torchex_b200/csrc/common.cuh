// Shared host-side helpers of the scatter library: status reporting, launch
// checks and process-wide tuning knobs.  Nothing here exits or throws.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/texb_scatter.h"

namespace texb {

// Records a message for texb_last_error() on the calling thread and returns
// `status` so call sites can `return fail(...)`.
int fail(int status, const char* fmt, ...);

// Returns TEXB_OK or records the pending CUDA launch error.
int check_launch(const char* what);

// Tuning knobs (see texb_tune_set).
struct Tuning {
  int rows_per_cta;  // rows of the segment-sorted order handled by one CTA; 0 = one wave
  int staged;        // row staging where the layout allows: 0 registers, 1 cp.async ring, 2 bulk-copy ring
  int compensated;   // 1: error-free (two-sum) accumulation in sum / mean
  int fixup_pdl;     // 1: launch the fix-up kernel with programmatic dependent launch
  int balanced;      // 1: use the plan's balance table to cut the rows by estimated cost
  int end_cost_x4;   // cost of closing a segment, in quarter rows, for that table
  int l2_stream_hint;  // 1: bulk copies of feature rows carry an L2 evict-first policy
  int chain_inline;    // 1: segments that span CTAs are finished inside the reduce kernel; 0: by the fix-up kernel
};
Tuning tuning();

constexpr int kCtaThreads = 256;

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

#ifdef __CUDACC__
// v[k] / float(count) for VEC values that share the divisor, rounded exactly like
// an IEEE fp32 division (what `sum / unq_cnts` and `g / unq_cnts` compute in
// torchex/operator_py/scatter_op.py:69, 76).  One reciprocal refined to nearly
// full double-word accuracy serves all VEC quotients; each quotient gets two
// residual corrections, which leaves it correctly rounded whenever the dividend
// is a normal number far from the overflow and underflow thresholds.  Anything
// else (zero, subnormal, huge, infinite, NaN dividend) takes the true division.
template <int VEC>
__device__ __forceinline__ void divide_by_count(float (&v)[VEC], int count) {
  if (count == 1) return;
  const float b = float(count);
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(b));
  y = fmaf(y, fmaf(-b, y, 1.f), y);
  y = fmaf(y, fmaf(-b, y, 1.f), y);
  float lo = fabsf(v[0]), hi = lo;
#pragma unroll
  for (int k = 1; k < VEC; ++k) {
    lo = fminf(lo, fabsf(v[k]));
    hi = fmaxf(hi, fabsf(v[k]));
  }
  if (lo > 1e-30f && hi < 1e30f) {  // false as well when a value is NaN
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const float a = v[k];
      float q = a * y;
      q = fmaf(fmaf(-b, q, a), y, q);
      q = fmaf(fmaf(-b, q, a), y, q);
      v[k] = q;
    }
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = __fdiv_rn(v[k], b);
  }
}
#endif

}  // namespace texb
