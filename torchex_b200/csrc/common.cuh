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
};
Tuning tuning();

constexpr int kCtaThreads = 256;

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace texb
