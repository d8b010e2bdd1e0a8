// Host entry of the forward segment reduction: argument checks, the choice of lane
// layout, the rows of empty segments, the reference-shaped helpers and the entry point
// that brings its own scratch.  The kernels themselves are templates in
// segment_reduce_kernels.cuh, instantiated one operator per translation unit
// (reduce_unit_*.cu) so that they compile in parallel.

#include "segment_reduce_kernels.cuh"

namespace texb {
using namespace reduce_detail;

namespace {

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


}  // namespace

// `out_sum` selects the two-output form: op (sum or mean) goes to out_sum, the
// maxima and their rows to out / arg, from one pass over the features.
int segment_reduce_impl(int op, const void* feats, int in_bytes, const int32_t* sid, const int32_t* perm,
                        const int32_t* offsets, int plan_flags, const int32_t* balance,
                        int balance_len, int64_t n, int C, int64_t m, float* out, int32_t* arg,
                        int32_t arg_base, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                        float* out_sum) {
  const bool pair = out_sum != nullptr;
  const bool has_empty = (plan_flags & TEXB_PLAN_HAS_EMPTY) != 0;
  const bool plan_settled = (plan_flags & TEXB_PLAN_SETTLED) != 0;
  const bool no_split = (plan_flags & TEXB_PLAN_NO_SPLIT) != 0;
  const bool no_wait = (plan_flags & TEXB_SEQUENCE_NEXT) != 0;
  const bool single_launch = no_wait || (plan_flags & TEXB_SEQUENCE_FIRST) != 0;
  if (no_wait && !plan_settled)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "TEXB_SEQUENCE_NEXT needs TEXB_PLAN_SETTLED: a reduction that does not "
                "wait for the stream may only read a plan the host knows to be complete");
  if (in_bytes != 4 && in_bytes != 2)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "features must be fp32 (4 bytes) or bf16 (2 bytes)");
  if (op != TEXB_OP_SUM && op != TEXB_OP_MEAN && op != TEXB_OP_MAX)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "unknown reduce op %d", op);
  if (pair && op == TEXB_OP_MAX)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "the two-output reduction pairs the maximum with sum or mean");
  if (n < 0 || m < 0 || C < 1)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "bad sizes n=%lld channel=%d num_segments=%lld",
                (long long)n, C, (long long)m);
  if (n >= (int64_t(1) << 31) - 65536 || m >= (int64_t(1) << 31) - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "n and num_segments must be below 2^31 - 65536");
  if (m > 0 && !out) return fail(TEXB_ERR_INVALID_ARGUMENT, "out is NULL");
  if (m > 0 && (op == TEXB_OP_MAX || pair) && !arg) return fail(TEXB_ERR_INVALID_ARGUMENT, "arg is NULL");
  if (n > 0 && (!feats || !sid)) return fail(TEXB_ERR_INVALID_ARGUMENT, "feats or sid is NULL");
  if ((has_empty || n == 0) && m > 0 && !offsets)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "offsets is required when has_empty is set or n == 0");
  if (m == 0) return TEXB_OK;

  if (has_empty || n == 0) {
    const int64_t total = m * C;
    const int64_t want = ceil_div(total, 256);
    const int blocks = int(want < 148 * 16 ? want : 148 * 16);
    fill_empty_kernel<<<blocks, 256, 0, stream>>>(offsets, out, arg, m, C, op == TEXB_OP_MAX || pair);
    if (pair) fill_empty_kernel<<<blocks, 256, 0, stream>>>(offsets, out_sum, nullptr, m, C, false);
    int st = check_launch("fill_empty_kernel");
    if (st != TEXB_OK || n == 0) return st;
  }

  const bool vec_ok = aligned16(feats) && aligned16(out) && ((op != TEXB_OP_MAX && !pair) || aligned16(arg)) &&
                      (!pair || aligned16(out_sum));
  if (in_bytes == 2 && (!vec_ok || C % 8 != 0 || C < 128))
    return fail(TEXB_ERR_UNSUPPORTED,
                "bf16 features need 16-byte aligned pointers and a channel count that is a multiple of 8 "
                "and at least 128 (got %d); convert to fp32 for other shapes", C);
  const Layout g = make_layout(C, vec_ok, in_bytes, n);
  if (balance && balance_len < 2)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "balance table needs at least 2 entries");
  Call c = {feats, sid, perm, out, out_sum, arg, workspace, workspace_bytes, int(n), C, op == TEXB_OP_MEAN, stream,
            balance, balance ? balance_len - 1 : 0, int(arg_base), int(m), plan_settled, no_split, single_launch,
            no_wait};
  if (pair) return reduce_dispatch_sum_max(g, c);
  if (op == TEXB_OP_MAX) return reduce_dispatch_max(g, c);
  if (tuning().compensated) return reduce_dispatch_sum(g, c);
  return reduce_dispatch_sum_plain(g, c);
}

int expand_offsets_impl(const int32_t* offsets, int32_t* sid, int64_t n, int64_t m,
                        cudaStream_t stream) {
  if (n == 0) return TEXB_OK;
  expand_offsets_kernel<<<unsigned(ceil_div(n, 256)), 256, 0, stream>>>(offsets, sid, int(n), int(m));
  return check_launch("expand_offsets_kernel");
}

size_t reduce_workspace_bytes_impl(int64_t n, int C) { return reduce_workspace_bytes(n, C); }
size_t reduce_pair_workspace_bytes_impl(int64_t n, int C) { return reduce_workspace_bytes(n, C, OpSumMax::kPlanes); }

// ---- reduce without a caller workspace -------------------------------------------------
// Some callers may not allocate device memory at all once they are running: a
// perception loop that sizes every buffer at start-up and forbids cudaMalloc
// afterwards, a plugin living inside a host application's fixed memory pool, or
// code between stream-ordered work where an allocation would stall the device.
// For them the records of the reduce kernels live in this array, which is part of
// the library image: every GPU that loads the library holds these 4 MiB until the
// process exits.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t static_scratch_bytes_impl() { return kStaticScratchBytes; }

int segment_reduce_static_impl(int op, const float* feats, const int32_t* sid, const int32_t* perm,
                               const int32_t* offsets, int plan_flags, const int32_t* balance,
                               int balance_len, int64_t n, int C, int64_t m, float* out, int32_t* arg,
                               int32_t arg_base, cudaStream_t stream) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* device_ptr[kMaxDevices] = {};
  // Sizes are validated before the scratch requirement is computed from them, so that a
  // nonsensical size is reported as such and not as "scratch too small".
  if (n < 0 || m < 0 || C < 1)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "bad sizes n=%lld channel=%d num_segments=%lld", (long long)n, C,
                (long long)m);
  if (n >= (int64_t(1) << 31) - 65536 || m >= (int64_t(1) << 31) - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "n and num_segments must be below 2^31 - 65536");
  const size_t need = reduce_workspace_bytes(n, C);
  if (need > kStaticScratchBytes)
    return fail(TEXB_ERR_UNSUPPORTED,
                "this shape needs %zu bytes of scratch but the built-in scratch holds %zu; "
                "use texb_segment_reduce with a caller workspace (or a larger rows_per_cta)",
                need, kStaticScratchBytes);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(TEXB_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!device_ptr[dev]) {
      // In host code the array's name is only a handle: ask the runtime for the
      // address the array has on the current device, once per device.  The address
      // is kept for the life of the process: a caller that destroys the device's
      // context (cudaDeviceReset) must not use this entry point afterwards.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p)
        return fail(TEXB_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
      device_ptr[dev] = p;
    }
    scratch = device_ptr[dev];
  }
  return segment_reduce_impl(op, feats, 4, sid, perm, offsets, plan_flags, balance, balance_len, n, C, m, out,
                             arg, arg_base, scratch, kStaticScratchBytes, stream, nullptr);
}

int small_bad_indices_impl(int* count);  // segment_small.cu
int plan_bad_indices_impl(int* count);   // segment_plan.cu

int device_status_impl(int* wait_timeouts, int* bad_indices) {
  int v = 0, w = 0, w_small = 0, w_plan = 0;
  int st = reduce_counters_sum(&v, &w);
  if (st == TEXB_OK) st = reduce_counters_sum_plain(&v, &w);
  if (st == TEXB_OK) st = reduce_counters_max(&v, &w);
  if (st == TEXB_OK) st = reduce_counters_sum_max(&v, &w);
  if (st == TEXB_OK) st = small_bad_indices_impl(&w_small);
  if (st == TEXB_OK) st = plan_bad_indices_impl(&w_plan);
  if (st != TEXB_OK) return st;
  if (wait_timeouts) *wait_timeouts = v;
  if (bad_indices) *bad_indices = w + w_small + w_plan;
  return TEXB_OK;
}

}  // namespace texb
