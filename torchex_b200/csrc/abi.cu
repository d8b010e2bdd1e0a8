// extern "C" surface of the library (declared in include/texb_scatter.h):
// argument plumbing, thread-local error text and the tuning knobs.

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace texb {

// implemented in the kernel files
int ids_inspect_impl(const void*, int, int64_t, int32_t*, cudaStream_t);
size_t plan_workspace_bytes_impl(int64_t, int64_t, int);
int plan_build_impl(const void*, int, int64_t, int64_t, int, int32_t*, int32_t*, int32_t*, int32_t*,
                    void*, size_t, cudaStream_t);
int get_pre_sum_impl(const int32_t*, int32_t*, int64_t, int64_t, cudaStream_t);
size_t reduce_workspace_bytes_impl(int64_t, int);
size_t reduce_pair_workspace_bytes_impl(int64_t, int);
int segment_reduce_impl(int, const void*, int, const int32_t*, const int32_t*, const int32_t*, int,
                        const int32_t*, int, int64_t, int, int64_t, float*, int32_t*, int32_t, void*,
                        size_t, cudaStream_t, float* out_sum = nullptr);
int plan_balance_impl(const int32_t*, int64_t, int32_t*, int, const int32_t*, cudaStream_t);
size_t unique_workspace_bytes_impl(int64_t);
int unique_count_impl(const void*, int, int64_t, int64_t, int, int32_t*, int32_t*, int32_t*, void*, size_t,
                      cudaStream_t);
int unique_fill_impl(const int32_t*, const int32_t*, int64_t, int64_t, int32_t*, int32_t*, int32_t*, int32_t*,
                     int32_t*, void*, size_t, cudaStream_t);
int segment_rank_impl(const int32_t*, const int32_t*, const int32_t*, int64_t, int64_t, int64_t*, cudaStream_t);
bool segment_small_ok_impl(int64_t, int, int64_t);
int segment_small_impl(int, const float*, const int32_t*, const int32_t*, int64_t, int, int64_t, float*, int32_t*,
                       int32_t, cudaStream_t);
int segment_reduce_static_impl(int, const float*, const int32_t*, const int32_t*, const int32_t*, int,
                               const int32_t*, int, int64_t, int, int64_t, float*, int32_t*, int32_t,
                               cudaStream_t);
size_t static_scratch_bytes_impl();
int device_status_impl(int*, int*);
int expand_offsets_impl(const int32_t*, int32_t*, int64_t, int64_t, cudaStream_t);
int sum_backward_impl(const float*, const int32_t*, const int32_t*, float*, int64_t, int, int64_t,
                      cudaStream_t);
int mean_backward_impl(const float*, const int32_t*, const int32_t*, const int32_t*, float*, int64_t, int,
                       int64_t, cudaStream_t);
int max_backward_impl(const float*, const int32_t*, const int32_t*, const int32_t*, float*, int64_t, int,
                      int64_t, cudaStream_t);
int mean_max_backward_impl(const float*, const float*, const int32_t*, const int32_t*, const int32_t*,
                           const int32_t*, float*, int64_t, int, int64_t, cudaStream_t);

int peer_buffer_create_impl(size_t, void**, unsigned char*);
int peer_buffer_destroy_impl(void*);
int peer_buffer_open_impl(const unsigned char*, void**);
int peer_buffer_close_impl(void*);
int peer_copy_impl(void*, const void*, size_t, cudaStream_t);
int peer_pull_impl(const void* const*, void* const*, const size_t*, int, void* const*, const int64_t*, const int32_t*, int,
                   cudaStream_t);
int mean_from_sum_impl(const float*, const int32_t*, int64_t, int, float*, cudaStream_t);

namespace {
thread_local char t_error[512] = "";

std::mutex g_tuning_mutex;
Tuning g_tuning = {0, 2, 1, 1, 1, 5, 0, 0};
bool g_tuning_env_read = false;

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  if (!v || !*v) return fallback;
  return std::atoi(v);
}

bool set_knob(Tuning& t, const char* key, int value) {
  if (!std::strcmp(key, "rows_per_cta")) {
    if (value != 0 && (value < 64 || value > (1 << 20))) return false;
    t.rows_per_cta = value;
    return true;
  }
  if (!std::strcmp(key, "staged")) {
    if (value < 0 || value > 2) return false;
    t.staged = value;
    return true;
  }
  if (!std::strcmp(key, "compensated")) {
    if (value != 0 && value != 1) return false;
    t.compensated = value;
    return true;
  }
  if (!std::strcmp(key, "fixup_pdl")) {
    if (value != 0 && value != 1) return false;
    t.fixup_pdl = value;
    return true;
  }
  if (!std::strcmp(key, "balanced")) {
    if (value != 0 && value != 1) return false;
    t.balanced = value;
    return true;
  }
  if (!std::strcmp(key, "l2_stream_hint")) {
    if (value != 0 && value != 1) return false;
    t.l2_stream_hint = value;
    return true;
  }
  if (!std::strcmp(key, "end_cost_x4")) {
    if (value < 0 || value > 1024) return false;
    t.end_cost_x4 = value;
    return true;
  }
  if (!std::strcmp(key, "chain_inline")) {
    if (value != 0 && value != 1) return false;
    t.chain_inline = value;
    return true;
  }
  return false;
}

void read_env_locked() {
  if (g_tuning_env_read) return;
  g_tuning_env_read = true;
  set_knob(g_tuning, "rows_per_cta", env_int("TEXB_ROWS_PER_CTA", g_tuning.rows_per_cta));
  set_knob(g_tuning, "staged", env_int("TEXB_STAGED", g_tuning.staged));
  set_knob(g_tuning, "compensated", env_int("TEXB_COMPENSATED", g_tuning.compensated));
  set_knob(g_tuning, "fixup_pdl", env_int("TEXB_FIXUP_PDL", g_tuning.fixup_pdl));
  set_knob(g_tuning, "balanced", env_int("TEXB_BALANCED", g_tuning.balanced));
  set_knob(g_tuning, "end_cost_x4", env_int("TEXB_END_COST_X4", g_tuning.end_cost_x4));
  set_knob(g_tuning, "l2_stream_hint", env_int("TEXB_L2_STREAM_HINT", g_tuning.l2_stream_hint));
  set_knob(g_tuning, "chain_inline", env_int("TEXB_CHAIN_INLINE", g_tuning.chain_inline));
}
}  // namespace

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return TEXB_OK;
  return fail(TEXB_ERR_CUDA, "%s: %s (cuda error %d)", what, cudaGetErrorString(e), int(e));
}

Tuning tuning() {
  std::lock_guard<std::mutex> lock(g_tuning_mutex);
  read_env_locked();
  return g_tuning;
}

}  // namespace texb

using namespace texb;

extern "C" {

int texb_version(void) { return 202; }

const char* texb_last_error(void) { return t_error; }

int texb_tune_set(const char* key, int value) {
  if (!key) return fail(TEXB_ERR_INVALID_ARGUMENT, "tune_set: NULL key");
  std::lock_guard<std::mutex> lock(g_tuning_mutex);
  read_env_locked();
  if (!set_knob(g_tuning, key, value))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "tune_set: unknown key or bad value: %s=%d", key, value);
  return TEXB_OK;
}

int texb_tune_get(const char* key) {
  if (!key) return -1;
  Tuning t = tuning();
  if (!std::strcmp(key, "rows_per_cta")) return t.rows_per_cta;
  if (!std::strcmp(key, "staged")) return t.staged;
  if (!std::strcmp(key, "compensated")) return t.compensated;
  if (!std::strcmp(key, "fixup_pdl")) return t.fixup_pdl;
  if (!std::strcmp(key, "balanced")) return t.balanced;
  if (!std::strcmp(key, "end_cost_x4")) return t.end_cost_x4;
  if (!std::strcmp(key, "l2_stream_hint")) return t.l2_stream_hint;
  if (!std::strcmp(key, "chain_inline")) return t.chain_inline;
  return -1;
}

int texb_device_status(int* wait_timeouts, int* bad_indices) {
  return device_status_impl(wait_timeouts, bad_indices);
}

int texb_ids_inspect(const void* ids, int id_bytes, int64_t n, int32_t* stats_dev, void* stream) {
  return ids_inspect_impl(ids, id_bytes, n, stats_dev, static_cast<cudaStream_t>(stream));
}

size_t texb_plan_workspace_bytes(int64_t n, int64_t num_segments, int sorted) {
  return plan_workspace_bytes_impl(n, num_segments, sorted);
}

int texb_plan_build(const void* ids, int id_bytes, int64_t n, int64_t num_segments, int sorted,
                    int32_t* sid_out, int32_t* perm_out, int32_t* offsets_out,
                    int32_t* plan_stats_dev, void* workspace, size_t workspace_bytes,
                    void* stream) {
  return plan_build_impl(ids, id_bytes, n, num_segments, sorted, sid_out, perm_out, offsets_out,
                         plan_stats_dev, workspace, workspace_bytes,
                         static_cast<cudaStream_t>(stream));
}

int texb_get_pre_sum(const int32_t* unq_inv, int32_t* pre_sum, int64_t num_total, int64_t num_unq,
                     void* stream) {
  return get_pre_sum_impl(unq_inv, pre_sum, num_total, num_unq, static_cast<cudaStream_t>(stream));
}

size_t texb_reduce_workspace_bytes(int64_t n, int channel) {
  if (n < 0 || channel < 1) return 0;
  return reduce_workspace_bytes_impl(n, channel);
}

int texb_plan_balance(const int32_t* sid, int64_t n, int32_t* balance_out, int balance_len,
                      const int32_t* plan_stats_dev, void* stream) {
  return plan_balance_impl(sid, n, balance_out, balance_len, plan_stats_dev, static_cast<cudaStream_t>(stream));
}

size_t texb_unique_workspace_bytes(int64_t n) { return unique_workspace_bytes_impl(n); }

int texb_unique_count(const void* keys, int key_bytes, int64_t n, int64_t key_bound, int sorted,
                      int32_t* sorted_keys_out, int32_t* perm_out, int32_t* stats_dev, void* workspace,
                      size_t workspace_bytes, void* stream) {
  return unique_count_impl(keys, key_bytes, n, key_bound, sorted, sorted_keys_out, perm_out, stats_dev,
                           workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int texb_unique_fill(const int32_t* sorted_keys, const int32_t* perm, int64_t n, int64_t num_segments,
                     int32_t* sid_out, int32_t* offsets_out, int32_t* unq_inv_out, int32_t* unique_keys_out,
                     int32_t* plan_stats_dev, void* workspace, size_t workspace_bytes, void* stream) {
  return unique_fill_impl(sorted_keys, perm, n, num_segments, sid_out, offsets_out, unq_inv_out,
                          unique_keys_out, plan_stats_dev, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream));
}

int texb_segment_rank(const int32_t* sid, const int32_t* perm, const int32_t* offsets, int64_t n,
                      int64_t num_segments, int64_t* rank_out, void* stream) {
  return segment_rank_impl(sid, perm, offsets, n, num_segments, rank_out, static_cast<cudaStream_t>(stream));
}

int texb_segment_reduce_small_ok(int64_t n, int channel, int64_t max_cnt) {
  return segment_small_ok_impl(n, channel, max_cnt) ? 1 : 0;
}

int texb_segment_reduce_small(int op, const float* feats, const int32_t* offsets, const int32_t* perm,
                              int64_t n, int channel, int64_t num_segments, float* out, int32_t* arg,
                              int32_t arg_base, void* stream) {
  return segment_small_impl(op, feats, offsets, perm, n, channel, num_segments, out, arg, arg_base,
                            static_cast<cudaStream_t>(stream));
}

int texb_segment_reduce(int op, const float* feats, const int32_t* sid, const int32_t* perm,
                        const int32_t* offsets, int plan_flags, const int32_t* balance,
                        int balance_len, int64_t n, int channel, int64_t num_segments, float* out,
                        int32_t* arg, int32_t arg_base, void* workspace, size_t workspace_bytes,
                        void* stream) {
  return segment_reduce_impl(op, feats, 4, sid, perm, offsets, plan_flags, balance, balance_len, n,
                             channel, num_segments, out, arg, arg_base, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream));
}

int texb_segment_reduce_bf16(int op, const void* feats_bf16, const int32_t* sid, const int32_t* perm,
                             const int32_t* offsets, int plan_flags, const int32_t* balance,
                             int balance_len, int64_t n, int channel, int64_t num_segments, float* out,
                             int32_t* arg, int32_t arg_base, void* workspace, size_t workspace_bytes,
                             void* stream) {
  return segment_reduce_impl(op, feats_bf16, 2, sid, perm, offsets, plan_flags, balance, balance_len, n,
                             channel, num_segments, out, arg, arg_base, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream));
}

size_t texb_reduce_pair_workspace_bytes(int64_t n, int channel) {
  if (n < 0 || channel < 1) return 0;
  return reduce_pair_workspace_bytes_impl(n, channel);
}

int texb_segment_reduce_pair(int op, const void* feats, int feature_bytes, const int32_t* sid,
                             const int32_t* perm, const int32_t* offsets, int plan_flags,
                             const int32_t* balance, int balance_len, int64_t n, int channel,
                             int64_t num_segments, float* out_sum, float* out_max, int32_t* arg,
                             int32_t arg_base, void* workspace, size_t workspace_bytes, void* stream) {
  if (num_segments > 0 && !out_sum) return fail(TEXB_ERR_INVALID_ARGUMENT, "out_sum is NULL");
  if (num_segments == 0) return TEXB_OK;
  return segment_reduce_impl(op, feats, feature_bytes, sid, perm, offsets, plan_flags, balance, balance_len, n,
                             channel, num_segments, out_max, arg, arg_base, workspace, workspace_bytes,
                             static_cast<cudaStream_t>(stream), out_sum);
}

size_t texb_static_scratch_bytes(void) { return static_scratch_bytes_impl(); }

int texb_segment_reduce_static(int op, const float* feats, const int32_t* sid, const int32_t* perm,
                               const int32_t* offsets, int plan_flags, const int32_t* balance,
                               int balance_len, int64_t n, int channel, int64_t num_segments,
                               float* out, int32_t* arg, int32_t arg_base, void* stream) {
  return segment_reduce_static_impl(op, feats, sid, perm, offsets, plan_flags, balance, balance_len, n,
                                    channel, num_segments, out, arg, arg_base,
                                    static_cast<cudaStream_t>(stream));
}

size_t texb_scatter_compat_workspace_bytes(int64_t num_total, int channel) {
  if (num_total < 0 || channel < 1) return 0;
  return align_up(size_t(num_total) * sizeof(int32_t), 256) + 256 +
         reduce_workspace_bytes_impl(num_total, channel);
}

static int compat_reduce(int op, const float* feats, const int32_t* pre_sum, float* out,
                         int32_t* arg, int channel, int num_unq, int max_cnt, int64_t num_total,
                         void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (num_total < 0 || num_unq < 0 || channel < 1)
    return fail(TEXB_ERR_INVALID_ARGUMENT, "scatter: bad sizes");
  if (!pre_sum) return fail(TEXB_ERR_INVALID_ARGUMENT, "scatter: preSum is NULL");
  // a small input of short segments: one launch straight from preSum, no workspace
  if (max_cnt > 0 && segment_small_ok_impl(num_total, channel, max_cnt))
    return segment_small_impl(op, feats, pre_sum, nullptr, num_total, channel, num_unq, out, arg, 0, stream);
  if (num_total >= (int64_t(1) << 31) - 65536)
    return fail(TEXB_ERR_UNSUPPORTED, "scatter: num_total must be below 2^31 - 65536");
  const size_t sid_bytes = align_up(size_t(num_total) * sizeof(int32_t), 256);
  uintptr_t base = align_up(reinterpret_cast<uintptr_t>(workspace), 256);
  const size_t pad = base - reinterpret_cast<uintptr_t>(workspace);
  if (!workspace || workspace_bytes < pad + sid_bytes)
    return fail(TEXB_ERR_WORKSPACE, "scatter workspace: need %zu bytes, got %zu",
                texb_scatter_compat_workspace_bytes(num_total, channel), workspace_bytes);
  int32_t* sid = reinterpret_cast<int32_t*>(base);
  int st = expand_offsets_impl(pre_sum, sid, num_total, num_unq, stream);
  if (st != TEXB_OK) return st;
  // The reference kernels write every row, including those of empty ranges.
  return segment_reduce_impl(op, feats, 4, sid, nullptr, pre_sum, TEXB_PLAN_HAS_EMPTY, nullptr, 0, num_total, channel,
                             num_unq, out, arg, /*arg_base=*/0, reinterpret_cast<void*>(base + sid_bytes),
                             workspace_bytes - pad - sid_bytes, stream);
}

int texb_scatter_sum(const float* feats, const int32_t* pre_sum, float* out, int channel,
                     int num_unq, int max_cnt, int64_t num_total, void* workspace,
                     size_t workspace_bytes, void* stream) {
  return compat_reduce(TEXB_OP_SUM, feats, pre_sum, out, nullptr, channel, num_unq, max_cnt, num_total,
                       workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int texb_scatter_max(const float* feats, const int32_t* pre_sum, float* out, int32_t* arg,
                     int channel, int num_unq, int max_cnt, int64_t num_total, void* workspace,
                     size_t workspace_bytes, void* stream) {
  return compat_reduce(TEXB_OP_MAX, feats, pre_sum, out, arg, channel, num_unq, max_cnt, num_total,
                       workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int texb_scatter_sum_backward(const float* g, const int32_t* ids, const int32_t* perm, float* g_in,
                              int64_t n, int channel, int64_t num_segments, void* stream) {
  return sum_backward_impl(g, ids, perm, g_in, n, channel, num_segments,
                           static_cast<cudaStream_t>(stream));
}

int texb_scatter_mean_backward(const float* g, const int32_t* ids, const int32_t* perm,
                               const int32_t* offsets, float* g_in, int64_t n, int channel,
                               int64_t num_segments, void* stream) {
  return mean_backward_impl(g, ids, perm, offsets, g_in, n, channel, num_segments,
                            static_cast<cudaStream_t>(stream));
}

int texb_scatter_max_backward(const float* g, const int32_t* arg, const int32_t* ids,
                              const int32_t* perm, float* g_in, int64_t n, int channel,
                              int64_t num_segments, void* stream) {
  return max_backward_impl(g, arg, ids, perm, g_in, n, channel, num_segments,
                           static_cast<cudaStream_t>(stream));
}

int texb_scatter_mean_max_backward(const float* g_mean, const float* g_max, const int32_t* arg,
                                   const int32_t* ids, const int32_t* perm, const int32_t* offsets,
                                   float* g_in, int64_t n, int channel, int64_t num_segments,
                                   void* stream) {
  return mean_max_backward_impl(g_mean, g_max, arg, ids, perm, offsets, g_in, n, channel, num_segments,
                                static_cast<cudaStream_t>(stream));
}

int texb_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle_out) {
  return peer_buffer_create_impl(bytes, dev_ptr, handle_out);
}
int texb_peer_buffer_destroy(void* dev_ptr) { return peer_buffer_destroy_impl(dev_ptr); }
int texb_peer_buffer_open(const unsigned char* handle, void** peer_ptr) {
  return peer_buffer_open_impl(handle, peer_ptr);
}
int texb_peer_buffer_close(void* peer_ptr) { return peer_buffer_close_impl(peer_ptr); }
int texb_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  return peer_copy_impl(dst, src, bytes, static_cast<cudaStream_t>(stream));
}
int texb_peer_pull(const void* const* srcs, void* const* dsts, const size_t* bytes, int n, void* stream) {
  return peer_pull_impl(srcs, dsts, bytes, n, nullptr, nullptr, nullptr, 0, static_cast<cudaStream_t>(stream));
}
int texb_peer_pull_mean(const void* const* srcs, void* const* dsts, void* const* mean_dsts, const size_t* bytes,
                        const int64_t* first_rows, int n, const int32_t* counts, int channel, void* stream) {
  if (!mean_dsts) return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull_mean: mean_dsts is NULL");
  return peer_pull_impl(srcs, dsts, bytes, n, mean_dsts, first_rows, counts, channel, static_cast<cudaStream_t>(stream));
}
int texb_mean_from_sum(const float* sums, const int32_t* counts, int64_t num_segments, int channel, float* out,
                       void* stream) {
  return mean_from_sum_impl(sums, counts, num_segments, channel, out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
