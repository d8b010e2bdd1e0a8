// C-callable doorway to the UNMODIFIED TorchEx scatter launchers, which are
// compiled from the reference tree by oracle/Makefile and linked with this
// file into oracle/_ref/libtorchex_scatter_ref.so.  Test infrastructure and
// benchmark baseline only; the shipped library never links it.
//
// The launchers are declared exactly as the reference binding declares them
// (torchex/src/scatter/scatter.cpp:12-18).  They launch on the legacy default
// stream and check nothing (scatter_kernel.cu:173-192), so each wrapper
// validates the documented limits first, then reports the launch status.
#include <cuda_runtime.h>
#include <stdint.h>

void scatter_sum_launcher(const float* const feats, const int* const preSum, float* const out,
                          int channel, int num_unq, int max_cnt);
void scatter_max_launcher(const float* const feats, const int* const preSum, float* const out,
                          int* const arg, int channel, int num_unq, int max_cnt);
void getPreSum_launcher(const int* const unq_inv, int* const preSum, int num_total);
// torchex/src/ingroup_inds/ingroup_inds.cpp:14-19 declares it like this
void ingroup_inds_launcher(const long* group_inds, long* out_inds, int N, int max_group_id);

namespace {
int block_x(int max_cnt) {
  int p = 1;
  while (p < max_cnt) p <<= 1;
  if (p > 1024) p = 1024;
  if (p < 32) p = 32;
  return p;
}
// The reference's grid is (channel, ceil(num_unq / (1024 / X))): both must fit
// the launch limits, and its row index arithmetic is 32-bit
// (scatter_kernel.cu:115, 147, 181, 189).  Returns 0 when the call is safe.
int limits_ok(int channel, int num_unq, int max_cnt, int64_t num_total) {
  if (channel < 1 || num_unq < 1 || max_cnt < 1) return 1;
  const int per_block = 1024 / block_x(max_cnt);
  const int64_t grid_y = (int64_t(num_unq) + per_block - 1) / per_block;
  if (grid_y > 65535) return 2;
  if (num_total * channel >= (int64_t(1) << 31)) return 3;
  return 0;
}
int finish() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return 100 + int(e);
  return 0;
}
}  // namespace

extern "C" {

// 0 = the reference can run this shape; otherwise the limit it would break.
int torchex_ref_limits(int channel, int num_unq, int max_cnt, int64_t num_total) {
  return limits_ok(channel, num_unq, max_cnt, num_total);
}

int torchex_ref_scatter_sum(const float* feats, const int* pre_sum, float* out, int channel,
                            int num_unq, int max_cnt, int64_t num_total) {
  int bad = limits_ok(channel, num_unq, max_cnt, num_total);
  if (bad) return bad;
  scatter_sum_launcher(feats, pre_sum, out, channel, num_unq, max_cnt);
  return finish();
}

int torchex_ref_scatter_max(const float* feats, const int* pre_sum, float* out, int* arg,
                            int channel, int num_unq, int max_cnt, int64_t num_total) {
  int bad = limits_ok(channel, num_unq, max_cnt, num_total);
  if (bad) return bad;
  scatter_max_launcher(feats, pre_sum, out, arg, channel, num_unq, max_cnt);
  return finish();
}

int torchex_ref_get_pre_sum(const int* unq_inv, int* pre_sum, int num_total) {
  if (num_total < 1) return 1;
  getPreSum_launcher(unq_inv, pre_sum, num_total);
  return finish();
}

// The reference's ingroup_inds (ingroup_inds_kernel.cu:17-59): out_inds[i] = arrival
// number of element i inside its group (an atomic counter per group, so the order
// within a group is not defined).  It allocates and frees its own counters.
int torchex_ref_ingroup_inds(const long* group_inds, long* out_inds, int n, int max_group_id) {
  if (n < 1 || max_group_id < 0) return 1;
  ingroup_inds_launcher(group_inds, out_inds, n, max_group_id);
  return finish();
}

}  // extern "C"
