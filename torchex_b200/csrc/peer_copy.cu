// Peer buffers and DMA copies for the multi-GPU frame driver (one process per GPU).
//
// When a caller wants every GPU to hold the full [num_segments, C] result of a sharded
// reduction, each GPU's shard has to reach the seven others.  The shards are hundreds of
// megabytes, so the transfer should run at what the NVLink fabric gives a plain device-
// to-device copy, on the copy engines, while the SMs go on with the next reduction.
// This file provides exactly that and nothing else:
//
//   * a buffer that other processes of the box can map (cudaMalloc + a CUDA IPC handle;
//     the reduce kernels write a shard into it like into any other device buffer),
//   * mapping a peer's buffer into this process (cudaIpcOpenMemHandle on the CURRENT
//     device, peer access enabled lazily),
//   * cudaMemcpyAsync from such a mapping into local memory on a stream of the caller,
//   * peer_pull: ONE kernel that reads up to 16 such mappings with plain vector loads and
//     writes the rows into local memory.  On an NVSwitch box it moves more bytes per
//     second than the copy engines do (measured with four GPUs: 619 GB/s inbound per GPU
//     against 536 GB/s for cudaMemcpyAsync on one stream per peer), because loads from
//     all peers are in flight at once.
//
// The pull kernel is the only kernel of this library that touches another GPU's memory,
// and it only LOADS from it (ld.global through the peer mapping; no TMA, no multicast,
// no stores to a peer, nothing it waits for).  Ordering between the processes (a shard
// is complete before it is pulled, pulled before it is overwritten) is the caller's job;
// torchex_b200/peer_ring.py does it with one small NCCL collective per gather.
// The reference has no multi-GPU code (every test pins cuda:0, test/test_scatter.py:9).

#include <cstring>

#include "common.cuh"

namespace texb {

int peer_buffer_create_impl(size_t bytes, void** dev_ptr, unsigned char* handle_out) {
  if (!dev_ptr || !handle_out || bytes == 0) return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_buffer_create: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == TEXB_PEER_HANDLE_BYTES, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaFree(p);
    return fail(TEXB_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  std::memcpy(handle_out, &h, sizeof(h));
  *dev_ptr = p;
  return TEXB_OK;
}

int peer_buffer_destroy_impl(void* dev_ptr) {
  if (!dev_ptr) return TEXB_OK;
  cudaError_t e = cudaFree(dev_ptr);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaFree: %s", cudaGetErrorString(e));
  return TEXB_OK;
}

int peer_buffer_open_impl(const unsigned char* handle, void** peer_ptr) {
  if (!handle || !peer_ptr) return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_buffer_open: bad argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(TEXB_ERR_CUDA, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  *peer_ptr = p;
  return TEXB_OK;
}

int peer_buffer_close_impl(void* peer_ptr) {
  if (!peer_ptr) return TEXB_OK;
  cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return TEXB_OK;
}

int peer_copy_impl(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) return TEXB_OK;
  if (!dst || !src) return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_copy: NULL pointer");
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "cudaMemcpyAsync (peer): %s", cudaGetErrorString(e));
  return TEXB_OK;
}

// ---- pull kernel ---------------------------------------------------------------------

struct PullRegions {
  const void* src[TEXB_PEER_PULL_MAX];
  void* dst[TEXB_PEER_PULL_MAX];
  unsigned long long bytes[TEXB_PEER_PULL_MAX];
  // only for the variant that also writes means: where they go, and the first row of each region
  // in `counts` (segment sizes of all rows, on this GPU); `words_per_row` = channel / 4
  float* mean_dst[TEXB_PEER_PULL_MAX];
  long long first_row[TEXB_PEER_PULL_MAX];
  const int32_t* counts;
  unsigned words_per_row;
  // CTAs [cta_begin[k], cta_begin[k + 1]) of the 1-D grid copy region k
  int cta_begin[TEXB_PEER_PULL_MAX + 1];
  int n;
};

// One small CTA per SM (256 threads, at most 64 registers: 16 K of the SM's 64 K) so that it fits beside
// the two resident CTAs of a running reduction instead of pushing one of them into a second wave;
// 148 of them with eight loads per thread keep 4.8 MB in flight, enough for the links.
constexpr int kPullThreads = 256;
constexpr int kPullUnroll = 8;    // 16-byte loads in flight per thread
constexpr int kPullCtas = 148;    // CTAs over all regions
constexpr double kPullLocalWeight = 0.25;  // share of CTAs per byte of a region in this GPU's own memory (its own shard)

// The mean row of the sums in 16-byte word `i` of a region: the division of the reduce kernels.
__device__ __forceinline__ void store_mean_word(const PullRegions& r, int reg, unsigned long long i, const uint4& v) {
  const int cnt = __ldg(r.counts + r.first_row[reg] + (long long)(i / r.words_per_row));
  float m[4] = {__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)};
  if (cnt > 1) divide_by_count<4>(m, cnt);
  __stcs(reinterpret_cast<float4*>(r.mean_dst[reg]) + i, make_float4(m[0], m[1], m[2], m[3]));
}

// Region k is copied by its range of CTAs (more for regions behind a link than for local ones) with a grid-stride loop of
// 16-byte words, kPullUnroll loads issued before the first store; a region whose addresses or size are
// not multiples of 16 bytes goes word by word (results are 4-byte types, so 4 bytes always divide it).
// MEAN: the regions hold rows of sums, and next to each copied word the kernel writes the word of means
// (sums divided by the size of their segment) into a second local tensor -- the copy is bound by the
// links, so the division and the second store ride along for nothing.
template <bool MEAN>
__global__ void __launch_bounds__(kPullThreads, 4) peer_pull_kernel(PullRegions r) {
  constexpr int U = kPullUnroll;
  int reg = 0;
  while (reg + 1 < r.n && int(blockIdx.x) >= r.cta_begin[reg + 1]) ++reg;
  const unsigned long long bytes = r.bytes[reg];
  const unsigned long long stride = (unsigned long long)(r.cta_begin[reg + 1] - r.cta_begin[reg]) * blockDim.x;
  unsigned long long i = (unsigned long long)(int(blockIdx.x) - r.cta_begin[reg]) * blockDim.x + threadIdx.x;
  const bool wide = ((reinterpret_cast<uintptr_t>(r.src[reg]) | reinterpret_cast<uintptr_t>(r.dst[reg]) | bytes) & 15) == 0;
  if (MEAN || wide) {   // (the host only launches MEAN on 16-byte aligned regions)
    const uint4* __restrict__ s = static_cast<const uint4*>(r.src[reg]);
    uint4* __restrict__ d = static_cast<uint4*>(r.dst[reg]);
    const unsigned long long n = bytes >> 4;
    for (; i + (U - 1) * stride < n; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = __ldcs(s + i + u * stride);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        __stcs(d + i + u * stride, v[u]);
        if (MEAN) store_mean_word(r, reg, i + u * stride, v[u]);
      }
    }
#pragma unroll 1
    for (; i < n; i += stride) {
      const uint4 v = __ldcs(s + i);
      __stcs(d + i, v);
      if (MEAN) store_mean_word(r, reg, i, v);
    }
  } else {
    const uint32_t* __restrict__ s = static_cast<const uint32_t*>(r.src[reg]);
    uint32_t* __restrict__ d = static_cast<uint32_t*>(r.dst[reg]);
    const unsigned long long n = bytes >> 2;
#pragma unroll 1
    for (; i < n; i += stride) d[i] = s[i];
  }
}

int peer_pull_impl(const void* const* srcs, void* const* dsts, const size_t* bytes, int n, void* const* mean_dsts,
                   const int64_t* first_rows, const int32_t* counts, int channel, cudaStream_t stream) {
  if (n < 0 || (n > 0 && (!srcs || !dsts || !bytes))) return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull: bad argument");
  const bool mean = mean_dsts != nullptr;
  if (mean && (!first_rows || !counts || channel <= 0 || channel % 4 != 0))
    return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull_mean: needs first_rows, counts and a channel count divisible by 4");
  for (int first = 0; first < n; first += TEXB_PEER_PULL_MAX) {
    PullRegions r;
    r.counts = counts;
    r.words_per_row = mean ? unsigned(channel / 4) : 1u;
    int m = 0, locals = 0;
    bool local[TEXB_PEER_PULL_MAX];
    int device = 0;
    (void)cudaGetDevice(&device);
    for (int k = first; k < n && k < first + TEXB_PEER_PULL_MAX; ++k) {
      if (bytes[k] == 0) continue;
      if (!srcs[k] || !dsts[k] || (mean && !mean_dsts[k]))
        return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull: NULL pointer in region %d", k);
      const uintptr_t bits = reinterpret_cast<uintptr_t>(srcs[k]) | reinterpret_cast<uintptr_t>(dsts[k]) | bytes[k] |
                             (mean ? reinterpret_cast<uintptr_t>(mean_dsts[k]) : 0);
      if (bits & (mean ? 15 : 3))
        return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull: region %d is not made of aligned %d-byte words", k, mean ? 16 : 4);
      if (mean && (first_rows[k] < 0 || bytes[k] % (size_t(channel) * 4) != 0))
        return fail(TEXB_ERR_INVALID_ARGUMENT, "peer_pull_mean: region %d is not made of whole rows", k);
      r.src[m] = srcs[k];
      r.dst[m] = dsts[k];
      r.bytes[m] = bytes[k];
      r.mean_dst[m] = mean ? static_cast<float*>(mean_dsts[k]) : nullptr;
      r.first_row[m] = mean ? first_rows[k] : 0;
      cudaPointerAttributes attr;   // a source in this GPU's own memory needs far fewer loads in flight than one behind a link
      local[m] = cudaPointerGetAttributes(&attr, srcs[k]) == cudaSuccess && attr.type == cudaMemoryTypeDevice &&
                 attr.device == device;
      (void)cudaGetLastError();
      locals += local[m] ? 1 : 0;
      ++m;
    }
    if (m == 0) continue;
    r.n = m;
    // CTAs in proportion to the time a region needs: its bytes, counted at a quarter when they are local
    // (a CTA moves local bytes about ten times faster than bytes from behind a link); nobody gets more
    // CTAs than it has work for
    (void)locals;
    double weight[TEXB_PEER_PULL_MAX], sum = 0;
    for (int k = 0; k < m; ++k) sum += weight[k] = double(r.bytes[k]) * (local[k] ? kPullLocalWeight : 1.0);
    const size_t per_cta = size_t(kPullThreads) * kPullUnroll * 16;
    int total = 0;
    for (int k = 0; k < m; ++k) {
      int ctas = int(kPullCtas * weight[k] / sum);
      if (ctas < 1) ctas = 1;
      const size_t useful = (size_t(r.bytes[k]) + per_cta - 1) / per_cta;
      if (size_t(ctas) > useful) ctas = int(useful);
      r.cta_begin[k] = total;
      total += ctas;
    }
    r.cta_begin[m] = total;
    if (mean) peer_pull_kernel<true><<<total, kPullThreads, 0, stream>>>(r);
    else peer_pull_kernel<false><<<total, kPullThreads, 0, stream>>>(r);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "peer_pull launch: %s", cudaGetErrorString(e));
  }
  return TEXB_OK;
}

// ---- mean rows from sum rows ---------------------------------------------------------

// out[s, :] = sums[s, :] / counts[s] with the division of the reduce kernels, so that a mean derived
// from a replicated sum has the bits of the mean the owning GPU would have sent.  Rows of empty
// segments (count 0) are copied as they are (the reduce kernels fill them with zeros).
__global__ void __launch_bounds__(256) mean_from_sum_kernel(const float* __restrict__ sums, const int32_t* __restrict__ counts,
                                                            long long total, int C, float* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float v[1] = {__ldcs(sums + i)};
    const int cnt = counts[i / C];
    if (cnt > 1) divide_by_count<1>(v, cnt);
    __stcs(out + i, v[0]);
  }
}

template <int VEC>
__global__ void __launch_bounds__(256) mean_from_sum_vec_kernel(const float* __restrict__ sums, const int32_t* __restrict__ counts,
                                                                long long groups, int groups_per_row, float* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(sums) + g);
    float v[4] = {x.x, x.y, x.z, x.w};
    const int cnt = counts[g / groups_per_row];
    if (cnt > 1) divide_by_count<4>(v, cnt);
    __stcs(reinterpret_cast<float4*>(out) + g, make_float4(v[0], v[1], v[2], v[3]));
  }
}

int mean_from_sum_impl(const float* sums, const int32_t* counts, int64_t num_segments, int channel, float* out, cudaStream_t stream) {
  if (num_segments < 0 || channel <= 0) return fail(TEXB_ERR_INVALID_ARGUMENT, "mean_from_sum: bad size");
  if (num_segments == 0) return TEXB_OK;
  if (!sums || !counts || !out) return fail(TEXB_ERR_INVALID_ARGUMENT, "mean_from_sum: NULL pointer");
  const long long total = (long long)num_segments * channel;
  const bool wide = channel % 4 == 0 && ((reinterpret_cast<uintptr_t>(sums) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const long long items = wide ? total / 4 : total;
  long long blocks = (items + 255) / 256;
  const long long cap = 148LL * 8 * 4;
  if (blocks > cap) blocks = cap;
  if (wide) mean_from_sum_vec_kernel<4><<<int(blocks), 256, 0, stream>>>(sums, counts, items, channel / 4, out);
  else mean_from_sum_kernel<<<int(blocks), 256, 0, stream>>>(sums, counts, total, channel, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TEXB_ERR_CUDA, "mean_from_sum launch: %s", cudaGetErrorString(e));
  return TEXB_OK;
}

}  // namespace texb
