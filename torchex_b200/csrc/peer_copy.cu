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
//   * cudaMemcpyAsync from such a mapping into local memory on a stream of the caller.
//
// No kernel of this library ever reads or writes another GPU's memory: the only access
// to a peer mapping is the driver's DMA copy issued here.  Ordering between the
// processes (a shard is complete before it is pulled, pulled before it is overwritten)
// is the caller's job; torchex_b200/frames.py does it with small NCCL collectives.
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

}  // namespace texb
