// Peer-memory plumbing for the multi-GPU form of MSDA: replication of the value tensor by the COPY ENGINES.
//
// The reference runs one device (src/gac/execution/cuda.py:132-138); nothing here has a counterpart there.
//
// Query-sharded MSDA needs the whole value tensor in every GPU's own memory.  When value starts out sharded
// (each rank holds 1/N of every batch entry's rows), an NCCL all-gather brings it together -- with kernels: their
// thread blocks need whole SMs, which the gather kernel's thousands of small thread blocks never leave free, so
// collective and gather end up running one after the other.  Peer copies over NVLink (cudaMemcpyAsync between
// two GPUs' memories, one process per GPU, CUDA IPC handles) are executed by the copy engines, take no SM, and
// run beside the gather kernel at the NVLink rate.  This file holds what that needs and torch does not offer:
//
//   gacb_ipc_alloc / gacb_ipc_open / gacb_ipc_close / gacb_ipc_free   a device buffer other processes can map
//   gacb_copy_async                                                  one copy on a stream (any two mapped addresses)
//   gacb_peer_barrier                                                "every rank has reached this point of its
//                                                                    stream": a one-block kernel that stores this
//                                                                    rank's step number into every peer's flag array
//                                                                    and waits -- with a limit -- for all of theirs.
// Kernels never gather from a peer's memory: the copies land in this GPU's own memory first.
#include "gacb_common.cuh"

namespace gacb {
namespace {

constexpr int kMaxRanks = 16;
constexpr uint32_t kBarrierSpinLimit = 1u << 19;      // polls, each followed by a 1 us sleep: about half a second

struct PeerBarrierArgs {
  uint32_t *peer_flags[kMaxRanks];   // peer r's flag array (mapped into this process); slot [rank] is ours to write
  uint32_t *local_flags;             // this rank's flag array: slot [r] is written by rank r
  uint32_t *local_step;              // this rank's barrier count, kept on the device so that a captured launch works
  int32_t *status;                   // set to 2 when a peer did not arrive in time
  int world, rank;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ PeerBarrierArgs p) {
  __shared__ uint32_t step_s;
  if (threadIdx.x == 0) step_s = ++(*p.local_step);
  __syncwarp();
  const uint32_t step = step_s;
  const int r = threadIdx.x;
  if (r >= p.world) return;
  __threadfence_system();                                   // what this stream wrote before is visible first
  *reinterpret_cast<volatile uint32_t *>(p.peer_flags[r] + p.rank) = step;
  __threadfence_system();
  const volatile uint32_t *mine = p.local_flags + r;
  for (uint32_t poll = 0; poll < kBarrierSpinLimit; ++poll) {
    if ((int32_t)(*mine - step) >= 0) return;               // rank r has reached this barrier (or a later one)
    __nanosleep(1000);
  }
  if (p.status) atomicExch(p.status, 2);                    // gave up: the caller's status word says so
}

}  // namespace
}  // namespace gacb

using namespace gacb;

GACB_API int gacb_ipc_alloc(size_t bytes, void **ptr, unsigned char *handle) {
  if (!ptr || !handle || bytes == 0) return fail(GACB_ERR_INVALID_ARGUMENT, "ipc_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == GACB_IPC_HANDLE_BYTES, "IPC handle size");
  void *p = nullptr;
  int rc = check_cuda(cudaMalloc(&p, bytes), "cudaMalloc(ipc buffer)");
  if (rc != GACB_OK) return rc;
  rc = check_cuda(cudaMemset(p, 0, bytes), "cudaMemset(ipc buffer)");
  cudaIpcMemHandle_t h;
  if (rc == GACB_OK) rc = check_cuda(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  if (rc != GACB_OK) {
    cudaFree(p);
    return rc;
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return GACB_OK;
}

GACB_API int gacb_ipc_open(const unsigned char *handle, void **ptr) {
  if (!ptr || !handle) return fail(GACB_ERR_INVALID_ARGUMENT, "ipc_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

GACB_API int gacb_ipc_close(void *ptr) {
  if (!ptr) return GACB_OK;
  return check_cuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle");
}

GACB_API int gacb_ipc_free(void *ptr) {
  if (!ptr) return GACB_OK;
  return check_cuda(cudaFree(ptr), "cudaFree(ipc buffer)");
}

GACB_API int gacb_copy_async(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return GACB_OK;
  if (!dst || !src) return fail(GACB_ERR_INVALID_ARGUMENT, "copy_async: NULL pointer");
  return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)), "cudaMemcpyAsync");
}

GACB_API int gacb_peer_barrier(void *const *peer_flags, void *local_flags, void *local_step, int world, int rank,
                               int32_t *status_word, void *stream) {
  if (!peer_flags || !local_flags || !local_step) return fail(GACB_ERR_INVALID_ARGUMENT, "peer_barrier: NULL pointer");
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return fail(GACB_ERR_INVALID_ARGUMENT, "peer_barrier: world %d / rank %d outside [1,%d]", world, rank, kMaxRanks);
  PeerBarrierArgs p{};
  for (int r = 0; r < world; ++r) {
    if (!peer_flags[r]) return fail(GACB_ERR_INVALID_ARGUMENT, "peer_barrier: flag array of rank %d is NULL", r);
    p.peer_flags[r] = static_cast<uint32_t *>(peer_flags[r]);
  }
  p.local_flags = static_cast<uint32_t *>(local_flags);
  p.local_step = static_cast<uint32_t *>(local_step);
  p.status = status_word;
  p.world = world;
  p.rank = rank;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return check_cuda(cudaGetLastError(), "peer_barrier_kernel launch");
}
