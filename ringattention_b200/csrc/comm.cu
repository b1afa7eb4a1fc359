// Symmetric-memory substrate for the fused ring kernels: device allocations exported to the
// other ranks of a node with CUDA IPC, a flag barrier whose waits are bounded, and a peer copy
// kernel (used by the bandwidth probe and by tests).
//
// Flag protocol: every rank owns `flags[N]` in its own memory. In barrier number `epoch` rank r
// stores `epoch` into flags[r] of every peer (release, system scope) and then waits until its own
// flags[p] >= epoch for every p (acquire, system scope). A wait that exceeds `timeout_ns` records
// kTimeoutPeerFlag in the status word and the kernel returns; nothing spins forever.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common/host_util.h"
#include "common/sm100.cuh"

namespace ra {
namespace comm {

// `epoch_ptr` (optional, local device memory) replaces the host-supplied epoch: the kernel uses
// *epoch_ptr + 1 and stores it back, so a launch recorded in a CUDA graph works on every replay.
__global__ void barrier_kernel(uint32_t* const* __restrict__ peer_flags, int rank, int n, uint32_t epoch,
                               unsigned long long timeout_ns, int* status, uint32_t* epoch_ptr) {
  const int t = threadIdx.x;
  if (epoch_ptr) epoch = *epoch_ptr + 1;
  __syncthreads();
  if (t < n) {
    __threadfence_system();
    uint32_t* remote = peer_flags[t] + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = peer_flags[rank] + t;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (((++it) & 255u) == 0u && globaltimer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, static_cast<int>(kTimeoutPeerFlag));
        break;
      }
      __nanosleep(200);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (epoch_ptr && t == 0) *epoch_ptr = epoch;
}

__global__ void copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

// rows x row16 units of 16 bytes; source and destination rows are src_ld16 / dst_ld16 units apart.
__global__ void copy_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, unsigned int rows,
                                 unsigned int row16, long long src_ld16, long long dst_ld16) {
  const unsigned long long total = static_cast<unsigned long long>(rows) * row16;
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < total; i += 4 * stride) {
    uint4 v[4];
    unsigned long long o[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned long long j = i + u * stride;
      const unsigned long long r = j / row16;
      const unsigned int c = static_cast<unsigned int>(j - r * row16);
      v[u] = src[r * src_ld16 + c];
      o[u] = r * dst_ld16 + c;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) dst[o[u]] = v[u];
  }
  for (; i < total; i += stride) {
    const unsigned long long r = i / row16;
    const unsigned int c = static_cast<unsigned int>(i - r * row16);
    dst[r * dst_ld16 + c] = src[r * src_ld16 + c];
  }
}

}  // namespace comm
}  // namespace ra

using namespace ra;

// Copy `rows` rows of `row_bytes` bytes between strided buffers (leading dimensions in bytes); everything a
// multiple of 16 bytes. Used to stage the K/V rows of a fused (B, S, 3, H, D) projection into the symmetric slot.
extern "C" int ra_copy_rows(const void* src, void* dst, long long rows, long long row_bytes, long long src_ld,
                            long long dst_ld, void* stream) {
  if (rows <= 0 || row_bytes <= 0 || (row_bytes % 16) || (src_ld % 16) || (dst_ld % 16) || rows >= (1ll << 32) ||
      row_bytes / 16 >= (1ll << 32) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_error("ra_copy_rows: sizes, strides and addresses must be multiples of 16 bytes");
    return kHostBadArg;
  }
  const long long total = rows * (row_bytes / 16);
  long long blocks = (total + 4 * 256 - 1) / (4 * 256);
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  comm::copy_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), static_cast<unsigned int>(rows),
      static_cast<unsigned int>(row_bytes / 16), src_ld / 16, dst_ld / 16);
  return check_launch("copy_rows_kernel");
}

extern "C" int ra_symm_alloc(unsigned long long bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    set_error("ra_symm_alloc: cudaMalloc failed");
    return kHostTooLarge;
  }
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    set_error("ra_symm_alloc: cudaMemset failed");
    return kHostLaunchFail;
  }
  *out = p;
  return kHostOk;
}
extern "C" int ra_symm_free(void* p) {
  return cudaFree(p) == cudaSuccess ? kHostOk : kHostLaunchFail;
}
// handle_out: 64 bytes (cudaIpcMemHandle_t)
extern "C" int ra_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    set_error(cudaGetErrorString(e));
    cudaGetLastError();
    return kHostLaunchFail;
  }
  memcpy(handle_out, &h, sizeof(h));
  return kHostOk;
}
extern "C" int ra_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error(cudaGetErrorString(e));
    cudaGetLastError();
    return kHostLaunchFail;
  }
  *out = p;
  return kHostOk;
}
extern "C" int ra_ipc_close(void* p) {
  return cudaIpcCloseMemHandle(p) == cudaSuccess ? kHostOk : kHostLaunchFail;
}

// peer_flags: device array of n pointers (one per rank, in this process' address space).
extern "C" int ra_symm_barrier(void* const* peer_flags, int rank, int n, unsigned int epoch,
                               unsigned long long timeout_ns, int* status, void* stream,
                               unsigned int* epoch_ptr) {
  if (n < 1 || n > 32 || rank < 0 || rank >= n) {
    set_error("ra_symm_barrier: bad rank/size");
    return kHostBadArg;
  }
  comm::barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint32_t* const*>(peer_flags), rank, n, epoch, timeout_ns, status, epoch_ptr);
  return check_launch("barrier_kernel");
}

extern "C" int ra_peer_copy(const void* src, void* dst, long long bytes, int ctas, void* stream) {
  if (bytes % 16 || ctas < 1) {
    set_error("ra_peer_copy: size must be a multiple of 16");
    return kHostBadArg;
  }
  comm::copy_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), bytes / 16);
  return check_launch("copy_kernel");
}
