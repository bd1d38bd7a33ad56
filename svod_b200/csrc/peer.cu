// The path's one collective as kernels of this library: an all-gather of pooled
// rows [rows, d] f32 over NVLink peer memory, with plain stores into the peers'
// staging buffers (no multimem, no multicast loads, no library collective).
//
// Every rank owns, in memory the others have mapped (CUDA IPC):
//   stage  [2 parities][world][rows][d] f32 — where the peers put their rows;
//   flags  [world] u32 — flags[q] = how many steps rank q has delivered here;
// and privately `local` = {steps completed, rows pushed, peers unstaged}.
//
// Step s on rank r, two launches on the caller's stream:
//   push   (one block per row): the row goes into stage[s & 1][r] of every peer;
//          a system-scope fence, then the block counts itself; the block that
//          counts last fences again and writes s + 1 into flags[r] of every peer.
//   unstage (one block per peer q): waits — with a limit, after which it reports
//          through the status word and copies nothing — until flags[q] >= s + 1,
//          then copies q's rows from the local stage into the gathered buffer; the
//          block that finishes last publishes s + 1 as the steps completed.
// A peer overwrites parity s & 1 of this rank's stage at its step s + 2 at the
// earliest, which it reaches only after this rank has delivered step s + 1, that is
// after this rank's unstage of step s has finished: two parities are enough.
// The two kernels of one rank never wait for each other (stream order); the only
// wait is for a flag another GPU writes.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "svodb.h"

namespace svodb {

namespace {

struct PeerParams {
  int world, rank;
  float* stage[8];
  uint32_t* flags[8];
  uint32_t* local;
};

__global__ void __launch_bounds__(256)
    peer_push_kernel(const PeerParams pg, const float* __restrict__ mine, int64_t rows, int d) {
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(pg.local);
  const int64_t row = blockIdx.x;
  const size_t slot = (((size_t)(step & 1u) * pg.world + pg.rank) * rows + row) * d;
  const float4* src = reinterpret_cast<const float4*>(mine + row * d);
  for (int p = 0; p < pg.world; ++p) {
    if (p == pg.rank) continue;
    float4* dst = reinterpret_cast<float4*>(pg.stage[p] + slot);
    for (int c = threadIdx.x; c < d / 4; c += blockDim.x) dst[c] = src[c];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool last = atomicAdd(&pg.local[1], 1u) == gridDim.x - 1;
    if (last) {
      __threadfence_system();
      for (int p = 0; p < pg.world; ++p)
        if (p != pg.rank) *reinterpret_cast<volatile uint32_t*>(pg.flags[p] + pg.rank) = step + 1u;
      pg.local[1] = 0u;
    }
  }
}

__global__ void __launch_bounds__(256)
    peer_unstage_kernel(const PeerParams pg, float* __restrict__ gathered, int64_t rows, int d, uint32_t wait_polls,
                        uint32_t* status) {
  __shared__ int arrived;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(pg.local);
  const int q = (int)blockIdx.x + ((int)blockIdx.x >= pg.rank ? 1 : 0);
  if (threadIdx.x == 0) {
    const volatile uint32_t* flag = pg.flags[pg.rank] + q;
    int ok = 0;
    for (uint32_t n = 0; n < wait_polls; ++n) {
      if (*flag >= step + 1u) {
        ok = 1;
        break;
      }
      __nanosleep(256);
    }
    if (!ok) atomicExch(status, (uint32_t)kStatusWaitTimeout);
    arrived = ok;
  }
  __syncthreads();
  if (arrived) {
    __threadfence_system();
    const size_t n4 = (size_t)rows * d / 4;
    const float4* src = reinterpret_cast<const float4*>(pg.stage[pg.rank] + ((size_t)(step & 1u) * pg.world + q) * rows * d);
    float4* dst = reinterpret_cast<float4*>(gathered + (size_t)q * rows * d);
    for (size_t c = threadIdx.x; c < n4; c += blockDim.x) dst[c] = src[c];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&pg.local[2], 1u) == gridDim.x - 1) {
      pg.local[2] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(pg.local) = step + 1u;
    }
  }
}

}  // namespace

}  // namespace svodb

using namespace svodb;

extern "C" {

size_t svodb_peer_stage_bytes(int32_t world, int64_t rows, int64_t d) {
  if (world < 1 || rows < 0 || d < 0) return 0;
  return (size_t)2 * world * rows * d * sizeof(float);
}

int svodb_ipc_export(const void* dev_ptr, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
  if (dev_ptr == nullptr || handle == nullptr) {
    set_last_error("ipc_export: null argument");
    return SVODB_ERR_SHAPE;
  }
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(dev_ptr));
  if (e != cudaSuccess) {
    set_last_error("ipc_export: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return SVODB_ERR_LAUNCH;
  }
  memcpy(handle, &h, 64);
  return SVODB_OK;
}

int svodb_ipc_open(const uint8_t handle[64], void** out) {
  if (handle == nullptr || out == nullptr) {
    set_last_error("ipc_open: null argument");
    return SVODB_ERR_SHAPE;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  const cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_last_error("ipc_open: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return SVODB_ERR_LAUNCH;
  }
  return SVODB_OK;
}

int svodb_ipc_close(void* ptr) {
  if (ptr == nullptr) return SVODB_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    set_last_error("ipc_close: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return SVODB_ERR_LAUNCH;
  }
  return SVODB_OK;
}

int svodb_memset(void* ptr, int32_t value, size_t bytes, void* stream) {
  if (bytes == 0) return SVODB_OK;
  if (ptr == nullptr) {
    set_last_error("memset: null pointer");
    return SVODB_ERR_SHAPE;
  }
  const cudaError_t e = cudaMemsetAsync(ptr, value, bytes, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_last_error("memset: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return SVODB_ERR_LAUNCH;
  }
  return SVODB_OK;
}

int svodb_peer_all_gather(const svodb_peer_gather* pg, const float* mine, float* gathered, int64_t rows, int64_t d,
                          void* stream) {
  if (pg == nullptr || mine == nullptr || gathered == nullptr) {
    set_last_error("peer_all_gather: null argument");
    return SVODB_ERR_SHAPE;
  }
  if (pg->world < 1 || pg->world > 8 || pg->rank < 0 || pg->rank >= pg->world || rows <= 0 || d <= 0 || d % 4 != 0 ||
      (reinterpret_cast<uintptr_t>(mine) & 15) != 0 || (reinterpret_cast<uintptr_t>(gathered) & 15) != 0) {
    set_last_error("peer_all_gather: world %d rank %d rows %lld d %lld (world <= 8, d a multiple of 4, 16-byte aligned rows)",
                   pg->world, pg->rank, (long long)rows, (long long)d);
    return SVODB_ERR_SHAPE;
  }
  if (pg->world == 1) return SVODB_OK;  // nothing to exchange: the rows are where they belong
  PeerParams p{};
  p.world = pg->world, p.rank = pg->rank;
  for (int i = 0; i < pg->world; ++i) {
    if (pg->stage[i] == nullptr || pg->flags[i] == nullptr) {
      set_last_error("peer_all_gather: rank %d's buffers are not mapped", i);
      return SVODB_ERR_SHAPE;
    }
    p.stage[i] = (float*)pg->stage[i];
    p.flags[i] = (uint32_t*)pg->flags[i];
  }
  if (pg->local == nullptr) {
    set_last_error("peer_all_gather: no local counters");
    return SVODB_ERR_SHAPE;
  }
  p.local = (uint32_t*)pg->local;
  cudaStream_t s = (cudaStream_t)stream;
  // ~256 ns a poll: the limit is a few seconds, after which the step reports a timeout
  const uint32_t polls = pg->wait_polls > 0 ? pg->wait_polls : (16u << 20);
  if (pg->phases != 2) peer_push_kernel<<<(unsigned)rows, 256, 0, s>>>(p, mine, rows, (int)d);
  if (pg->phases != 1)
    peer_unstage_kernel<<<(unsigned)(pg->world - 1), 256, 0, s>>>(p, gathered, rows, (int)d, polls, device_status_word());
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("peer_all_gather: %s", cudaGetErrorString(e));
    return SVODB_ERR_LAUNCH;
  }
  return SVODB_OK;
}

}  // extern "C"
