// Split attention for callers that cannot allocate device memory.
//
// A key-split attention (`Attn::splits > 1`) needs scratch for its f32 partial
// results: `o_part [S,B,T,H,D]`, `m_part`, `l_part [S,B,T,H]`. The regular
// entry point takes that scratch from the caller. Some callers cannot provide
// it: code that runs while a stream is being captured or while a prepared plan
// is replayed has its device memory laid out ahead of time (svod plans every
// intermediate into one arena when a plan is prepared and allocates nothing
// when it executes), and `cudaMalloc` is not allowed there anyway: it
// synchronises the device and is illegal during capture. A decode step that
// finds out only at run time that it wants key splits is the typical case.
//
// `svodb_attention_splits_noalloc` serves them from a fixed scratch array that
// is part of the library image: every GPU that loads the library holds
// SVODB_NOALLOC_SCRATCH_BYTES of it until the process exits. The call
// allocates nothing (no cudaMalloc / cudaFree, no allocating library routine).
//
// Rules that follow from the array being shared:
//   * it is one array per device: calls that overlap on the GPU (two streams,
//     two threads) race on it; callers serialise them on one stream;
//   * it keeps the last call's contents. Nothing in it has to start at zero:
//     each call's kernels write every partial they later read (a share that saw
//     no key writes its sentinel maximum and zero sum), so no clearing is done;
//   * a shape whose partials do not fit is refused with SVODB_ERR_WORKSPACE.
//
// The first call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and caches it; make that
// first call before starting any stream capture.
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "kernels.h"
#include "svodb.h"

namespace {

constexpr size_t kScratchFloats = SVODB_NOALLOC_SCRATCH_BYTES / sizeof(float);

// The scratch itself. In host code this name is only a handle for the runtime
// (cudaGetSymbolAddress); it is never passed to a kernel as if it were a pointer.
static __device__ __align__(256) float g_split_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_mu;

// The device address of the scratch array on the current device, looked up once
// per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SVODB_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_split_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return SVODB_ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return SVODB_OK;
}

}  // namespace

extern "C" int svodb_attention_splits_noalloc(const svodb_tensor* q, const svodb_tensor* k, const svodb_tensor* v,
                                              const svodb_attn_opts* opts, svodb_tensor* o, void* stream) {
  if (q == nullptr || opts == nullptr || q->rank != 4)
    return svodb_attention(q, k, v, opts, o, stream);  // let the regular entry point report it
  svodb_attn_opts with_scratch = *opts;
  // the split count the attention will really run with (a request above the key
  // tile count is capped), so that what fits after capping is not refused
  int64_t keys = k != nullptr && k->rank == 4 ? k->shape[1] : 0;
  if (opts->has_cache && opts->cache_app_k != nullptr && opts->cache_app_k->rank == 4) keys += opts->cache_app_k->shape[1];
  const int splits = svodb::capped_splits(keys, opts->splits);
  if (splits > 1) {
    const size_t need = svodb_attention_workspace_bytes(q->shape[0], q->shape[1], q->shape[2], q->shape[3], splits);
    if (need > SVODB_NOALLOC_SCRATCH_BYTES) {
      svodb::set_last_error("attention: %d key splits of this shape need %zu scratch bytes, the built-in scratch holds %zu",
                           splits, need, (size_t)SVODB_NOALLOC_SCRATCH_BYTES);
      return SVODB_ERR_WORKSPACE;
    }
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != SVODB_OK) {
      svodb::set_last_error("attention: the built-in scratch array could not be located on this device");
      return rc;
    }
    with_scratch.workspace = scratch;
    with_scratch.workspace_bytes = SVODB_NOALLOC_SCRATCH_BYTES;
  }
  return svodb_attention(q, k, v, &with_scratch, o, stream);
}
