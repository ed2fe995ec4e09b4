// fdb_attn_fwd_static: the fused forward with its scratch in a fixed device array instead of a caller workspace.
//
// Meant for hosts that cannot allocate device memory where they call the library (a server whose arena already owns
// the GPU, a plug-in inside a latency-critical loop where cudaMalloc/cudaFree would synchronise the device, a bare C
// host without an allocator).  The array below is part of the library image: every GPU that loads the library holds
// kScratchBytes of it until the process exits.
//
// g_scratch is a device symbol.  In host code its name is only a handle (a host-side shadow), not a device address, so
// it is never passed to a kernel directly: the address is looked up once per device with cudaGetSymbolAddress, with
// that device current, and that pointer is what the launchers receive.
#include <cuda_runtime.h>

#include <mutex>

#include "internal.h"

namespace fdb {
namespace {

constexpr size_t kScratchBytes = FDB_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_scratch on the current device (looked up on the first call per device).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FDB_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(FDB_ERR_LIMIT, "device ordinal %d outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(FDB_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return FDB_OK;
}

}  // namespace
}  // namespace fdb

using namespace fdb;

extern "C" FDB_API int fdb_attn_fwd_static(const fdb_attn_params* p, void* stream) {
  clear_error();
  int rc = validate(p, true);
  if (rc != FDB_OK) return rc;
  if (p->batch == 0 || p->total_rows == 0) return FDB_OK;
  ExpandGeometry g = {0, 0, 0, 0};
  if (p->pos_key != nullptr || p->pos_query != nullptr) g = expand_geometry(p->lut_d_min, p->lut_len);
  const WorkspaceLayout w = workspace_layout(*p, g, /*allow_split=*/false);  // no room for partial results
  if (w.total > kScratchBytes)
    return fail(FDB_ERR_LIMIT,
                "these parameters need %llu bytes of scratch, the built-in array holds %llu (FDB_STATIC_SCRATCH_BYTES); "
                "use fdb_attn_fwd with a caller workspace",
                (unsigned long long)w.total, (unsigned long long)kScratchBytes);
  void* scratch = nullptr;
  if ((rc = scratch_for_current_device(&scratch)) != FDB_OK) return rc;
  fdb_attn_params q = *p;  // same call, scratch swapped in
  q.workspace = scratch;
  q.workspace_bytes = kScratchBytes;
  q.prepared = 0;  // the scratch is shared by every call on this device
  q.tune = (p->tune & ~FDB_TUNE_TWO_LAUNCHES) | FDB_TUNE_ONE_LAUNCH;  // one launch: no partial-result buffers
  // Nothing in the scratch has to start at zero: seq_info_kernel and expand_tables_kernel write every entry the fused
  // kernel reads, on this stream, before it runs.
  if ((rc = launch_prepare(q, g, w, stream)) != FDB_OK) return rc;
  return launch_attn_fwd_sm100(q, g, w, stream);
}
