// Forest forward for callers that cannot hand the library any scratch memory.
//
// ht_forest_forward_f32 needs a caller-provided workspace (compact feature indices and the
// per-tree records of the tile kernel).  Some callers have no way to provide one: code that
// runs inside a region where device allocation is forbidden or must not be triggered (a
// real-time inference loop with a frozen memory pool, a plugin host that only passes input
// and output buffers through, a runtime whose allocator the binding cannot reach).  For them
// the entry point below keeps that scratch in a fixed array that is part of the loaded
// library image on every device, and otherwise behaves exactly like ht_forest_forward_f32.
#include "ht_common.cuh"

#include <mutex>

namespace {

// Scratch shared by every call on a device.  16 MiB covers, for example, 1024 trees of depth 10
// or 4096 trees of depth 8.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_forest_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_address[kMaxDevices] = {};

// Device address of the scratch array on the current device.  `g_forest_scratch` in host code is
// only a handle for the runtime, not an address a kernel could use; the address is looked up
// once per device, with that device current.  The cached address lives as long as the device's
// primary context: a caller that destroys it (cudaDeviceReset) must not call this entry again.
int resolve_scratch(void **address) {
  int device = 0;
  HT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return HT_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void *ptr = nullptr;
    HT_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_forest_scratch));
    if (ptr == nullptr) return HT_ERR_CUDA;
    g_scratch_address[device] = ptr;
  }
  *address = g_scratch_address[device];
  return HT_OK;
}

}  // namespace

extern "C" {

size_t ht_forest_static_scratch_bytes(void) { return kStaticScratchBytes; }

int ht_forest_forward_static_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                                 const float *w, float *out, uint32_t *status_word, ht_stream_t stream) {
  const int rc = ht::check_forest_problem(p);
  if (rc != HT_OK) return rc;
  // the forward needs no backward records: size the request without them, whatever the caller's flags say
  ht_forest_problem forward_only = *p;
  forward_only.flags &= ~HT_WORKSPACE_FOR_BACKWARD;
  if (ht_forest_workspace_bytes(&forward_only) > kStaticScratchBytes) return HT_ERR_WORKSPACE;
  void *scratch = nullptr;
  const int src = resolve_scratch(&scratch);
  if (src != HT_OK) return src;
  return ht_forest_forward_f32(&forward_only, x, thr, ord, w, out, scratch, kStaticScratchBytes, status_word, stream);
}

}  // extern "C"
