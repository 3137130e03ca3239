// ri_wave_decode_layer_static: the fused decode step for callers that may not allocate.
//
// Who needs this: serving runtimes that hand the whole of HBM to their own memory pool when they
// start (after which a cudaMalloc from a plug-in simply fails), and decode loops that ban driver
// allocation calls because cudaMalloc and cudaFree stall every stream of the device while they
// run.  Such a caller has nowhere to get the ~8 MB of scratch that ri_wave_decode_layer expects
// in `d_scratch`.  Here the scratch is a fixed array that is part of the library image itself:
// the driver sets it aside once, when the library is loaded onto a GPU, and it stays there until
// the process exits.
//
// Rules that follow from sharing one array:
//  * Geometries whose scratch would exceed RI_WAVE_STATIC_SCRATCH_BYTES are refused.
//  * Every call (any layer, any stream, any thread) uses the same bytes and finds whatever the
//    previous call left.  That is harmless: each stage writes everything a later stage reads, so
//    no part of the array has to be initialised.
//  * Two calls whose GPU work overlaps in time (different streams, or different host threads
//    without ordering) would overwrite each other's intermediate results.  Order them.
//  * The device address of the array is looked up on the first call made on each device, with
//    that device current.  Make that first call during start-up, outside any stream capture.
#include <mutex>

#include "ri_common.cuh"

namespace {

// The name below is only a host-side handle; it is not a device pointer.  Host code must ask
// the runtime for the array's device address (cudaGetSymbolAddress) and pass that to kernels.
static __device__ __align__(256) unsigned char g_static_scratch[RI_WAVE_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_addr_mutex;

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  RI_CUDA_OK(cudaGetDevice(&dev));
  RI_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d beyond the %d this entry point tracks", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_addr_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* addr = nullptr;
    RI_CUDA_OK(cudaGetSymbolAddress(&addr, g_static_scratch));
    RI_REQUIRE(addr != nullptr, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return RI_OK;
}

}  // namespace

extern "C" int ri_wave_decode_layer_static(const ri_wave_layer* p, void* stream) {
  RI_REQUIRE(p != nullptr, "ri_wave_layer is null");
  const int64_t need = ri_wave_scratch_bytes(p);
  if (need < 0) return (int)need;   // geometry rejected; message already set
  RI_REQUIRE(need <= (int64_t)RI_WAVE_STATIC_SCRATCH_BYTES,
             "this geometry needs %lld bytes of scratch, the built-in array holds %lld; "
             "use ri_wave_decode_layer with caller-provided scratch",
             (long long)need, (long long)RI_WAVE_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != RI_OK) return rc;
  ri_wave_layer q = *p;
  q.d_scratch = scratch;
  return ri_wave_decode_layer(&q, stream);
}
