// mlops_fbla_decode_static: decode for callers that cannot allocate device memory.
//
// Some callers of this library have no way to obtain the decode scratch: code running where every device allocation
// was made up front and the allocator is closed (a serving engine that hands out a fixed arena at start-up, a plugin
// loaded into a host process that forbids cudaMalloc after initialisation, a real-time loop that must not enter the
// allocator's locks). For them this entry point runs the same four decode passes as mlops_fbla_decode on a scratch
// that is part of the library image: a file-scope device array of FBLA_STATIC_SCRATCH_BYTES (32 MiB) that every GPU
// holding the loaded library keeps until the process exits. Nothing here calls cudaMalloc, cudaFree or any
// allocating routine.
//
// The array's name is only a host-side handle; kernels need its device address, which differs per device. The first
// call on a device (with that device current) asks the runtime for it with cudaGetSymbolAddress, checks the answer
// and caches it. That first call should therefore be made before any stream capture begins on that device.
// "Allocates nothing" is about this library's calls: the CUDA driver itself commits the 32 MiB and the kernels' code
// when it first loads this module on a device (lazy loading, the default, does that at the first use). A caller whose
// arena will take all device memory calls mlops_fbla_decode_static_prepare() on every device at start-up, BEFORE it
// takes the arena (and before any capture): it forces that load and looks the address up, and launches nothing. The
// cached address does not survive cudaDeviceReset. Rejections of this entry point are reported by
// mlops_fbla_decode_static_error() (mlops_fbla_last_error() keeps the text of the ordinary entry points).
//
// All calls on one device share the one array. The decode passes write every scratch word before they read it and
// clear their own status word, so nothing has to be zeroed between calls and the previous call's contents are
// harmless; but two calls whose kernels overlap on the GPU (different streams, or concurrent host threads) would
// write the same words and race. Issue these calls on one stream, or order them yourself.
#include "../../../include/mlops_fbla.h"

#include <cstdio>
#include <mutex>

#define FBLA_STATIC_SCRATCH_BYTES (32u << 20)

static __device__ __align__(256) unsigned char fbla_static_scratch[FBLA_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void *g_scratch[kMaxDevices] = {nullptr};
thread_local char g_error[256] = {0};

// device address of the static scratch on the current device (set up once per device), or null with g_error set
void *static_scratch() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_error, sizeof g_error, "mlops_fbla_decode_static: no usable current device (%s)", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, fbla_static_scratch);
    if (e != cudaSuccess || !p) {
      snprintf(g_error, sizeof g_error, "mlops_fbla_decode_static: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch[dev] = p;
  }
  return g_scratch[dev];
}
}  // namespace

extern "C" size_t mlops_fbla_decode_static_scratch_limit(void) { return FBLA_STATIC_SCRATCH_BYTES; }

extern "C" mlops_fbla_status mlops_fbla_decode_static_prepare(void) {
  g_error[0] = 0;
  return static_scratch() ? MLOPS_FBLA_OK : MLOPS_FBLA_CUDA_ERROR;
}

extern "C" const char *mlops_fbla_decode_static_error(void) { return g_error; }

extern "C" mlops_fbla_status mlops_fbla_decode_static(const mlops_fbla_config *cfg, const uint16_t *q, const mlops_fbla_cache *cache,
                                                       uint16_t *output, cudaStream_t stream) {
  g_error[0] = 0;
  const size_t need = mlops_fbla_decode_scratch_bytes(cfg);
  if (need == 0) {
    snprintf(g_error, sizeof g_error, "mlops_fbla_decode_static: invalid configuration");
    return MLOPS_FBLA_INVALID_VALUE;
  }
  if (need > FBLA_STATIC_SCRATCH_BYTES) {
    snprintf(g_error, sizeof g_error, "mlops_fbla_decode_static: this decode needs %zu bytes of scratch, the built-in scratch holds %u; "
             "use mlops_fbla_decode with a caller-provided scratch", need, FBLA_STATIC_SCRATCH_BYTES);
    return MLOPS_FBLA_INVALID_VALUE;
  }
  void *scratch = static_scratch();
  if (!scratch) return MLOPS_FBLA_CUDA_ERROR;
  const mlops_fbla_status st = mlops_fbla_decode(cfg, q, cache, output, scratch, FBLA_STATIC_SCRATCH_BYTES, stream);
  if (st != MLOPS_FBLA_OK) snprintf(g_error, sizeof g_error, "%s", mlops_fbla_last_error());
  return st;
}
