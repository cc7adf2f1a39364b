// Host-side runtime of the kernel library: last-error string, TMA descriptor
// encoding, the device status word written by bounded waits.
#include "host.h"

#include <mutex>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

namespace ksa {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available from the driver");
    return kErrNoDriver;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i];
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_last_error("TMA base address %p is not 16-byte aligned", base);
    return kErrArgument;
  }
  for (int i = 1; i < rank; ++i) {
    if (strides_bytes[i] % 16 != 0) {
      set_last_error("TMA stride %d = %llu bytes is not a multiple of 16", i, (unsigned long long)strides_bytes[i]);
      return kErrArgument;
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)", (int)r,
                   rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0), box[0],
                   rank > 1 ? box[1] : 0);
    return kErrCuda;
  }
  return kErrNone;
}

int ensure_device(const void* device_ptr) {
  static thread_local int bound_device = -1;
  if (bound_device >= 0 || device_ptr == nullptr) return kErrNone;
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, device_ptr);
  if (e != cudaSuccess || (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged)) {
    cudaGetLastError();
    set_last_error("pointer %p is not device memory (%s)", device_ptr, e == cudaSuccess ? "host pointer" : cudaGetErrorString(e));
    return kErrArgument;
  }
  e = cudaSetDevice(attr.device);
  if (e != cudaSuccess) {
    set_last_error("cudaSetDevice(%d) failed: %s", attr.device, cudaGetErrorString(e));
    return kErrCuda;
  }
  cudaFree(0);  // force the primary context to be current on this thread
  bound_device = attr.device;
  return kErrNone;
}

constexpr long long kDefaultPeerWaitMs = 10000;   // 10 s
static int* g_status[64] = {nullptr};
static std::mutex g_status_mu;

int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    // word 1: limit of waits on flags written by OTHER GPUs, in units of 2^20 clock cycles (0 = the built-in limit).
    // Ranks drift apart on the host (graph capture, a slow data loader), so this limit is longer than the one of the
    // waits inside a kernel; KSA_PEER_WAIT_MS overrides it, ksa_set_peer_wait_ms changes it at run time.
    int units = (int)(kDefaultPeerWaitMs * 2000LL / 1049);      // ~2 GHz: 2e6 cycles per ms
    if (const char* e = getenv("KSA_PEER_WAIT_MS")) {
      const long long ms = atoll(e);
      if (ms > 0) units = (int)(ms * 2000LL / 1049 + 1);
    }
    cudaMemcpy(p + 1, &units, sizeof(int), cudaMemcpyHostToDevice);
    g_status[dev] = p;
  }
  return g_status[dev];
}

}  // namespace ksa

KSA_API const char* ksa_last_error() { return ksa::g_last_error; }

// Address of the status word of the current device (for torch to wrap / read).
KSA_API void* ksa_status_ptr() { return ksa::status_word(); }

// Read and clear the status word (synchronises the device).  Returns the status, or -1 on a CUDA error.
KSA_API int ksa_read_status(int clear) {
  int* p = ksa::status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (clear && v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

// Limit (milliseconds at ~2 GHz) of device-side waits on flags written by other GPUs, for the current device.
KSA_API int ksa_set_peer_wait_ms(int ms) {
  int* p = ksa::status_word();
  if (!p || ms <= 0) return -1;
  const int units = (int)((long long)ms * 2000LL / 1049 + 1);
  return cudaMemcpy(p + 1, &units, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
}

namespace ksa {
static bool g_dependent_launch = false;
bool dependent_launch_enabled() { return g_dependent_launch; }
}  // namespace ksa

// Switch dependent launches of the decode-step kernels on (1) or off (0); returns the previous setting.
KSA_API int ksa_set_dependent_launch(int on) {
  const int before = ksa::g_dependent_launch ? 1 : 0;
  ksa::g_dependent_launch = on != 0;
  return before;
}

KSA_API int ksa_abi_version() { return 1; }
