// Host-side helpers shared by the launchers: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda), error reporting, and
// the per-device status word that bounded waits write to.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define KSA_API extern "C" __attribute__((visibility("default")))

namespace ksa {

// Error codes returned by the C entry points (0 = success).
enum HostError : int {
  kErrNone = 0,
  kErrCuda = -1,       // a CUDA runtime/driver call failed; see ksa_last_error()
  kErrArgument = -2,   // unsupported shape / alignment / size
  kErrNoDriver = -3,   // cuTensorMapEncodeTiled could not be resolved
};

void set_last_error(const char* fmt, ...);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// Encode a bf16 (elem_bytes = 2) or fp32 (4) tiled tensor map with a 128-byte swizzle.
// dims / strides are innermost-first; strides[0] is implied (element size) and strides[i>0] are bytes.
int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

// Device status word for the current device (allocated once per device on first use).
int* status_word();

// Make the device that owns `device_ptr` current on the calling thread.  Callers may arrive on threads that have
// never touched CUDA through this library's runtime (autograd worker threads): without this, descriptor encoding
// fails for lack of a context and launches would go to device 0.  Cached per thread; returns 0 on success.
int ensure_device(const void* device_ptr);

#define KSA_ENTER(ptr)                                   \
  do {                                                   \
    int _rc = ksa::ensure_device(ptr);                   \
    if (_rc) return _rc;                                 \
  } while (0)

#define KSA_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      ksa::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return ksa::kErrCuda;                                                               \
    }                                                                                     \
  } while (0)

// Dependent launches (programmatic stream serialization).  While the switch is on (ksa_set_dependent_launch), the
// kernels of the decode step are launched so that each may start while its predecessor on the stream still runs;
// every such kernel calls grid_dependency_wait() before it touches memory an earlier kernel may write.  Off by
// default: training steps launch the same kernels the ordinary way.
bool dependent_launch_enabled();

template <typename Kern, typename... Args>
inline cudaError_t launch_kernel(bool dependent, Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

#define KSA_REQUIRE(cond, ...)                  \
  do {                                          \
    if (!(cond)) {                              \
      ksa::set_last_error(__VA_ARGS__);         \
      return ksa::kErrArgument;                 \
    }                                           \
  } while (0)

}  // namespace ksa
