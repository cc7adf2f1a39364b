// RMSNorm backward that allocates nothing: the scratch for the per-CTA partial sums of the
// weight gradient is a fixed array inside the library image (see noalloc.h for who needs
// this and for the contract).  The arithmetic is the same as rmsnorm_bwd_kernel +
// colsum_partials_kernel in elementwise.cu; only the home of the scratch differs.
#include "noalloc.h"

#include <mutex>

#include "common.cuh"
#include "host.h"

namespace ksa {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = KSA_NOALLOC_RMSNORM_MAX_D / (kThreads * 8);  // 16-byte vectors per thread
static_assert(kMaxVec * kThreads * 8 == KSA_NOALLOC_RMSNORM_MAX_D, "max D must be a multiple of 2048");

// Scratch shared by every call on this device: [MAX_PARTS][MAX_D] fp32, 2.4 MB, lives as long as the process.
// In host code this name is only a handle for cudaGetSymbolAddress; the kernels get the device address as an argument.
static __device__ __align__(256) float g_dw_partial[KSA_NOALLOC_RMSNORM_MAX_PARTS * KSA_NOALLOC_RMSNORM_MAX_D];

__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(u[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void st8(bf16* p, const float (&f)[8]) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const float t = (lane < kThreads / 32) ? red[lane] : 0.f;
  return warp_sum(t);
}

// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and writes ONE full row of D partial sums to
// partial[blockIdx.x * D ...]; every element the reduction kernel reads is therefore written by this launch.
__global__ void __launch_bounds__(kThreads)
rmsnorm_bwd_static_scratch_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                  const float* __restrict__ rstd_in, const bf16* __restrict__ dres,
                                  bf16* __restrict__ dx, float* __restrict__ partial, int rows, int D) {
  __shared__ float red[32];
  float wv[kMaxVec][8], dw[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
    if (c < D) ld8(w + c, wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = (long long)row * D;
    const float rstd = rstd_in[row];
    float xh[kMaxVec][8], g[kMaxVec][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < D) {
        float xv[8], dyv[8];
        ld8(x + base + c, xv);
        ld8(dy + base + c, dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * rstd;
          g[i][j] = dyv[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
          dw[i][j] += dyv[j] * xh[i][j];
        }
      }
    }
    dot = cta_sum(dot, red) / (float)D;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = (i * kThreads + threadIdx.x) * 8;
      if (c < D) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float r[8];
          ld8(dres + base + c, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        st8(dx + base + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < D) {
      float* p = partial + (long long)blockIdx.x * D + c;
      *reinterpret_cast<float4*>(p) = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

__global__ void colsum_static_scratch_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts,
                                             int D, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * D + c];
  dw[c] = accumulate ? dw[c] + s : s;
}

// Device address of g_dw_partial on the current device, looked up once per device.
int scratch_address(float** out) {
  static float* addr[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  KSA_CHECK_CUDA(cudaGetDevice(&dev));
  KSA_REQUIRE(dev >= 0 && dev < 64, "rmsnorm_bwd_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (addr[dev] == nullptr) {
    float* p = nullptr;
    KSA_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partial));
    KSA_REQUIRE(p != nullptr, "rmsnorm_bwd_noalloc: cudaGetSymbolAddress returned a null address");
    addr[dev] = p;
  }
  *out = addr[dev];
  return kErrNone;
}

}  // namespace
}  // namespace ksa

extern "C" int ksa_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const void* rstd,
                                       const void* dres, void* dx, void* dw, int accumulate_dw, int rows, int D,
                                       void* stream) {
  using namespace ksa;
  KSA_REQUIRE(rows >= 0, "rmsnorm_bwd_noalloc: rows = %d is negative", rows);
  KSA_REQUIRE(D > 0 && D % 8 == 0, "rmsnorm_bwd_noalloc: D = %d must be a positive multiple of 8", D);
  KSA_REQUIRE(D <= KSA_NOALLOC_RMSNORM_MAX_D,
              "rmsnorm_bwd_noalloc: D = %d exceeds the built-in scratch (max D = %d); use ksa_rmsnorm_bwd with a "
              "caller-provided buffer instead", D, KSA_NOALLOC_RMSNORM_MAX_D);
  KSA_REQUIRE(dy && x && w && rstd && dx, "rmsnorm_bwd_noalloc: null input/output pointer");
  if (rows == 0) return kErrNone;
  float* scratch = nullptr;
  const int rc = scratch_address(&scratch);
  if (rc != kErrNone) return rc;
  const int parts = rows < KSA_NOALLOC_RMSNORM_MAX_PARTS ? rows : KSA_NOALLOC_RMSNORM_MAX_PARTS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  rmsnorm_bwd_static_scratch_kernel<<<parts, kThreads, 0, st>>>(
      static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w),
      static_cast<const float*>(rstd), static_cast<const bf16*>(dres), static_cast<bf16*>(dx), scratch, rows, D);
  KSA_CHECK_CUDA(cudaGetLastError());
  if (dw != nullptr) {
    colsum_static_scratch_kernel<<<(D + 255) / 256, 256, 0, st>>>(scratch, static_cast<float*>(dw), parts, D,
                                                                  accumulate_dw);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  return kErrNone;
}
