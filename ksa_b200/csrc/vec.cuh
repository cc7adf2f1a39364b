// 16-byte bf16 vector loads/stores and block-wide reductions shared by the row-wise kernels.
#pragma once
#include "common.cuh"

namespace ksa {

struct alignas(16) BF8 {
  uint32_t u[4];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  BF8 v = *reinterpret_cast<const BF8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = unpack_bf16x2(v.u[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  BF8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.u[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<BF8*>(p) = v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : 0.f;
  return warp_sum(t);
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? red[lane] : -INFINITY;
  return warp_max(t);
}

}  // namespace ksa
