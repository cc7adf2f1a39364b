// Skinny GEMM for decoding: C[M, N] = A[M, K] * B[N, K]^T with M <= 16 rows (one token per sequence of the batch).
// The work is a stream of the weight matrix B, so the kernel is laid out for memory bandwidth, not for the tensor
// cores: every CTA owns a slab of output columns small enough that the grid covers all SMs several times (a 128-row
// MMA tile would leave N/256 = 10 CTAs busy for a 2560-wide projection), each warp streams whole weight rows with
// 16-byte loads, the activation rows sit in shared memory, and the dot products are accumulated in fp32.
#include "common.cuh"
#include "host.h"

namespace ksa {

constexpr int kGemvThreads = 256;
constexpr int kGemvKTile = 2048;   // activation columns staged in shared memory per pass

// 16-byte read-only load that does not pollute L1: every weight byte is used once per step
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int MT, int R>
__global__ void __launch_bounds__(kGemvThreads)
gemv_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, int M, int N, int K,
            long long lda, long long ldb, long long ldc) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  bf16* sA = reinterpret_cast<bf16*>(gemv_smem);           // [MT][kGemvKTile]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * (kGemvThreads / 32) + warp) * R;
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kGemvKTile) {
    const int kt = min(kGemvKTile, K - k0);          // multiple of 8
    __syncthreads();
    for (int i = threadIdx.x; i < MT * (kGemvKTile / 8); i += kGemvThreads) {
      const int m = i / (kGemvKTile / 8), c = (i % (kGemvKTile / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < M && c < kt) v = *reinterpret_cast<const uint4*>(A + (long long)m * lda + k0 + c);
      *reinterpret_cast<uint4*>(sA + m * kGemvKTile + c) = v;
    }
    __syncthreads();
    // U chunks of every row are requested before any is used, so that enough loads are in flight per SM
    constexpr int U = (R >= 4) ? 2 : (R == 2 ? 4 : 8);
    for (int c0 = lane * 8; c0 < kt; c0 += 256 * U) {
      uint4 w[U][R];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int c = c0 + u * 256;
          w[u][r] = make_uint4(0, 0, 0, 0);
          if (c < kt && n0 + r < N) w[u][r] = ld_stream_16(B + (long long)(n0 + r) * ldb + k0 + c);
        }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * 256;
        if (c >= kt) break;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4 a = *reinterpret_cast<const uint4*>(sA + m * kGemvKTile + c);
          const uint32_t au[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const uint32_t wu[4] = {w[u][r].x, w[u][r].y, w[u][r].z, w[u][r].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 x = unpack_bf16x2(au[q]), y = unpack_bf16x2(wu[q]);
              acc[r][m] = fmaf(x.x, y.x, acc[r][m]);
              acc[r][m] = fmaf(x.y, y.y, acc[r][m]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float v = warp_sum(acc[r][m]);
      if (lane == 0 && m < M && n0 + r < N) C[(long long)m * ldc + n0 + r] = __float2bfloat16(v);
    }
}

template <int MT, int R>
static int launch_gemv(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, cudaStream_t st) {
  const int rows_per_cta = (kGemvThreads / 32) * R;
  const size_t smem = (size_t)MT * kGemvKTile * sizeof(bf16);
  auto kern = gemv_kernel<MT, R>;
  static bool attr = false;
  if (!attr && smem > 48 * 1024) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = true;
  }
  kern<<<(N + rows_per_cta - 1) / rows_per_cta, kGemvThreads, smem, st>>>((const bf16*)a, (const bf16*)b, (bf16*)c, M, N, K,
                                                                          lda, ldb, ldc);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace ksa

// C[M, N] (bf16, ldc) = A[M, K] (bf16, lda) * B[N, K]^T (bf16, ldb) for 1 <= M <= 16; K, lda, ldb multiples of 8.
KSA_API int ksa_gemv_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M >= 1 && M <= 16, "gemv: M=%d out of range (1..16)", M);
  KSA_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemv: K, lda, ldb must be multiples of 8");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // rows per warp: fewer for narrow outputs so that the grid still covers every SM a few times
  const bool narrow = N <= 8192;
  if (M == 1) return narrow ? launch_gemv<1, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<1, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 2) return narrow ? launch_gemv<2, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<2, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 4) return narrow ? launch_gemv<4, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<4, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 8) return narrow ? launch_gemv<8, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<8, 2>(a, b, c, M, N, K, lda, ldb, ldc, st);
  return narrow ? launch_gemv<16, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<16, 2>(a, b, c, M, N, K, lda, ldb, ldc, st);
}
