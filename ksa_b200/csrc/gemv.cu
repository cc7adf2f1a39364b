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

// ------------------------------------------------------------------------------------------ tensor-core variant
// For 5..16 activation rows the SIMT kernel above is bound by its FMA issue rate, so the dot products go to the tensor
// cores with warp-level mma.sync m16n8k16 (the 128-row tcgen05 tile has no use for 16 rows): a CTA owns 16 weight
// rows, its 8 warps take the 32-wide k blocks round-robin, and the partial sums meet in shared memory.  Both operands
// are read as 16 contiguous bytes per lane along k; a lane's 8 elements are given to the instruction as its k slots
// {2t, 2t+1, 2t+8, 2t+9} of two MMAs.  That permutes k inside a 32-block, identically for weights and activations,
// which a dot product does not see.
constexpr int kMmaKTile = 1024;               // activation columns staged per pass (32 blocks of 32)
constexpr int kMmaRowStride = kMmaKTile + 32;  // +64 bytes: the two row groups of a quarter warp hit different banks

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NB>   // batch blocks of 8 rows: 1 (M <= 8) or 2 (M <= 16)
__global__ void __launch_bounds__(kGemvThreads)
gemv_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, int M, int N, int K,
                long long lda, long long ldb, long long ldc) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  bf16* sX = reinterpret_cast<bf16*>(gemv_smem);                       // [NB*8][kMmaRowStride]
  float* sRed = reinterpret_cast<float*>(gemv_smem);                   // reused after the k loop: [8 warps][16][NB*8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);       // clamped: rows past N are never written
  float acc[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[b][i] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kMmaKTile) {
    const int kt = min(kMmaKTile, K - k0);   // multiple of 32
    __syncthreads();
    for (int i = threadIdx.x; i < NB * 8 * (kMmaKTile / 8); i += kGemvThreads) {
      const int m = i / (kMmaKTile / 8), c = (i % (kMmaKTile / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < M && c < kt) v = *reinterpret_cast<const uint4*>(A + (long long)m * lda + k0 + c);
      *reinterpret_cast<uint4*>(sX + m * kMmaRowStride + c) = v;
    }
    __syncthreads();
    // this warp's 32-wide blocks of the tile: warp, warp + 8, warp + 16, warp + 24; all weight loads first
    uint4 w0[4], w1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = (warp + 8 * u) * 32 + t * 8;
      w0[u] = make_uint4(0, 0, 0, 0);
      w1[u] = make_uint4(0, 0, 0, 0);
      if (c < kt) {
        w0[u] = ld_stream_16(B + (long long)r0 * ldb + k0 + c);
        w1[u] = ld_stream_16(B + (long long)r1 * ldb + k0 + c);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = (warp + 8 * u) * 32 + t * 8;
      if (c >= kt) break;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const uint4 x = *reinterpret_cast<const uint4*>(sX + (b * 8 + g) * kMmaRowStride + c);
        mma_bf16_16x8x16(acc[b], w0[u].x, w1[u].x, w0[u].y, w1[u].y, x.x, x.y);
        mma_bf16_16x8x16(acc[b], w0[u].z, w1[u].z, w0[u].w, w1[u].w, x.z, x.w);
      }
    }
  }
  // acc[b] = {C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1]} with rows = weight rows, columns = batch b*8 + ...
  __syncthreads();
  constexpr int NBATCH = NB * 8;
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    float* dst = sRed + warp * 16 * NBATCH;
    dst[g * NBATCH + b * 8 + 2 * t] = acc[b][0];
    dst[g * NBATCH + b * 8 + 2 * t + 1] = acc[b][1];
    dst[(g + 8) * NBATCH + b * 8 + 2 * t] = acc[b][2];
    dst[(g + 8) * NBATCH + b * 8 + 2 * t + 1] = acc[b][3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * NBATCH; i += kGemvThreads) {
    const int row = i % 16, m = i / 16;          // consecutive threads -> consecutive output columns
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kGemvThreads / 32; ++w) v += sRed[w * 16 * NBATCH + row * NBATCH + m];
    if (m < M && n0 + row < N) C[(long long)m * ldc + n0 + row] = __float2bfloat16(v);
  }
}

template <int NB>
static int launch_gemv_mma(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, cudaStream_t st) {
  const size_t smem = (size_t)NB * 8 * kMmaRowStride * sizeof(bf16);    // >= the 8 KB / 16 KB of the final reduction
  gemv_mma_kernel<NB><<<(N + 15) / 16, kGemvThreads, smem, st>>>((const bf16*)a, (const bf16*)b, (bf16*)c, M, N, K, lda,
                                                                 ldb, ldc);
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
  if (M > 4 && K % 32 == 0) {
    return M <= 8 ? launch_gemv_mma<1>(a, b, c, M, N, K, lda, ldb, ldc, st)
                  : launch_gemv_mma<2>(a, b, c, M, N, K, lda, ldb, ldc, st);
  }
  // rows per warp: fewer for narrow outputs so that the grid still covers every SM a few times
  const bool narrow = N <= 8192;
  if (M == 1) return narrow ? launch_gemv<1, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<1, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 2) return narrow ? launch_gemv<2, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<2, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 4) return narrow ? launch_gemv<4, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<4, 4>(a, b, c, M, N, K, lda, ldb, ldc, st);
  if (M <= 8) return narrow ? launch_gemv<8, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<8, 2>(a, b, c, M, N, K, lda, ldb, ldc, st);
  return narrow ? launch_gemv<16, 1>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<16, 2>(a, b, c, M, N, K, lda, ldb, ldc, st);
}
