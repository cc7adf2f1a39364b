// Skinny GEMM for decoding: C[M, N] = A[M, K] * B[N, K]^T with M <= 16 rows (one token per sequence of the batch).
// The work is a stream of the weight matrix B, so the kernel is laid out for memory bandwidth, not for the tensor
// cores: every CTA owns a slab of output columns small enough that the grid covers all SMs several times (a 128-row
// MMA tile would leave N/256 = 10 CTAs busy for a 2560-wide projection), each warp streams whole weight rows with
// 16-byte loads, the activation rows sit in shared memory, and the dot products are accumulated in fp32.
//
// A decode step is a chain of such kernels, each a few microseconds long, so the engine switches dependent launches
// on (host.h): a CTA may then start while the previous kernel of the stream is still running, asks for its first
// weight bytes (which no earlier kernel writes), and only then waits for the previous kernel (griddepcontrol.wait)
// before it reads the activations.  The gate/up projection can apply SwiGLU itself (kGlu): a
// warp (a CTA in the tensor-core variant) then owns matching gate and up rows and writes silu(gate) * up.
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

// kGlu: B holds N/2 gate rows followed by N/2 up rows; weight row r of a warp is gate row f for even r and up row f
// for odd r (f = first feature + r / 2), and C[m, f] = silu(gate) * up has N/2 columns.
// Optional residual add + RMSNorm in front of the projection (a decode step's `x + delta -> norm -> projection`): the
// activation rows are then A = bf16(rms_norm(bf16(A + delta)) * w), computed by every CTA while it stages them (the
// rows are a few kilobytes), and CTA 0 also writes the new residual stream bf16(A + delta) to `res_out`.
struct GemvNorm {
  const bf16* delta;     // [delta_rows, K] or null
  const bf16* w;         // [K] norm weight; null: no norm, A is used as it is
  bf16* res_out;         // [M, K] or null
  long long ld_delta, ld_res;
  float eps;
  int delta_rows;
};

template <int MT, int R, bool kGlu>
__global__ void __launch_bounds__(kGemvThreads)
gemv_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, int M, int N, int K,
            long long lda, long long ldb, long long ldc, GemvNorm nrm) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  bf16* sA = reinterpret_cast<bf16*>(gemv_smem);           // [MT][kGemvKTile]
  __shared__ float s_rstd[MT];
  __shared__ float s_red[kGemvThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * (kGemvThreads / 32) + warp) * (kGlu ? R / 2 : R);   // first row / first feature
  const int n_out = kGlu ? N / 2 : N;
  long long row_of[R];       // weight row of slot r, or -1 past the end
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int f = kGlu ? n0 + r / 2 : n0 + r;
    row_of[r] = f < n_out ? (long long)(kGlu && (r & 1) ? n_out + f : f) : -1;
  }
  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  // U chunks of every row are requested before any is used, so that enough loads are in flight per SM
  constexpr int U = (R >= 4) ? 2 : (R == 2 ? 4 : 8);
  uint4 w[U][R];
  auto load_w = [&](int k0, int kt, int c0) {
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int c = c0 + u * 256;
        w[u][r] = make_uint4(0, 0, 0, 0);
        if (c < kt && row_of[r] >= 0) w[u][r] = ld_stream_16(B + row_of[r] * ldb + k0 + c);
      }
  };
  // weights are never written by an earlier kernel of the stream: ask for the first chunks, then wait for the
  // kernel that produces the activations
  load_w(0, min(kGemvKTile, K), lane * 8);
  grid_dependency_wait();
  grid_dependency_launch();

  // eight elements of the (residual-added, bf16-rounded) activation row m at column c
  auto load_row8 = [&](int m, int c, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(A + (long long)m * lda + c);
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16x2(uu[q]); v[2 * q] = f.x; v[2 * q + 1] = f.y; }
    if (nrm.delta != nullptr && m < nrm.delta_rows) {
      const uint4 d = *reinterpret_cast<const uint4*>(nrm.delta + (long long)m * nrm.ld_delta + c);
      const uint32_t du[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(du[q]);
        v[2 * q] = __bfloat162float(__float2bfloat16(v[2 * q] + f.x));
        v[2 * q + 1] = __bfloat162float(__float2bfloat16(v[2 * q + 1] + f.y));
      }
    }
  };
  if (nrm.w != nullptr) {
    for (int m = 0; m < MT; ++m) {
      float ss = 0.f;
      if (m < M) {
        for (int c = threadIdx.x * 8; c < K; c += kGemvThreads * 8) {
          float v[8];
          load_row8(m, c, v);
#pragma unroll
          for (int q = 0; q < 8; ++q) ss += v[q] * v[q];
          if (blockIdx.x == 0 && nrm.res_out != nullptr) {
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(nrm.res_out + (long long)m * nrm.ld_res + c) = o;
          }
        }
      }
      ss = warp_sum(ss);
      __syncthreads();
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < kGemvThreads / 32; ++k) t += s_red[k];
        s_rstd[m] = rsqrtf(t / (float)K + nrm.eps);
      }
    }
  }

  for (int k0 = 0; k0 < K; k0 += kGemvKTile) {
    const int kt = min(kGemvKTile, K - k0);          // multiple of 8
    __syncthreads();
    for (int i = threadIdx.x; i < MT * (kGemvKTile / 8); i += kGemvThreads) {
      const int m = i / (kGemvKTile / 8), c = (i % (kGemvKTile / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < M && c < kt) {
        if (nrm.w == nullptr) {
          v = *reinterpret_cast<const uint4*>(A + (long long)m * lda + k0 + c);
        } else {
          float x[8];
          load_row8(m, k0 + c, x);
          const uint4 wv = *reinterpret_cast<const uint4*>(nrm.w + k0 + c);
          const uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
          const float rstd = s_rstd[m];
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = unpack_bf16x2(wu[q]);
            o[q] = pack_bf16x2(x[2 * q] * rstd * f.x, x[2 * q + 1] * rstd * f.y);
          }
          v = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      *reinterpret_cast<uint4*>(sA + m * kGemvKTile + c) = v;
    }
    __syncthreads();
    for (int c0 = lane * 8; c0 < kt; c0 += 256 * U) {
      if (k0 != 0 || c0 != lane * 8) load_w(k0, kt, c0);      // the very first chunks are already on their way
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
    for (int m = 0; m < MT; ++m) acc[r][m] = warp_sum(acc[r][m]);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; r += (kGlu ? 2 : 1)) {
      const int f = kGlu ? n0 + r / 2 : n0 + r;
      if (f >= n_out) break;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= M) break;
        float v = acc[r][m];
        if (kGlu) {
          // gate and up are rounded to bf16 first, as the separate projection + SwiGLU kernels do
          const float g = __bfloat162float(__float2bfloat16(v));
          const float u = __bfloat162float(__float2bfloat16(acc[r + (kGlu ? 1 : 0)][m]));
          v = g / (1.f + __expf(-g)) * u;
        }
        C[(long long)m * ldc + f] = __float2bfloat16(v);
      }
    }
  }
}

template <int MT, int R, bool kGlu>
static int launch_gemv(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, cudaStream_t st, const GemvNorm& nrm = GemvNorm{}) {
  const int per_cta = (kGemvThreads / 32) * (kGlu ? R / 2 : R);      // output columns per CTA
  const int n_out = kGlu ? N / 2 : N;
  const size_t smem = (size_t)MT * kGemvKTile * sizeof(bf16);
  auto kern = gemv_kernel<MT, R, kGlu>;
  static bool attr = false;
  if (!attr && smem > 48 * 1024) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = true;
  }
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), kern, dim3((n_out + per_cta - 1) / per_cta),
                              dim3(kGemvThreads), smem, st, (const bf16*)a, (const bf16*)b, (bf16*)c, M, N, K, lda, ldb,
                              ldc, nrm));
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

// A CTA owns RB blocks of 16 weight rows and stages the activations once for all of them (RB = 2 for wide outputs:
// the activation tile is as large as 16 weight rows, so with one block a CTA would read as many activation bytes
// from L2 as weight bytes from HBM).  kGlu: a block is 8 features, rows 0-7 their gate rows and rows 8-15 their up
// rows.
template <int NB, bool kGlu, int RB>   // NB: batch blocks of 8 rows, 1 (M <= 8) or 2 (M <= 16)
__global__ void __launch_bounds__(kGemvThreads, 2)
gemv_mma_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, bf16* __restrict__ C, int M, int N, int K,
                long long lda, long long ldb, long long ldc) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  bf16* sX = reinterpret_cast<bf16*>(gemv_smem);                       // [NB*8][kMmaRowStride]
  float* sRed = reinterpret_cast<float*>(gemv_smem);                   // reused after the k loop: [8 warps][RB*16][NB*8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_out = kGlu ? N / 2 : N;
  constexpr int kBlockOut = kGlu ? 8 : 16;                              // output columns per row block
  const int n0 = blockIdx.x * kBlockOut * RB;
  int r0[RB], r1[RB];                                                   // clamped: rows past the end are never written
#pragma unroll
  for (int rb = 0; rb < RB; ++rb) {
    r0[rb] = min(n0 + rb * kBlockOut + g, n_out - 1);
    r1[rb] = kGlu ? n_out + r0[rb] : min(n0 + rb * 16 + g + 8, N - 1);
  }
  float acc[RB][NB][4];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rb][b][i] = 0.f;

  // this warp's 32-wide blocks of a tile: warp, warp + 8, warp + 16, warp + 24; all weight loads first
  uint4 w0[RB][4], w1[RB][4];
  auto load_w = [&](int k0, int kt) {
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = (warp + 8 * u) * 32 + t * 8;
        w0[rb][u] = make_uint4(0, 0, 0, 0);
        w1[rb][u] = make_uint4(0, 0, 0, 0);
        if (c < kt) {
          w0[rb][u] = ld_stream_16(B + (long long)r0[rb] * ldb + k0 + c);
          w1[rb][u] = ld_stream_16(B + (long long)r1[rb] * ldb + k0 + c);
        }
      }
  };
  load_w(0, min(kMmaKTile, K));     // weights do not depend on the previous kernel; the activations do
  grid_dependency_wait();
  grid_dependency_launch();

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
    if (k0 != 0) load_w(k0, kt);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = (warp + 8 * u) * 32 + t * 8;
      if (c >= kt) break;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const uint4 x = *reinterpret_cast<const uint4*>(sX + (b * 8 + g) * kMmaRowStride + c);
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          mma_bf16_16x8x16(acc[rb][b], w0[rb][u].x, w1[rb][u].x, w0[rb][u].y, w1[rb][u].y, x.x, x.y);
          mma_bf16_16x8x16(acc[rb][b], w0[rb][u].z, w1[rb][u].z, w0[rb][u].w, w1[rb][u].w, x.z, x.w);
        }
      }
    }
  }
  // acc[rb][b] = {C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1]}: rows = weight rows of block rb, columns = batch
  __syncthreads();
  constexpr int NBATCH = NB * 8;
  constexpr int kRows = RB * 16;
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float* dst = sRed + (warp * kRows + rb * 16) * NBATCH;
      dst[g * NBATCH + b * 8 + 2 * t] = acc[rb][b][0];
      dst[g * NBATCH + b * 8 + 2 * t + 1] = acc[rb][b][1];
      dst[(g + 8) * NBATCH + b * 8 + 2 * t] = acc[rb][b][2];
      dst[(g + 8) * NBATCH + b * 8 + 2 * t + 1] = acc[rb][b][3];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < RB * kBlockOut * NBATCH; i += kGemvThreads) {
    const int col = i % (RB * kBlockOut), m = i / (RB * kBlockOut);   // consecutive threads -> consecutive outputs
    const int rb = col / kBlockOut, row = rb * 16 + col % kBlockOut;    // row inside the CTA's RB * 16 weight rows
    float v = 0.f, u = 0.f;
#pragma unroll
    for (int w = 0; w < kGemvThreads / 32; ++w) {
      v += sRed[(w * kRows + row) * NBATCH + m];
      if (kGlu) u += sRed[(w * kRows + row + 8) * NBATCH + m];
    }
    if (kGlu) {
      const float gt = __bfloat162float(__float2bfloat16(v)), up = __bfloat162float(__float2bfloat16(u));
      v = gt / (1.f + __expf(-gt)) * up;
    }
    if (m < M && n0 + col < n_out) C[(long long)m * ldc + n0 + col] = __float2bfloat16(v);
  }
}

template <int NB, bool kGlu, int RB>
static int launch_gemv_mma(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, cudaStream_t st) {
  // the activation tile, reused for the final reduction [8 warps][RB * 16][NB * 8] floats
  const size_t x_bytes = (size_t)NB * 8 * kMmaRowStride * sizeof(bf16), red_bytes = (size_t)8 * RB * 16 * NB * 8 * 4;
  const size_t smem = x_bytes > red_bytes ? x_bytes : red_bytes;
  const int per_cta = (kGlu ? 8 : 16) * RB, n_out = kGlu ? N / 2 : N;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), gemv_mma_kernel<NB, kGlu, RB>,
                              dim3((n_out + per_cta - 1) / per_cta), dim3(kGemvThreads), smem, st, (const bf16*)a,
                              (const bf16*)b, (bf16*)c, M, N, K, lda, ldb, ldc));
  return 0;
}

}  // namespace ksa

namespace ksa {
template <bool kGlu>
static int gemv_dispatch(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, cudaStream_t st, const GemvNorm& nrm = GemvNorm{}) {
  if (M > 4 && K % 32 == 0 && nrm.w == nullptr) {
    if (N >= 16384)   // wide outputs: 32 weight rows per CTA still give every SM several CTAs
      return M <= 8 ? launch_gemv_mma<1, kGlu, 2>(a, b, c, M, N, K, lda, ldb, ldc, st)
                    : launch_gemv_mma<2, kGlu, 2>(a, b, c, M, N, K, lda, ldb, ldc, st);
    return M <= 8 ? launch_gemv_mma<1, kGlu, 1>(a, b, c, M, N, K, lda, ldb, ldc, st)
                  : launch_gemv_mma<2, kGlu, 1>(a, b, c, M, N, K, lda, ldb, ldc, st);
  }
  // rows per warp: fewer for narrow outputs so that the grid still covers every SM a few times (with SwiGLU a warp
  // needs at least one gate row and one up row)
  const bool narrow = N <= 8192;
  constexpr int R1 = kGlu ? 2 : 1;
  if (M == 1) return narrow ? launch_gemv<1, R1, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm) : launch_gemv<1, 4, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm);
  if (M <= 2) return narrow ? launch_gemv<2, R1, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm) : launch_gemv<2, 4, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm);
  if (M <= 4) return narrow ? launch_gemv<4, R1, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm) : launch_gemv<4, 4, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st, nrm);
  if (M <= 8) return narrow ? launch_gemv<8, R1, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<8, 2, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st);
  return narrow ? launch_gemv<16, R1, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st) : launch_gemv<16, 2, kGlu>(a, b, c, M, N, K, lda, ldb, ldc, st);
}
}  // namespace ksa

// C[M, N] (bf16, ldc) = A[M, K] (bf16, lda) * B[N, K]^T (bf16, ldb) for 1 <= M <= 16; K, lda, ldb multiples of 8.
KSA_API int ksa_gemv_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M >= 1 && M <= 16, "gemv: M=%d out of range (1..16)", M);
  KSA_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemv: K, lda, ldb must be multiples of 8");
  return gemv_dispatch<false>(a, b, c, M, N, K, lda, ldb, ldc, reinterpret_cast<cudaStream_t>(stream));
}

// The gate/up projection of a SwiGLU feed-forward block with its activation: B holds N/2 gate rows followed by N/2
// up rows, C[M, N/2] = silu(A * gate^T) * (A * up^T), gate and up rounded to bf16 before the activation.
KSA_API int ksa_gemv_swiglu_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M >= 1 && M <= 16, "gemv_swiglu: M=%d out of range (1..16)", M);
  KSA_REQUIRE(N > 0 && N % 2 == 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0,
              "gemv_swiglu: N must be even and K, lda, ldb multiples of 8");
  return gemv_dispatch<true>(a, b, c, M, N, K, lda, ldb, ldc, reinterpret_cast<cudaStream_t>(stream));
}

// A decode step's `residual add -> RMSNorm -> projection` in one launch, for at most 4 rows:
//   res = bf16(x + delta)  (delta may be null or have fewer rows; written to res_out by one CTA when res_out is given)
//   C   = rms_norm(res, norm_w, eps) * B^T          (glu = 0; C is [M, N])
//   C   = silu(. * gate^T) * (. * up^T)             (glu = 1; B = gate rows then up rows, C is [M, N/2])
KSA_API int ksa_gemv_norm_bf16(const void* x, const void* delta, const void* norm_w, void* res_out, const void* b, void* c,
                               int M, int N, int K, long long ldx, long long ld_delta, long long ld_res, long long ldb,
                               long long ldc, float eps, int delta_rows, int glu, void* stream) {
  KSA_ENTER(x);
  using namespace ksa;
  KSA_REQUIRE(M >= 1 && M <= 4, "gemv_norm: M=%d out of range (1..4)", M);
  KSA_REQUIRE(norm_w != nullptr, "gemv_norm: the norm weight is required");
  KSA_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && ldb % 8 == 0 && ld_delta % 8 == 0 && ld_res % 8 == 0,
              "gemv_norm: K and the leading dimensions must be multiples of 8");
  KSA_REQUIRE(!glu || N % 2 == 0, "gemv_norm: N must be even with glu");
  GemvNorm nrm{(const bf16*)delta, (const bf16*)norm_w, (bf16*)res_out, ld_delta, ld_res, eps, delta ? delta_rows : 0};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return glu ? gemv_dispatch<true>(x, b, c, M, N, K, ldx, ldb, ldc, st, nrm)
             : gemv_dispatch<false>(x, b, c, M, N, K, ldx, ldb, ldc, st, nrm);
}
