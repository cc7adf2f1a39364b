// bf16 GEMM on the 5th-generation tensor cores: C[M,N] (+)= A * B with fp32
// accumulation in tensor memory.
//
//   * persistent CTAs (one per SM) walk output tiles of 128 x BN in an
//     L2-friendly grouped order;
//   * warp 0 is the TMA producer (128-byte-swizzled boxes into a 4-stage ring),
//     warp 1 issues tcgen05.mma (one elected thread), warps 2..5 are the epilogue;
//   * the accumulator is double-buffered in TMEM (2 x BN columns), so the
//     epilogue of tile i overlaps the main loop of tile i+1;
//   * either operand may be K-major ("row-major along the reduction") or
//     MN-major, which covers y = x W^T, dx = dy W and dW = dy^T x without any
//     transposed copy.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (muse/models/qwen3_sa/modeling.py:299-314, muse/layers/feed_forward.py:70-83).
#include "common.cuh"
#include "host.h"

namespace ksa {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kGroupM = 16;

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

struct GemmEpilogue {
  void* c;            // output (bf16 or fp32), row-major [M, N]
  long long ldc;      // leading dimension in elements
  int out_fp32;       // 0: bf16, 1: fp32
  int accumulate;     // 1: C += acc (fp32 output only)
  float alpha;        // scale applied to the accumulator
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmEpilogue ep,
                 int M, int N, int K, int* status) {
  using S = GemmSmem<BN>;
  const int cta_first = (int)blockIdx.x;
  const int cta_stride = (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + S::kStages * S::kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + S::kStages;
  uint64_t* acc_full = empty + S::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, status};

  const int tiles_m = (M + kBM - 1) / kBM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int tile, int& mb, int& nb) {
    const int per_group = kGroupM * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int group_rows = min(tiles_m - first_m, kGroupM);
    const int in_group = tile - group * per_group;
    mb = first_m + in_group % group_rows;
    nb = in_group / group_rows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta_first; tile < num_tiles && ok; tile += cta_stride) {
        int mb, nb;
        tile_coords(tile, mb, nb);
        if (!KSA_DEV_CHECK(mb >= 0 && mb < tiles_m && nb >= 0 && nb < tiles_n && stage < S::kStages, status)) break;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, guard, kTimeoutStageEmpty)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_expect_tx(&full[stage], S::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, kb * kBK, mb * kBM, &full[stage]);
          } else {
#pragma unroll
            for (int a = 0; a < kBM / 64; ++a)
              tma_load_2d(sa + a * 8192, &tmA, mb * kBM + a * 64, kb * kBK, &full[stage]);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, kb * kBK, nb * BN, &full[stage]);
          } else {
#pragma unroll
            for (int a = 0; a < BN / 64; ++a)
              tma_load_2d(sb + a * 8192, &tmB, nb * BN + a * 64, kb * kBK, &full[stage]);
          }
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(kBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = cta_first; tile < num_tiles && ok; tile += cta_stride, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, guard, kTimeoutAccEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        if (!KSA_DEV_CHECK((d_tmem & 0xFFFF) + BN <= (tmem_base & 0xFFFF) + 2 * BN, status)) break;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, guard, kTimeoutTmaFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = A_MN ? smem_desc_mnmajor_sw128(sa + k * 2048, 8192) : smem_desc_kmajor_sw128(sa + k * 32);
            const uint64_t db = B_MN ? smem_desc_mnmajor_sw128(sb + k * 2048, 8192) : smem_desc_kmajor_sw128(sb + k * 32);
            umma_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == S::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int local = 0;
    bool ok = true;
    for (int tile = cta_first; tile < num_tiles && ok; tile += cta_stride, ++local) {
      int mb, nb;
      tile_coords(tile, mb, nb);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase, guard, kTimeoutAccFull)) { ok = false; break; }
      tc_fence_after();
      const int row = mb * kBM + quad * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = nb * BN + c * 32;
        if (row < M && col0 < N) {
          if (ep.out_fp32) {
            float* dst = reinterpret_cast<float*>(ep.c) + (long long)row * ep.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < N) {
                float4 v = make_float4(__uint_as_float(r[j]) * ep.alpha, __uint_as_float(r[j + 1]) * ep.alpha,
                                       __uint_as_float(r[j + 2]) * ep.alpha, __uint_as_float(r[j + 3]) * ep.alpha);
                float4* p = reinterpret_cast<float4*>(dst + j);
                if (ep.accumulate) {
                  float4 o = *p;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *p = v;
              }
            }
          } else {
            bf16* dst = reinterpret_cast<bf16*>(ep.c) + (long long)row * ep.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < N) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[j]) * ep.alpha, __uint_as_float(r[j + 1]) * ep.alpha);
                v.y = pack_bf16x2(__uint_as_float(r[j + 2]) * ep.alpha, __uint_as_float(r[j + 3]) * ep.alpha);
                v.z = pack_bf16x2(__uint_as_float(r[j + 4]) * ep.alpha, __uint_as_float(r[j + 5]) * ep.alpha);
                v.w = pack_bf16x2(__uint_as_float(r[j + 6]) * ep.alpha, __uint_as_float(r[j + 7]) * ep.alpha);
                *reinterpret_cast<uint4*>(dst + j) = v;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ----------------------------------------------------------------------------------------------
template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* a, const void* b, const GemmEpilogue& ep, int M, int N, int K, long long lda,
                       long long ldb, int sm_limit, cudaStream_t stream) {
  using S = GemmSmem<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[2] = {2, (uint64_t)lda * 2};
    uint32_t box[2] = {kBK, kBM};
    rc = make_tmap(&tmA, a, 2, 2, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[2] = {2, (uint64_t)lda * 2};
    uint32_t box[2] = {64, kBK};
    rc = make_tmap(&tmA, a, 2, 2, dims, str, box, true);
  }
  if (rc) return rc;
  if (!B_MN) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[2] = {2, (uint64_t)ldb * 2};
    uint32_t box[2] = {kBK, BN};
    rc = make_tmap(&tmB, b, 2, 2, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[2] = {2, (uint64_t)ldb * 2};
    uint32_t box[2] = {64, kBK};
    rc = make_tmap(&tmB, b, 2, 2, dims, str, box, true);
  }
  if (rc) return rc;

  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    KSA_CHECK_CUDA(cudaGetDevice(&dev));
    KSA_CHECK_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    attr_set = true;
  }
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  int ctas = num_sms;
  if (sm_limit > 0 && sm_limit < ctas) ctas = sm_limit;
  if (tiles < ctas) ctas = tiles;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  kern<<<ctas, kGemmThreads, S::kTotal, stream>>>(tmA, tmB, ep, M, N, K, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return kErrNone;
}

}  // namespace ksa

// C[M,N] = alpha * op(A) * op(B) (+ C).  Layouts:
//   a_mn_major = 0: A is [M, K] row-major (lda >= K);  1: A is stored as [K, M] row-major (lda >= M)
//   b_mn_major = 0: B is [N, K] row-major (ldb >= K);  1: B is stored as [K, N] row-major (ldb >= N)
// All leading dimensions are in elements and must be multiples of 8; pointers 16-byte aligned.
// sm_limit > 0 caps the number of CTAs (to leave SMs for a concurrent communication kernel).
KSA_API int ksa_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, float alpha,
                          int sm_limit, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %d x %d x %d", M, N, K);
  KSA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda/ldb must be multiples of 8 elements (got %lld, %lld)", lda, ldb);
  KSA_REQUIRE(N % 8 == 0 && ldc % (out_fp32 ? 4 : 8) == 0, "gemm: N and ldc must keep 16-byte row alignment (N=%d ldc=%lld)", N, ldc);
  KSA_REQUIRE((reinterpret_cast<uintptr_t>(c) & 15) == 0, "gemm: C must be 16-byte aligned");
  KSA_REQUIRE(!(accumulate && !out_fp32), "gemm: accumulate needs an fp32 output");
  GemmEpilogue ep{c, ldc, out_fp32, accumulate, alpha};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool wide = (N >= 256) && (((long long)((M + 127) / 128) * ((N + 255) / 256)) >= 96 || N % 256 == 0);
#define KSA_GEMM_DISPATCH(BN)                                                                        \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BN, false, false>(a, b, ep, M, N, K, lda, ldb, sm_limit, st); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BN, false, true>(a, b, ep, M, N, K, lda, ldb, sm_limit, st);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BN, true, false>(a, b, ep, M, N, K, lda, ldb, sm_limit, st);   \
  return launch_gemm<BN, true, true>(a, b, ep, M, N, K, lda, ldb, sm_limit, st);
  if (wide) {
    KSA_GEMM_DISPATCH(256)
  } else {
    KSA_GEMM_DISPATCH(128)
  }
#undef KSA_GEMM_DISPATCH
}
