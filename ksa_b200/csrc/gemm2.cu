// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster, on the two SMs of one TPC, share a
// 256 x 256 output tile.  Each CTA stages its own 128 rows of A and its own 128 of the 256 rows of B, the leader CTA
// issues one MMA for the pair, and each CTA's tensor memory receives its 128 x 256 half of the accumulator.  Per SM and
// k-step that is 8 KB of shared-memory operands for a 128 x 256 x 16 product instead of 12 KB with single-CTA MMAs,
// which is what keeps the tensor pipe fed (a 128 x 256 single-CTA MMA needs more operand bytes per clock than shared
// memory delivers).
//
// Roles per CTA (224 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only), warps 2..5 epilogue,
// warp 6 communication (idle in a plain GEMM).
// Barriers: `full` lives in the leader and collects the bytes of both CTAs' loads (the peer's TMA loads name the
// leader's barrier); `empty` and `acc_full` exist in both CTAs and are signalled for both by one multicast
// tcgen05.commit; `acc_empty` lives in the leader and collects one arrival per epilogue warp of both CTAs.
// No TMA load here uses cluster multicast.  Every wait is bounded.
//
// All-gather -> GEMM in one launch (ksa_gemm2_gather_bf16): warp 6 of every CTA is a communication warp.  One of
// its threads pulls this CTA's share of the other ranks' shards of an operand out of the peers' memory with bulk
// copies through a small shared-memory ring (run_gather_job_bulk) and counts the landed chunks of every shard in
// `done[r]`; the TMA producers wait (bounded) for the shards that hold the rows of their next tile, and the tile order
// starts at this rank's own rows and follows the order in which the shards arrive.  The NVLink transfer of shard r+1
// therefore runs under the tensor-core tiles of shard r, and no SM is taken away from the math: one SM copies only
// about 40 GB/s, so the transfer is spread over all 148.
#include "comm.cuh"
#include "host.h"

#include <stdlib.h>

namespace ksa {

constexpr int k2BM = 128;          // rows of A (and of the accumulator) per CTA
constexpr int k2BN = 256;          // accumulator columns per pair
constexpr int k2BNh = 128;         // rows of B staged per CTA
constexpr int k2BK = 64;
constexpr int k2Threads = 224;      // warps 0..5 as described above, warp 6 for communication
constexpr int k2Stages = 6;
constexpr int k2GroupM = 8;        // pair-tile rows per scheduling group
constexpr int k2ABytes = k2BM * k2BK * 2;
constexpr int k2BBytes = k2BNh * k2BK * 2;
constexpr int k2StageBytes = k2ABytes + k2BBytes;
constexpr int k2BarrierBytes = 256;
constexpr int k2SmemTotal = k2Stages * k2StageBytes + k2BarrierBytes + kBulkRingBytes + 1024;
static_assert(kMaxPeers * kBulkSegs <= 32, "one bit per segment in the producers' bookkeeping");
static_assert(k2SmemTotal <= 232448, "the operand ring, the barriers and the copy ring must fit 227 KB");

struct Gemm2Epilogue {
  void* c;
  long long ldc;
  int out_fp32, accumulate;
  float alpha;
  // GEMM -> reduce-scatter (bf16 output only): output row `row` belongs to rank row / c_shard_rows and is stored, from
  // the epilogue, straight into that rank's memory at c_peer[owner] + (row - owner * c_shard_rows) * ldc.
  int c_shard_rows;          // 0: every row goes to `c`
  int c_world;
  int c_tma;                 // 1: 32-row blocks that lie in one owner's rows leave through TMA stores (c_map)
  void* c_peer[kMaxPeers];
};

// Tensor maps over the owners' output buffers ([rows of that owner, N] bf16, box 64 columns x 32 rows, 128-byte
// swizzle) for the scattering epilogue.
struct ScatterMaps {
  CUtensorMap m[kMaxPeers];
};

// Communication work riding in a pair-GEMM launch, and what the math waits for.
struct Comm2Work {
  int active;                // 1: warp 6 of every CTA gathers
  GatherJob gather;          // gather.done is required when dep_operand != 0
  int dep_operand;           // 0: the math does not read the gathered buffer; 1: A rows live in it; 2: B rows
  long long dep_offset;      // byte offset of the operand's row 0 inside the gathered buffer
  long long dep_row_bytes;   // bytes from one operand row to the next
  int m_rotate;              // pair-tile row that is worked on first
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_smem_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA tile load whose completion bytes are counted by a barrier that may sit in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void umma2_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once all MMAs issued so far are done.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(k2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ Gemm2Epilogue ep,
                  int M, int N, int K, int* status, const __grid_constant__ Comm2Work comm,
                  const __grid_constant__ ScatterMaps smaps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem + k2Stages * k2StageBytes;      // copy ring of the communication warp, or the epilogue's
                                                       // staging for TMA stores (1024-byte aligned)
  uint8_t* bar_base = ring + kBulkRingBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);   // used in the leader
  uint64_t* empty = full + k2Stages;                         // both CTAs
  uint64_t* acc_full = empty + k2Stages;                     // both CTAs, 2 buffers
  uint64_t* acc_empty = acc_full + 2;                        // used in the leader, 2 buffers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();     // 0 = leader
  const WaitGuard guard{abort_flag, status};
  const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
  const int tiles_m = (M + 2 * k2BM - 1) / (2 * k2BM);
  const int tiles_n = (N + k2BN - 1) / k2BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + k2BK - 1) / k2BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < k2Stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 2) { tmem_alloc2(tmem_slot, 512); tmem_relinquish2(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before any remote arrival
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int tile, int& mb, int& nb) {
    const int per_group = k2GroupM * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * k2GroupM;
    const int group_rows = min(tiles_m - first_m, k2GroupM);
    const int in_group = tile - group * per_group;
    mb = first_m + in_group % group_rows + comm.m_rotate;
    if (mb >= tiles_m) mb -= tiles_m;
    nb = in_group / group_rows;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t segs_seen = 0;       // kMaxPeers x kBulkSegs = 32 segments
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int mb, nb;
        tile_coords(tile, mb, nb);
        if (!KSA_DEV_CHECK(mb >= 0 && mb < tiles_m && nb >= 0 && nb < tiles_n && rank < 2 && stage < k2Stages, status)) break;
        const int row0 = mb * 2 * k2BM + (int)rank * k2BM;      // this CTA's rows of A
        const int col0 = nb * k2BN + (int)rank * k2BNh;         // this CTA's rows of B
        if (comm.dep_operand != 0) {
          // the rows of this tile that live in the gathered buffer: wait for the segments of the shards that hold them
          const long long r_lo = comm.dep_operand == 1 ? row0 : col0;
          const long long r_end = comm.dep_operand == 1 ? min(row0 + k2BM, M) : min(col0 + k2BNh, N);
          if (r_lo < r_end) {
            const long long sb = comm.gather.shard_bytes;
            const long long n_chunks = bulk_chunks(sb);
            const int segs = bulk_segs(n_chunks, (int)gridDim.x, comm.gather.max_segs);
            const long long b_lo = comm.dep_offset + r_lo * comm.dep_row_bytes;
            const long long b_hi = comm.dep_offset + r_end * comm.dep_row_bytes - 1;          // last byte read
            const int s_lo = max((int)(b_lo / sb), 0), s_hi = min((int)(b_hi / sb), comm.gather.world - 1);
            bool waited = false;
            for (int s = s_lo; s <= s_hi && ok; ++s) {
              if (s == comm.gather.rank) continue;
              const long long in_lo = max(b_lo - s * sb, 0LL), in_hi = min(b_hi - s * sb, sb - 1);
              const int g_lo = bulk_seg_of(n_chunks, segs, in_lo / kBulkChunk);
              const int g_hi = bulk_seg_of(n_chunks, segs, in_hi / kBulkChunk);
              for (int g = g_lo; g <= g_hi && ok; ++g) {
                const int idx = s * kBulkSegs + g;
                if ((segs_seen >> idx) & 1u) continue;
                const uint32_t need = (uint32_t)(bulk_seg_begin(n_chunks, segs, g + 1) - bulk_seg_begin(n_chunks, segs, g));
                if (!flag_wait_ge(comm.gather.done + idx, need, status, kTimeoutPeerFlag, true)) {
                  *abort_flag = 1;
                  ok = false;
                }
                segs_seen |= 1u << idx;
                waited = true;
              }
            }
            if (!ok) break;
            if (waited) fence_proxy_async_all();     // written by other CTAs' bulk stores; TMA reads it next
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, guard, kTimeoutStageEmpty)) { ok = false; break; }
          uint8_t* sa = smem + stage * k2StageBytes;
          uint8_t* sb = sa + k2ABytes;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * k2StageBytes);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, kb * k2BK, row0, bar);
          } else {
#pragma unroll
            for (int a = 0; a < k2BM / 64; ++a) tma_load_2d_pair(sa + a * 8192, &tmA, row0 + a * 64, kb * k2BK, bar);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmB, kb * k2BK, col0, bar);
          } else {
#pragma unroll
            for (int a = 0; a < k2BNh / 64; ++a) tma_load_2d_pair(sb + a * 8192, &tmB, col0 + a * 64, kb * k2BK, bar);
          }
          if (++stage == k2Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * k2BM, k2BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, guard, kTimeoutAccEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * k2BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, guard, kTimeoutTmaFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * k2StageBytes);
          const uint32_t sb = sa + k2ABytes;
#pragma unroll
          for (int k = 0; k < k2BK / 16; ++k) {
            const uint64_t da = A_MN ? smem_desc_mnmajor_sw128(sa + k * 2048, 8192) : smem_desc_kmajor_sw128(sa + k * 32);
            const uint64_t db = B_MN ? smem_desc_mnmajor_sw128(sb + k * 2048, 8192) : smem_desc_kmajor_sw128(sb + k * 32);
            umma2_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma2_commit_both(&empty[stage]);
          if (++stage == k2Stages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma2_commit_both(&acc_full[buf]);
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ communication warp (both CTAs, one thread)
    if (lane == 0 && comm.active)
      run_gather_job_bulk(comm.gather, (int)blockIdx.x, (int)gridDim.x, ring, status);
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
      int mb, nb;
      tile_coords(tile, mb, nb);
      const int buf = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], acc_phase, guard, kTimeoutAccFull)) { ok = false; break; }
      tc_fence_after();
      const int row_w = mb * 2 * k2BM + (int)rank * k2BM + quad * 32;   // first of this warp's 32 rows
      const int row = row_w + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * k2BN;
      // scattering epilogue: a 32-row block that lies in ONE owner's rows leaves through shared memory and TMA
      // stores of 64 columns x 32 rows (128-byte rows on the wire); a block that straddles two owners' rows
      // falls back to the per-row stores below
      int owner_w = 0;
      bool tma_block = false;
      if (ep.c_tma && row_w < M) {
        owner_w = min(row_w / ep.c_shard_rows, ep.c_world - 1);
        tma_block = min(min(row_w + 31, M - 1) / ep.c_shard_rows, ep.c_world - 1) == owner_w;
      }
#pragma unroll 1
      for (int c = 0; c < k2BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = nb * k2BN + c * 32;
        if (tma_block) {
          const int piece = c >> 1, half = c & 1;                   // 64-column piece, 32-column half of it
          uint8_t* stage = ring + ((warp - 2) * 2 + (piece & 1)) * 4096;
          const bool live = nb * k2BN + piece * 64 < N;             // N is a multiple of 64 on this path
          if (half == 0) {
            // this buffer was read by the store issued two pieces ago; at most the newest store may be pending
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
          }
          if (live) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * j]) * ep.alpha, __uint_as_float(r[8 * j + 1]) * ep.alpha);
              v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * ep.alpha, __uint_as_float(r[8 * j + 3]) * ep.alpha);
              v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * ep.alpha, __uint_as_float(r[8 * j + 5]) * ep.alpha);
              v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * ep.alpha, __uint_as_float(r[8 * j + 7]) * ep.alpha);
              const int chunk = (half * 4 + j) ^ (lane & 7);        // 128-byte swizzle: 16-byte chunk ^ (row mod 8)
              *reinterpret_cast<uint4*>(stage + lane * 128 + chunk * 16) = v;
            }
          }
          if (half == 1) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && live) {
              tma_store_2d(&smaps.m[owner_w], stage, nb * k2BN + piece * 64, row_w - owner_w * ep.c_shard_rows);
              tma_store_commit();
            }
          }
          continue;
        }
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
                  const float4 o = *p;
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *p = v;
              }
            }
          } else {
            bf16* dst;
            if (ep.c_shard_rows > 0) {
              const int owner = min(row / ep.c_shard_rows, ep.c_world - 1);
              dst = reinterpret_cast<bf16*>(ep.c_peer[owner]) + (long long)(row - owner * ep.c_shard_rows) * ep.ldc + col0;
            } else {
              dst = reinterpret_cast<bf16*>(ep.c) + (long long)row * ep.ldc + col0;
            }
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
      // one arrival per epilogue warp of either CTA on the leader's barrier: this accumulator buffer may be rewritten
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
    }
  }

  // TMA stores of the scattering epilogue have written their destination before the kernel ends
  if (ep.c_tma && warp >= 2 && warp < 6 && lane == 0) tma_store_wait0();
  // The peer's tensor memory and barriers are written by the leader's MMAs and commits: nobody leaves, and nothing
  // is deallocated, before both CTAs are done.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

static const ScatterMaps kNoScatterMaps{};

template <bool A_MN, bool B_MN>
static int launch_gemm2(const void* a, const void* b, const Gemm2Epilogue& ep, int M, int N, int K, long long lda,
                        long long ldb, cudaStream_t stream, const Comm2Work& comm,
                        const ScatterMaps& smaps = kNoScatterMaps) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[2] = {2, (uint64_t)lda * 2};
    uint32_t box[2] = {k2BK, k2BM};
    rc = make_tmap(&tmA, a, 2, 2, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[2] = {2, (uint64_t)lda * 2};
    uint32_t box[2] = {64, k2BK};
    rc = make_tmap(&tmA, a, 2, 2, dims, str, box, true);
  }
  if (rc) return rc;
  if (!B_MN) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[2] = {2, (uint64_t)ldb * 2};
    uint32_t box[2] = {k2BK, k2BNh};
    rc = make_tmap(&tmB, b, 2, 2, dims, str, box, true);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[2] = {2, (uint64_t)ldb * 2};
    uint32_t box[2] = {64, k2BK};
    rc = make_tmap(&tmB, b, 2, 2, dims, str, box, true);
  }
  if (rc) return rc;
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    KSA_CHECK_CUDA(cudaGetDevice(&dev));
    KSA_CHECK_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  auto kern = gemm2_bf16_kernel<A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k2SmemTotal));
    attr_set = true;
  }
  const int tiles = ((M + 2 * k2BM - 1) / (2 * k2BM)) * ((N + k2BN - 1) / k2BN);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  kern<<<2 * pairs, k2Threads, k2SmemTotal, stream>>>(tmA, tmB, ep, M, N, K, status, comm, smaps);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace ksa

// Same contract as ksa_gemm_bf16 (without sm_limit and without attached communication work), on CTA pairs.
KSA_API int ksa_gemm2_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, float alpha,
                           void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm2: empty problem %d x %d x %d", M, N, K);
  KSA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm2: lda/ldb must be multiples of 8 elements (got %lld, %lld)", lda, ldb);
  KSA_REQUIRE(N % 8 == 0 && ldc % (out_fp32 ? 4 : 8) == 0, "gemm2: N and ldc must keep 16-byte row alignment");
  KSA_REQUIRE((reinterpret_cast<uintptr_t>(c) & 15) == 0, "gemm2: C must be 16-byte aligned");
  KSA_REQUIRE(!(accumulate && !out_fp32), "gemm2: accumulate needs an fp32 output");
  Gemm2Epilogue ep{};
  ep.c = c; ep.ldc = ldc; ep.out_fp32 = out_fp32; ep.accumulate = accumulate; ep.alpha = alpha;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const Comm2Work none{};
  if (!a_mn_major && !b_mn_major) return launch_gemm2<false, false>(a, b, ep, M, N, K, lda, ldb, st, none);
  if (!a_mn_major && b_mn_major) return launch_gemm2<false, true>(a, b, ep, M, N, K, lda, ldb, st, none);
  if (a_mn_major && !b_mn_major) return launch_gemm2<true, false>(a, b, ep, M, N, K, lda, ldb, st, none);
  return launch_gemm2<true, true>(a, b, ep, M, N, K, lda, ldb, st, none);
}

// All-gather -> GEMM in one launch.  The GEMM arguments are those of ksa_gemm2_bf16; both operands K-major.
//   peers/world/rank/shard_bytes/ready_flags/epoch_ptr/epoch_add: the gather, as in ksa_peer_gather (shard r of every
//     rank's buffer is bytes [r*shard_bytes, (r+1)*shard_bytes); shards r != rank are pulled into peers[rank]).
//   done: 32 uint32 counters in own memory, used by this launch only (the call zeroes them on the stream first):
//     landed chunks per (shard, segment).  Required when dep_operand != 0.
//   dep_operand: 1 if A (the [M, K] operand) lies inside the gathered buffer, 2 if B does, 0 if neither (the
//     gather then only shares the launch); dep_offset: byte offset of that operand's first row in the buffer; the
//     row pitch is lda (ldb) elements.
KSA_API int ksa_gemm2_gather_bf16(const void* a, const void* b, void* c, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, int out_fp32, int accumulate, float alpha,
                                  const void* const* peers, int world, int rank, long long shard_bytes,
                                  const void* ready_flags, const void* epoch_ptr, unsigned epoch_add, void* done,
                                  int dep_operand, long long dep_offset, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm2_gather: empty problem %d x %d x %d", M, N, K);
  KSA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm2_gather: lda/ldb must be multiples of 8 elements (got %lld, %lld)", lda, ldb);
  KSA_REQUIRE(N % 8 == 0 && ldc % (out_fp32 ? 4 : 8) == 0, "gemm2_gather: N and ldc must keep 16-byte row alignment");
  KSA_REQUIRE((reinterpret_cast<uintptr_t>(c) & 15) == 0, "gemm2_gather: C must be 16-byte aligned");
  KSA_REQUIRE(!(accumulate && !out_fp32), "gemm2_gather: accumulate needs an fp32 output");
  KSA_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "gemm2_gather: rank %d of %d out of range", rank, world);
  KSA_REQUIRE(shard_bytes > 0 && shard_bytes % 16 == 0, "gemm2_gather: shard bytes must be a positive multiple of 16");
  KSA_REQUIRE(dep_operand >= 0 && dep_operand <= 2 && dep_offset >= 0, "gemm2_gather: bad dependency description");
  KSA_REQUIRE(dep_operand == 0 || done != nullptr, "gemm2_gather: a dependency needs the done counters");
  Gemm2Epilogue ep{};
  ep.c = c; ep.ldc = ldc; ep.out_fp32 = out_fp32; ep.accumulate = accumulate; ep.alpha = alpha;
  Comm2Work comm{};
  if (world > 1) {
    comm.active = 1;
    for (int r = 0; r < world; ++r) {
      KSA_REQUIRE(peers[r] != nullptr && (reinterpret_cast<uintptr_t>(peers[r]) & 15) == 0, "gemm2_gather: peer %d buffer missing or misaligned", r);
      comm.gather.peers[r] = static_cast<const uint8_t*>(peers[r]);
    }
    comm.gather.world = world; comm.gather.rank = rank; comm.gather.shard_bytes = shard_bytes;
    comm.gather.ready_flags = static_cast<const uint32_t*>(ready_flags);
    comm.gather.epoch_ptr = static_cast<const uint32_t*>(epoch_ptr); comm.gather.epoch_add = epoch_add;
    comm.gather.done = static_cast<uint32_t*>(done);
    static int max_segs = 0;               // KSA_BULK_SEGS=1..4 caps the segments per shard (for A/B runs)
    if (max_segs == 0) {
      const char* e = getenv("KSA_BULK_SEGS");
      max_segs = e ? atoi(e) : kBulkSegs;
      if (max_segs < 1 || max_segs > kBulkSegs) max_segs = kBulkSegs;
    }
    comm.gather.max_segs = max_segs;
    comm.dep_operand = dep_operand;
    comm.dep_offset = dep_offset;
    comm.dep_row_bytes = (dep_operand == 2 ? ldb : lda) * 2;
    if (done != nullptr)
      KSA_CHECK_CUDA(cudaMemsetAsync(done, 0, sizeof(uint32_t) * kMaxPeers * kBulkSegs, reinterpret_cast<cudaStream_t>(stream)));
    if (dep_operand == 1) {
      // start with the first tile row that lies entirely in this rank's own rows; a tile row that straddles the
      // boundary to the previous rank's shard (the last one to arrive) then comes last
      const long long first_row = ((long long)rank * shard_bytes - dep_offset + comm.dep_row_bytes - 1) / comm.dep_row_bytes;
      const int tiles_m = (M + 2 * k2BM - 1) / (2 * k2BM);
      if (first_row > 0 && first_row < M) comm.m_rotate = (int)((first_row + 2 * k2BM - 1) / (2 * k2BM)) % tiles_m;
    }
  }
  return launch_gemm2<false, false>(a, b, ep, M, N, K, lda, ldb, reinterpret_cast<cudaStream_t>(stream), comm);
}

// GEMM -> reduce-scatter, producer side: C = A B^T (both K-major, bf16 output) whose row block r (rows
// [r*shard_rows, (r+1)*shard_rows), the last block takes the remainder) is written by the epilogue directly into
// rank r's memory at c_peers[r] (row pitch ldc elements) with P2P stores, so the transfer runs under the remaining
// tiles and the reduction that follows reads only local memory.  c_peers[r] must be 16-byte aligned.  With N a
// multiple of 64, every 32-row block that lies within one rank's rows goes through shared memory and TMA stores
// (128-byte rows over NVLink instead of 16-byte register stores).
KSA_API int ksa_gemm2_scatter_bf16(const void* a, const void* b, int M, int N, int K, long long lda, long long ldb,
                                   long long ldc, const void* const* c_peers, int world, int shard_rows, void* stream) {
  KSA_ENTER(a);
  using namespace ksa;
  KSA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm2_scatter: empty problem %d x %d x %d", M, N, K);
  KSA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0 && N % 8 == 0, "gemm2_scatter: leading dimensions and N must be multiples of 8");
  KSA_REQUIRE(world >= 1 && world <= kMaxPeers && shard_rows > 0, "gemm2_scatter: world %d / shard rows %d out of range", world, shard_rows);
  KSA_REQUIRE((long long)shard_rows * world >= M, "gemm2_scatter: %d shards of %d rows do not cover %d rows", world, shard_rows, M);
  KSA_REQUIRE(ldc >= N, "gemm2_scatter: row pitch %lld of the owners' buffers is smaller than N = %d", ldc, N);
  Gemm2Epilogue ep{};
  ep.ldc = ldc; ep.alpha = 1.f; ep.c_shard_rows = shard_rows; ep.c_world = world;
  for (int r = 0; r < world; ++r) {
    KSA_REQUIRE(c_peers[r] != nullptr && (reinterpret_cast<uintptr_t>(c_peers[r]) & 15) == 0, "gemm2_scatter: output of rank %d missing or misaligned", r);
    ep.c_peer[r] = const_cast<void*>(c_peers[r]);
  }
  ep.c = ep.c_peer[0];
  ScatterMaps smaps{};
  if (N % 64 == 0) {
    // one tensor map per owner over the rows it really gets: rows past the end of the product are clipped by the map
    ep.c_tma = 1;
    for (int r = 0; r < world; ++r) {
      const long long rows_r = (long long)M - (long long)r * shard_rows;
      if (rows_r <= 0) break;
      uint64_t dims[2] = {(uint64_t)N, (uint64_t)(rows_r < shard_rows ? rows_r : shard_rows)};
      uint64_t str[2] = {2, (uint64_t)ldc * 2};
      uint32_t box[2] = {64, 32};
      const int rc = make_tmap(&smaps.m[r], ep.c_peer[r], 2, 2, dims, str, box, true);
      if (rc) return rc;
    }
  }
  return launch_gemm2<false, false>(a, b, ep, M, N, K, lda, ldb, reinterpret_cast<cudaStream_t>(stream), Comm2Work{},
                                    smaps);
}
