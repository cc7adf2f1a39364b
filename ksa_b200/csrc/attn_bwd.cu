// Backward attention for text queries on tcgen05 tensor cores, as two deterministic
// kernels that never accumulate across CTAs (no fp32 atomics, no dQ staging buffer,
// no pre/post-processing launches):
//
//   attn_bwd_dq    query-stationary.  One CTA = 128 query rows of one head; for every
//                  visible key tile: S = Q K^T, dP = dO V^T (tensor cores) ->
//                  P = exp2(S c - LSE), dS = P (dP - delta) scale (registers) ->
//                  dQ += dS K (dS is fed to the tensor cores from TMEM).  Also emits
//                  delta = rowsum(O * dO) for the second kernel.
//   attn_bwd_dkv   key-stationary.  One CTA = one 128-row key tile (text or summary)
//                  of one KV head; loops over the query tiles that see it and over
//                  the query heads of the group: S^T = K Q^T, dP^T = V dO^T ->
//                  P^T, dS^T -> dV += P^T dO, dK += dS^T Q, all four accumulators
//                  resident in TMEM (4 x 128 columns), GQA heads summed for free.
//
// The reference's sm_100 backward is key-stationary with dQ added into a global
// fp32 buffer by bulk reduce-adds plus separate pre- and post-processing kernels
// (flash_attn/cute/flash_bwd_sm100.py:1645-1798, :2422-2636 in the reference's flash_attn_cute wheel).
#include "attn_common.cuh"
#include "host.h"

namespace ksa {

constexpr int kBwdThreads = 320;   // TMA warp, MMA warp, two compute warpgroups
constexpr int kSumSeg = 8;          // query tiles per CTA for a summary-key tile (its query range is split)

template <int HD>
struct BwdSmem {
  static constexpr int kTile = 128 * HD * 2;
  static constexpr int kStationary = 2 * kTile;       // (Q, dO) or (K, V)
  static constexpr int kStages = 2;
  static constexpr int kRing = kStages * 2 * kTile;   // (K, V) or (Q, dO) pairs
  static constexpr int kStats = 2 * 2 * 128 * 4;      // LSE and delta of the current query tile, double-buffered
  static constexpr int kBar = 256;
  static constexpr int kTotal = kStationary + kRing + kStats + kBar + 1024;
};

struct BwdParams {
  AttnShape s;
  float scale, scale_log2;
  const bf16* o;   // [B, Lq, Hq, HD]
  const bf16* d_o; // same layout as o
  long long o_row_stride, o_batch_stride;
  const float* lse;  // [B, Hq, Lq]
  float* delta;      // [B, Hq, Lq]
  bf16* dq;          // [B, Lq, Hq, HD] (strides below)
  long long dq_row_stride, dq_batch_stride;
  bf16* dk; bf16* dv;     // text key grads [B, Lk, Hkv, HD]
  long long dk_row_stride, dk_batch_stride, dv_row_stride, dv_batch_stride;
  bf16* dks; bf16* dvs;   // summary key grads [B, Ns, Hkv, HD]
  long long dks_row_stride, dks_batch_stride, dvs_row_stride, dvs_batch_stride;
  float* dks32; float* dvs32;  // fp32 partial sums [B, Ns, Hkv, HD] when a summary tile's query range is split
  int n_seg;                   // segments per summary key tile (1: no split)
  int* status;
};

template <int HD>
__device__ __forceinline__ void load_tile_b(uint8_t* dst, const CUtensorMap* m, int row0, int h, int b, uint64_t* bar) {
#pragma unroll
  for (int half = 0; half < HD / 64; ++half) tma_load_4d(dst + half * 16384, m, half * 64, row0, h, b, bar);
}


// Store a row of HD fp32 accumulators from TMEM as bf16 to global memory.
template <int HD>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, bf16* dst, bool valid, float mul) {
#pragma unroll
  for (int c = 0; c < HD / 32; ++c) {
    uint32_t o[32];
    tmem_ld32(taddr + c * 32, o);
    tmem_wait_ld();
    if (valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(o[i]) * mul, __uint_as_float(o[i + 1]) * mul);
        v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * mul, __uint_as_float(o[i + 3]) * mul);
        v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * mul, __uint_as_float(o[i + 5]) * mul);
        v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * mul, __uint_as_float(o[i + 7]) * mul);
        *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
      }
    }
  }
}

// ================================================================================ dQ
template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmKs, const __grid_constant__ CUtensorMap tmVs, BwdParams p) {
  using S = BwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + S::kTile;
  uint8_t* sRing = smem + S::kStationary;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kStationary + S::kRing + S::kStats);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                 // kStages
  uint64_t* kv_empty = kv_full + S::kStages;    // kStages
  uint64_t* sp_full = kv_empty + S::kStages;    // 2: one per key half
  uint64_t* ds_full = sp_full + 2;              // 2
  uint64_t* dq_full = ds_full + 2;              // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};
  const AttnShape& sh = p.s;
  const int n_qtiles = (sh.Lq + 127) / 128;
  const int q_tile = n_qtiles - 1 - (int)blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (sh.Hq / sh.Hkv);
  const TileRange tr = key_tiles_for_query_tile(sh, q_tile, b);
  const int total = tr.total();

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < S::kStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int h = 0; h < 2; ++h) { mbar_init(&sp_full[h], 1); mbar_init(&ds_full[h], 128); }
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 2) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * S::kTile);
      load_tile_b<HD>(sQ, &tmQ, q_tile * 128, head, b, q_full);
      load_tile_b<HD>(sdO, &tmdO, q_tile * 128, head, b, q_full);
      for (int j = 0; j < total; ++j) {
        const int stage = j % S::kStages;
        const uint32_t phase = (j / S::kStages) & 1;
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, guard, kTimeoutStageEmpty)) break;
        const bool is_sum = j < tr.n_sum_tiles;
        const int kt = is_sum ? j : tr.text_first + (j - tr.n_sum_tiles);
        uint8_t* dst = sRing + stage * 2 * S::kTile;
        mbar_expect_tx(&kv_full[stage], 2 * S::kTile);
        load_tile_b<HD>(dst, is_sum ? &tmKs : &tmK, kt * 128, kv_head, b, &kv_full[stage]);
        load_tile_b<HD>(dst + S::kTile, is_sum ? &tmVs : &tmV, kt * 128, kv_head, b, &kv_full[stage]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The 128 keys of a tile are handled as two halves of 64 (one per softmax warpgroup), software-pipelined:
      // while a warpgroup turns the scores of its half into dS, the tensor pipe runs the other half's dQ update and
      // the next tile's S / dP for the half that has just been consumed.  tcgen05 MMAs issued by one thread execute
      // in order, so S/dP of step j+1 may be issued right behind the dQ MMA that reads dS of step j from the same
      // TMEM columns.
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, HD, 0, 1);
      const uint32_t qa = smem_u32(sQ), doa = smem_u32(sdO);
      auto issue_sdp = [&](int h, uint32_t ka, uint32_t va) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tS + h * 64, smem_desc_kmajor_sw128(qa + off), smem_desc_kmajor_sw128(ka + h * 8192 + off), idesc_s,
                  kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tdP + h * 64, smem_desc_kmajor_sw128(doa + off), smem_desc_kmajor_sw128(va + h * 8192 + off), idesc_s,
                  kk != 0);
        }
        umma_commit(&sp_full[h]);
      };
      bool ok = mbar_wait(q_full, 0, guard, kTimeoutTmaFull);
      if (ok && total > 0) {
        ok = mbar_wait(&kv_full[0], 0, guard, kTimeoutTmaFull);
        if (ok) {
          tc_fence_after();
          const uint32_t ka0 = smem_u32(sRing);
          issue_sdp(0, ka0, ka0 + S::kTile);
          issue_sdp(1, ka0, ka0 + S::kTile);
        }
      }
      for (int j = 0; j < total && ok; ++j) {
        const int stage = j % S::kStages;
        const uint32_t ka = smem_u32(sRing + stage * 2 * S::kTile);
        const int nstage = (j + 1) % S::kStages;
        const uint32_t kan = smem_u32(sRing + nstage * 2 * S::kTile);
        for (int h = 0; h < 2 && ok; ++h) {
          if (!mbar_wait(&ds_full[h], j & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = h * 4 + k4;
            umma_ts(tdQ, tS + h * 64 + k4 * 8, smem_desc_mnmajor_sw128(ka + kk * 2048, 16384), idesc_dq, (j | kk) != 0);
          }
          if (h == 1) umma_commit(&kv_empty[stage]);
          if (j + 1 < total) {
            if (h == 0) {
              if (!mbar_wait(&kv_full[nstage], ((j + 1) / S::kStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
              tc_fence_after();
            }
            issue_sdp(h, kan, kan + S::kTile);
          }
        }
      }
      if (ok) umma_commit(dq_full);
    }
  } else {
    // Two warpgroups share the 128 rows: warps 2-5 take score columns 0..63, warps 6-9 columns 64..127.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int q_local = q_tile * 128 + r;
    const bool valid = q_local < sh.Lq;
    const int t_glob = sh.q_off + q_local;
    const int doc_start = (sh.q_doc_start && valid) ? sh.q_doc_start[(long long)b * sh.Lq + q_local] : 0;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    // delta = rowsum(O * dO); LSE in log2 units
    float delta = 0.f, lse2 = INFINITY;
    if (valid) {
      const long long off = (long long)b * p.o_batch_stride + (long long)q_local * p.o_row_stride + (long long)head * HD;
      const uint4* po = reinterpret_cast<const uint4*>(p.o + off);
      const uint4* pd = reinterpret_cast<const uint4*>(p.d_o + off);
#pragma unroll 4
      for (int i = 0; i < HD / 8; ++i) {
        const uint4 a = po[i], g = pd[i];
        const uint32_t au[4] = {a.x, a.y, a.z, a.w}, gu[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = unpack_bf16x2(au[k]), y = unpack_bf16x2(gu[k]);
          delta += x.x * y.x + x.y * y.y;
        }
      }
      const long long sidx = ((long long)b * sh.Hq + head) * sh.Lq + q_local;
      lse2 = p.lse[sidx] * 1.4426950408889634f;
      if (half == 0) p.delta[sidx] = delta;
    }
    bool ok = true;
    for (int j = 0; j < total; ++j) {
      if (!mbar_wait(&sp_full[half], j & 1, guard, kTimeoutAccFull)) { ok = false; break; }
      tc_fence_after();
      const bool is_sum = j < tr.n_sum_tiles;
      const int kt = is_sum ? j : tr.text_first + (j - tr.n_sum_tiles);
      int lo, hi;
      allowed_columns(sh, t_glob, is_sum, kt, lo, hi, doc_start);
      // dS (bf16, two per column) overwrites the scores this warpgroup has already read:
      // chunk c goes to columns (c/2)*64 + (c%2)*16.  All four loads are issued before the single wait, so the
      // TMEM latency is paid once per step.
      uint32_t sr[2][32], dr[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld32(tS + lane_addr + (half * 2 + cc) * 32, sr[cc]);
        tmem_ld32(tdP + lane_addr + (half * 2 + cc) * 32, dr[cc]);
      }
      tmem_wait_ld();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + 2 * i + e;
            const float pr = (col >= lo && col <= hi)
                                 ? fast_exp2(fmaf(__uint_as_float(sr[cc][2 * i + e]), p.scale_log2, -lse2)) : 0.f;
            ds[e] = pr * (__uint_as_float(dr[cc][2 * i + e]) - delta) * p.scale;
          }
          pk[i] = pack_bf16x2(ds[0], ds[1]);
        }
        tmem_st16(tS + lane_addr + half * 64 + cc * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&ds_full[half]);
    }
    if (ok) ok = mbar_wait(dq_full, 0, guard, kTimeoutAccFull);
    if (ok) {
      tc_fence_after();
      bf16* dst = p.dq + (long long)b * p.dq_batch_stride + (long long)q_local * p.dq_row_stride + (long long)head * HD;
      store_acc_row<HD / 2>(tdQ + lane_addr + half * (HD / 2), dst + half * (HD / 2), valid, 1.f);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ================================================================================ dK / dV
// Grid x: first every (summary key tile, query segment) pair, then the text key tiles.  A summary key tile is
// seen by almost every later query tile, so its query range is cut into segments of kSumSeg tiles that run as
// separate CTAs and add their fp32 partial results into dks32/dvs32 (zeroed by the caller); the summary-query
// kernel, which runs next, folds those partials into the bf16 gradients.  With a single segment the CTA writes
// bf16 directly.  Text key tiles are seen by at most window+1 query tiles (all later ones for causal attention,
// where tile 0 is the heaviest and is scheduled first).
template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmKs, const __grid_constant__ CUtensorMap tmVs, BwdParams p) {
  using S = BwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + S::kTile;
  uint8_t* sRing = smem + S::kStationary;
  float* sLse = reinterpret_cast<float*>(smem + S::kStationary + S::kRing);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kStationary + S::kRing + S::kStats);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                // kStages
  uint64_t* q_empty = q_full + S::kStages;    // kStages
  uint64_t* sp_full = q_empty + S::kStages;   // 2: one per query half
  uint64_t* pds_full = sp_full + 2;           // 2
  uint64_t* acc_full = pds_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};
  const AttnShape& sh = p.s;
  const int n_sum_tiles = (sh.Ns + 127) / 128;
  const int n_seg = p.n_seg;
  const int n_sum_ctas = n_sum_tiles * n_seg;
  const bool is_sum = (int)blockIdx.x < n_sum_ctas;
  const int kt = is_sum ? (int)blockIdx.x / n_seg : (int)blockIdx.x - n_sum_ctas;
  const int seg = is_sum ? (int)blockIdx.x % n_seg : 0;
  const int kv_head = blockIdx.y, b = blockIdx.z;
  const int G = sh.Hq / sh.Hkv;
  QueryRange qr = is_sum ? query_tiles_for_summary_key_tile(sh, kt) : query_tiles_for_text_key_tile(sh, kt, blockIdx.z);
  if (is_sum && n_seg > 1) {
    qr.first = max(qr.first, seg * kSumSeg);
    qr.last = min(qr.last, seg * kSumSeg + kSumSeg - 1);
  }
  const int n_q = qr.last >= qr.first ? (qr.last - qr.first + 1) : 0;
  const int total = n_q * G;
  const bool atomic_out = is_sum && n_seg > 1;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < S::kStages; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int h = 0; h < 2; ++h) { mbar_init(&sp_full[h], 1); mbar_init(&pds_full[h], 128); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 2) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0 && total > 0) {
      mbar_expect_tx(kv_full, 2 * S::kTile);
      load_tile_b<HD>(sK, is_sum ? &tmKs : &tmK, kt * 128, kv_head, b, kv_full);
      load_tile_b<HD>(sV, is_sum ? &tmVs : &tmV, kt * 128, kv_head, b, kv_full);
      for (int i = 0; i < total; ++i) {
        const int stage = i % S::kStages;
        if (!mbar_wait(&q_empty[stage], ((i / S::kStages) & 1) ^ 1, guard, kTimeoutStageEmpty)) break;
        const int qt = qr.first + i / G, head = kv_head * G + i % G;
        uint8_t* dst = sRing + stage * 2 * S::kTile;
        mbar_expect_tx(&q_full[stage], 2 * S::kTile);
        load_tile_b<HD>(dst, &tmQ, qt * 128, head, b, &q_full[stage]);
        load_tile_b<HD>(dst + S::kTile, &tmdO, qt * 128, head, b, &q_full[stage]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && total > 0) {
      // Same software pipeline as the dQ kernel, over the two halves of 64 query columns: warpgroup h turns
      // S^T / dP^T of its half into P^T / dS^T while the tensor pipe updates dV / dK with the other half and computes
      // the next step's scores for the half that has just been consumed.
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, 0, 1);
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      auto issue_sdp = [&](int h, uint32_t qa, uint32_t doa) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tS + h * 64, smem_desc_kmajor_sw128(ka + off), smem_desc_kmajor_sw128(qa + h * 8192 + off), idesc_s,
                  kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
          umma_ss(tdP + h * 64, smem_desc_kmajor_sw128(va + off), smem_desc_kmajor_sw128(doa + h * 8192 + off), idesc_s,
                  kk != 0);
        }
        umma_commit(&sp_full[h]);
      };
      bool ok = mbar_wait(kv_full, 0, guard, kTimeoutTmaFull);
      if (ok) {
        ok = mbar_wait(&q_full[0], 0, guard, kTimeoutTmaFull);
        if (ok) {
          tc_fence_after();
          const uint32_t qa0 = smem_u32(sRing);
          issue_sdp(0, qa0, qa0 + S::kTile);
          issue_sdp(1, qa0, qa0 + S::kTile);
        }
      }
      for (int i = 0; i < total && ok; ++i) {
        const int stage = i % S::kStages, nstage = (i + 1) % S::kStages;
        const uint32_t qa = smem_u32(sRing + stage * 2 * S::kTile), doa = qa + S::kTile;
        const uint32_t qan = smem_u32(sRing + nstage * 2 * S::kTile);
        for (int h = 0; h < 2 && ok; ++h) {
          if (!mbar_wait(&pds_full[h], i & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = h * 4 + k4;
            umma_ts(tdV, tS + h * 64 + k4 * 8, smem_desc_mnmajor_sw128(doa + kk * 2048, 16384), idesc_acc, (i | kk) != 0);
          }
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = h * 4 + k4;
            umma_ts(tdK, tdP + h * 64 + k4 * 8, smem_desc_mnmajor_sw128(qa + kk * 2048, 16384), idesc_acc, (i | kk) != 0);
          }
          if (h == 1) umma_commit(&q_empty[stage]);
          if (i + 1 < total) {
            if (h == 0) {
              if (!mbar_wait(&q_full[nstage], ((i + 1) / S::kStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
              tc_fence_after();
            }
            issue_sdp(h, qan, qan + S::kTile);
          }
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // Two warpgroups share the 128 key rows: warps 2-5 take query columns 0..63, warps 6-9 columns 64..127.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int k_local = kt * 128 + r;
    const bool valid = k_local < (is_sum ? sh.Ns : sh.Lk);
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    // queries t (global) that may see this key: [t_lo, t_hi]
    long long t_lo, t_hi;
    if (is_sum) {
      const int sg = sh.s_off + k_local;
      t_lo = (long long)(sg / sh.n_sum + sh.window + 1) * sh.chunk;
      t_hi = (1LL << 40);
    } else {
      const int ug = sh.k_off + k_local;
      t_lo = ug;
      t_hi = (sh.window >= (1 << 29)) ? (1LL << 40) : (long long)(ug / sh.chunk + sh.window + 1) * sh.chunk - 1;
      if (sh.tok_window > 0) t_hi = min(t_hi, (long long)ug + sh.tok_window - 1);
      if (sh.k_doc_end && valid) t_hi = min(t_hi, (long long)sh.k_doc_end[(long long)b * sh.Lk + k_local] - 1);
    }
    if (!valid) { t_lo = 1; t_hi = 0; }
    bool ok = true;
    // LSE (threads 0..63 of the warpgroup) or delta (threads 64..127) of query column `half*64 + (r & 63)`; the value
    // for step i+1 is requested while step i is processed, so its global-memory latency is off the critical path.
    auto load_stat = [&](int i) -> float {
      const int qt = qr.first + i / G, head = kv_head * G + i % G;
      const int ql = qt * 128 + half * 64 + (r & 63);
      if (ql >= sh.Lq) return r < 64 ? INFINITY : 0.f;
      const long long sidx = ((long long)b * sh.Hq + head) * sh.Lq + ql;
      return r < 64 ? p.lse[sidx] * 1.4426950408889634f : p.delta[sidx];
    };
    float stat_next = total > 0 ? load_stat(0) : 0.f;
    for (int i = 0; i < total; ++i) {
      const int qt = qr.first + i / G;
      const bool got = mbar_wait(&sp_full[half], i & 1, guard, kTimeoutAccFull);
      // Staged per warpgroup and double-buffered by iteration parity: the buffer written here was last read two
      // iterations ago, and every thread of the warpgroup has passed its barrier between.
      // Layout per parity: [half][lse 64 | delta 64].
      float* lse_s = sLse + (i & 1) * 256 + half * 128;
      float* delta_s = lse_s + 64;
      lse_s[r] = stat_next;                   // r < 64: lse_s[r]; r >= 64: delta_s[r - 64]
      if (i + 1 < total) stat_next = load_stat(i + 1);
      (void)got;  // a failed wait has raised the CTA abort flag before returning
      if (half == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
      else asm volatile("bar.sync 2, 128;" ::: "memory");
      if (*abort_flag) { ok = false; break; }  // a raised flag stays raised: the other warpgroup sees it at its next step
      tc_fence_after();
      const long long tq0 = (long long)sh.q_off + qt * 128;
      const int lo = (int)max(t_lo - tq0, 0LL), hi = (int)min(t_hi - tq0, 127LL);
      // P^T and dS^T (bf16, two per column) overwrite scores this warpgroup has already read:
      // chunk c goes to columns (c/2)*64 + (c%2)*16.  All four loads are issued before the single wait.
      uint32_t sr[2][32], dr[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld32(tS + lane_addr + (half * 2 + cc) * 32, sr[cc]);
        tmem_ld32(tdP + lane_addr + (half * 2 + cc) * 32, dr[cc]);
      }
      tmem_wait_ld();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float pr[2], ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + 2 * k + e;
            pr[e] = (col >= lo && col <= hi)
                        ? fast_exp2(fmaf(__uint_as_float(sr[cc][2 * k + e]), p.scale_log2, -lse_s[col - half * 64])) : 0.f;
            ds[e] = pr[e] * (__uint_as_float(dr[cc][2 * k + e]) - delta_s[col - half * 64]) * p.scale;
          }
          pk[k] = pack_bf16x2(pr[0], pr[1]);
          dk[k] = pack_bf16x2(ds[0], ds[1]);
        }
        tmem_st16(tS + lane_addr + half * 64 + cc * 16, pk);
        tmem_st16(tdP + lane_addr + half * 64 + cc * 16, dk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&pds_full[half]);
    }
    // Epilogue: warpgroup 0 stores dV, warpgroup 1 stores dK.
    const bool do_k = half == 1;
    const uint32_t t_acc = (do_k ? tdK : tdV) + lane_addr;
    if (atomic_out) {
      if (total > 0) {
        if (ok) ok = mbar_wait(acc_full, 0, guard, kTimeoutAccFull);
        if (ok) {
          tc_fence_after();
          float* base = (do_k ? p.dks32 : p.dvs32) + (((long long)b * sh.Ns + k_local) * sh.Hkv + kv_head) * HD;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_acc + c * 32, o);
            tmem_wait_ld();
            if (valid) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                atomicAdd(reinterpret_cast<float4*>(base + c * 32 + i),
                          make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]), __uint_as_float(o[i + 2]),
                                      __uint_as_float(o[i + 3])));
            }
          }
        }
      }
    } else {
      bf16* gbase = is_sum ? (do_k ? p.dks : p.dvs) : (do_k ? p.dk : p.dv);
      const long long rs = is_sum ? (do_k ? p.dks_row_stride : p.dvs_row_stride) : (do_k ? p.dk_row_stride : p.dv_row_stride);
      const long long bs = is_sum ? (do_k ? p.dks_batch_stride : p.dvs_batch_stride)
                                  : (do_k ? p.dk_batch_stride : p.dv_batch_stride);
      bf16* dst = gbase + (long long)b * bs + (long long)k_local * rs + (long long)kv_head * HD;
      if (total == 0) {
        if (valid) {
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4*>(dst)[i] = z;
        }
      } else {
        if (ok) ok = mbar_wait(acc_full, 0, guard, kTimeoutAccFull);
        if (ok) {
          tc_fence_after();
          store_acc_row<HD>(t_acc, dst, valid, 1.f);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

static int make_head_tmap_b(CUtensorMap* m, const void* base, int HD, long long T, int H, int B, long long row_stride,
                            long long batch_stride) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)(T > 0 ? T : 1), (uint64_t)H, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)row_stride * 2, (uint64_t)HD * 2, (uint64_t)batch_stride * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap(m, base, 2, 4, dims, str, box, true);
}

template <int HD>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tks, const CUtensorMap& tvs, const BwdParams& p, cudaStream_t st) {
  auto k1 = attn_bwd_dq_kernel<HD>;
  auto k2 = attn_bwd_dkv_kernel<HD>;
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<HD>::kTotal));
    KSA_CHECK_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<HD>::kTotal));
    attr = true;
  }
  dim3 g1((p.s.Lq + 127) / 128, p.s.Hq, p.s.B);
  k1<<<g1, kBwdThreads, BwdSmem<HD>::kTotal, st>>>(tq, tdo, tk, tv, tks, tvs, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  dim3 g2((p.s.Lk + 127) / 128 + ((p.s.Ns + 127) / 128) * p.n_seg, p.s.Hkv, p.s.B);
  k2<<<g2, kBwdThreads, BwdSmem<HD>::kTotal, st>>>(tq, tdo, tk, tv, tks, tvs, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace ksa

// Number of CTAs a summary key tile's query range is split into for Lq local query rows.  When it is > 1 the
// caller passes zeroed fp32 buffers dks32/dvs32 [B, Ns, Hkv, HD] to ksa_attn_bwd and the same buffers to
// ksa_summary_attn_bwd, which adds them into the bf16 summary-key gradients.
KSA_API int ksa_attn_bwd_num_segments(int Lq) {
  const int n_qtiles = (Lq + 127) / 128;
  return (n_qtiles + ksa::kSumSeg - 1) / ksa::kSumSeg;
}

// Backward of ksa_attn_fwd.  Extra inputs: o, d_o [B, Lq, Hq, HD] (same strides), lse [B, Hq, Lq];
// outputs dq (strides dq_rs/dq_bs), dk/dv (text keys), dks/dvs (summary keys), and delta [B, Hq, Lq] (scratch the
// caller provides: rowsum(O*dO), written by the first kernel and read by the second).
KSA_API int ksa_attn_bwd(const void* q, const void* k, const void* v, const void* ks, const void* vs, const void* o,
                         const void* d_o, const void* lse, void* delta, void* dq, void* dk, void* dv, void* dks,
                         void* dvs, int B, int Hq, int Hkv, int HD, int Lq, int Lk, int Ns, long long q_rs,
                         long long q_bs, long long k_rs, long long k_bs, long long v_rs, long long v_bs,
                         long long ks_rs, long long ks_bs, long long vs_rs, long long vs_bs, long long o_rs,
                         long long o_bs, long long dq_rs, long long dq_bs, long long dk_rs, long long dk_bs,
                         long long dv_rs, long long dv_bs, long long dks_rs, long long dks_bs, long long dvs_rs,
                         long long dvs_bs, int q_off, int k_off, int s_off, int chunk, int n_sum, int window,
                         int tok_window, float scale, void* dks32, void* dvs32, const void* q_doc_start,
                         const void* k_doc_end, void* stream) {
  KSA_ENTER(q);
  using namespace ksa;
  KSA_REQUIRE(HD == 128 || HD == 64, "attn_bwd: head_dim %d unsupported (64 or 128)", HD);
  KSA_REQUIRE(Hq % Hkv == 0, "attn_bwd: Hq %% Hkv != 0");
  KSA_REQUIRE(o_rs % 8 == 0 && dq_rs % 8 == 0 && dk_rs % 8 == 0 && dv_rs % 8 == 0, "attn_bwd: row strides must be multiples of 8");
  if (B == 0 || Lq == 0) return 0;
  CUtensorMap tq, tdo, tk, tv, tks, tvs;
  int rc;
  if ((rc = make_head_tmap_b(&tq, q, HD, Lq, Hq, B, q_rs, q_bs))) return rc;
  if ((rc = make_head_tmap_b(&tdo, d_o, HD, Lq, Hq, B, o_rs, o_bs))) return rc;
  if ((rc = make_head_tmap_b(&tk, k, HD, Lk, Hkv, B, k_rs, k_bs))) return rc;
  if ((rc = make_head_tmap_b(&tv, v, HD, Lk, Hkv, B, v_rs, v_bs))) return rc;
  if (Ns > 0) {
    if ((rc = make_head_tmap_b(&tks, ks, HD, Ns, Hkv, B, ks_rs, ks_bs))) return rc;
    if ((rc = make_head_tmap_b(&tvs, vs, HD, Ns, Hkv, B, vs_rs, vs_bs))) return rc;
  } else {
    tks = tk;
    tvs = tv;
  }
  BwdParams p;
  p.s = AttnShape{B, Hq, Hkv, Lq, Lk, Ns, q_off, k_off, s_off, chunk, n_sum > 0 ? n_sum : 1, window, tok_window,
                  (const int*)q_doc_start, (const int*)k_doc_end};
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = (const bf16*)o; p.d_o = (const bf16*)d_o; p.o_row_stride = o_rs; p.o_batch_stride = o_bs;
  p.lse = (const float*)lse; p.delta = (float*)delta;
  p.dq = (bf16*)dq; p.dq_row_stride = dq_rs; p.dq_batch_stride = dq_bs;
  p.dk = (bf16*)dk; p.dv = (bf16*)dv;
  p.dk_row_stride = dk_rs; p.dk_batch_stride = dk_bs; p.dv_row_stride = dv_rs; p.dv_batch_stride = dv_bs;
  p.dks = (bf16*)dks; p.dvs = (bf16*)dvs;
  p.dks_row_stride = dks_rs; p.dks_batch_stride = dks_bs; p.dvs_row_stride = dvs_rs; p.dvs_batch_stride = dvs_bs;
  p.dks32 = (float*)dks32; p.dvs32 = (float*)dvs32;
  p.n_seg = (Ns > 0 && dks32 != nullptr && dvs32 != nullptr) ? ksa_attn_bwd_num_segments(Lq) : 1;
  p.status = status_word();
  KSA_REQUIRE(p.status != nullptr, "could not allocate the status word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return HD == 128 ? launch_bwd<128>(tq, tdo, tk, tv, tks, tvs, p, st) : launch_bwd<64>(tq, tdo, tk, tv, tks, tvs, p, st);
}
