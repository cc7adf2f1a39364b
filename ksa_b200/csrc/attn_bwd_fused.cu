// Backward attention for text queries as ONE key-stationary tcgen05 kernel (head dim 128): the scores and
// dP of every (key tile, query tile) pair are computed once and feed dV, dK and dQ (five products per pair
// instead of the seven of the two-kernel form in attn_bwd.cu, which stays as the bit-reproducible path).
//
// One CTA owns one 128-row key tile (text or summary) of one KV head and walks the query tiles that see it
// and the query heads of the group.  A step is one 128-query tile of one head.  Its scores and dP are issued as
// 128-column products (a product whose A operand comes from shared memory takes the time of reading that 128 x 16
// block however narrow it is, so 64-column products would run at half rate); everything after them works on two
// halves of 64 query columns, one per compute warpgroup:
//
//   S^T    = K Q^T,    dP^T   = V dO^T                         (tensor cores, 128 keys x 128 queries each)
//   P^T_h  = exp2(S^T_h c - LSE),  dS^T_h = P^T_h (dP^T_h - delta)   (registers; bf16 back to TMEM, dS^T_h also to smem)
//   dQ^T_h = K^T dS^T_h    (128 head dims x 64 queries; replaces dP^T_h in TMEM and is added to a global fp32
//                           buffer with TMA reductions by the same warpgroup, 32 head dims per warp)
//   dV    += P^T_h dO_h,  dK += dS^T_h Q_h                     (accumulators stay in TMEM for the whole CTA)
//
// The next step's S^T is issued behind dV / dK (the last readers of P^T and dS^T), its dP^T once both halves of
// dQ^T have been read out.
//
//   warp 0      TMA producer: K, V once; then (Q, dO, -LSE*log2e, -delta) per step, 2-stage ring
//   warp 1      MMA issuer (one elected thread)
//   warps 2-5   compute warpgroup of half 0 (thread = key row)
//   warps 6-9   compute warpgroup of half 1
//
// TMEM (512 columns): S^T_h @ h*64 (P^T_h, bf16, over its columns 0..31 and dS^T_h over 32..63),
// dP^T_h / dQ^T_h @ 128 + h*64, dV @ 256, dK @ 384.
//
// Two small kernels surround it: a preparation pass (delta = rowsum(O * dO), scaled LSE, zeroing of the fp32
// dQ buffer) and a conversion pass (dQ fp32 -> bf16, times the softmax scale).  The key-stationary order,
// the five products and the fp32 dQ buffer filled by reductions are those of the reference wheel's sm_100
// backward (flash_attn/cute/flash_bwd_sm100.py:1645-1798, :2422-2636 in the flash_attn_cute wheel); the tile
// enumeration is closed-form (attn_common.cuh) instead of block lists.
#include "attn_common.cuh"
#include "host.h"
#include <string.h>

namespace ksa {

constexpr int kFbThreads = 320;
constexpr int kFbStages = 2;   // stages of the (Q, dO) ring, one 128-query tile of one head each
constexpr int kFbSumSeg = 8;   // query tiles per CTA for a summary-key tile (must match ksa_attn_bwd_num_segments)

struct FbSmem {
  static constexpr int kTile = 128 * 128 * 2;        // K or V: [2 head-dim halves][128 rows][128 B]
  static constexpr int kHalfTile = 64 * 128 * 2;     // Q_h or dO_h: [2 head-dim halves][64 rows][128 B]
  static constexpr int kStage = 2 * kTile;           // Q tile then dO tile, each [2 head-dim halves][128 rows][128 B]
  static constexpr int kRing = kFbStages * kStage;
  static constexpr int kDs = 2 * kHalfTile;          // dS^T_h: [128 key rows][64 queries] bf16, one per half
  static constexpr int kStats = kFbStages * 1024;    // per stage: -LSE*log2e [128], -delta [128]
  static constexpr int kBar = 256;
  static constexpr int kOffRing = 2 * kTile;
  static constexpr int kOffDs = kOffRing + kRing;
  static constexpr int kOffStats = kOffDs + kDs;
  static constexpr int kOffBar = kOffStats + kStats;
  static constexpr int kTotal = kOffBar + kBar;      // 231680 bytes: the dynamic segment must start 1024-aligned
  static constexpr int kStageBytes = kStage + 1024;  // bytes a full stage receives
};

struct FbParams {
  AttnShape s;
  float scale, scale_log2;
  const float* stats;   // [2][B, Hq, Lq_pad]: -LSE*log2e, then -delta
  int lq_pad;
  float* dq32;          // [B, Lq, Hq, 128] fp32, zeroed by the preparation kernel
  bf16* dk; bf16* dv;   // text key grads [B, Lk, Hkv, 128]
  long long dk_row_stride, dk_batch_stride, dv_row_stride, dv_batch_stride;
  bf16* dks; bf16* dvs; // summary key grads [B, Ns, Hkv, 128]
  long long dks_row_stride, dks_batch_stride, dvs_row_stride, dvs_batch_stride;
  float* dks32; float* dvs32;  // fp32 partial sums [B, Ns, Hkv, 128] when a summary tile's query range is split
  int n_seg;
  int* status;
};

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// fp32 add of a box in shared memory (row-major, as the tensor map's box says: here 32 query rows of 32 head
// dimensions, 128-byte rows) into a 4-D fp32 tensor.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int x, int y, int z, int w) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(m), "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

// 32 score columns and 32 dP columns of one key row -> 16 packed P and 16 packed dS words.
// `st` points at -LSE*log2e of the first column, `sd` at its -delta; columns outside [lo, lo + span] are masked
// when `masked` is set (col0 is the first column's index inside the half).
__device__ __forceinline__ void softmax_grad_32(const uint32_t (&s)[32], const uint32_t (&d)[32], const float* st,
                                                const float* sd, float scale_log2, bool masked, int col0, int lo,
                                                unsigned span, uint32_t (&pk)[16], uint32_t (&dk)[16]) {
  const uint64_t sc2 = f2_pack(scale_log2, scale_log2);
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const float4 nl = *reinterpret_cast<const float4*>(st + g * 4);
    const float4 nd = *reinterpret_cast<const float4*>(sd + g * 4);
    const float nls[4] = {nl.x, nl.y, nl.z, nl.w}, nds[4] = {nd.x, nd.y, nd.z, nd.w};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = g * 4 + e * 2;
      const uint64_t x = f2_fma(f2_pack(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2,
                                f2_pack(nls[e * 2], nls[e * 2 + 1]));
      float x0, x1;
      f2_unpack(x, x0, x1);
      float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
      if (masked) {
        if ((unsigned)(col0 + i - lo) > span) p0 = 0.f;
        if ((unsigned)(col0 + i + 1 - lo) > span) p1 = 0.f;
      }
      const uint64_t t = f2_add(f2_pack(__uint_as_float(d[i]), __uint_as_float(d[i + 1])),
                                f2_pack(nds[e * 2], nds[e * 2 + 1]));
      float g0, g1;
      f2_unpack(f2_mul(f2_pack(p0, p1), t), g0, g1);
      pk[i >> 1] = pack_bf16x2(p0, p1);
      dk[i >> 1] = pack_bf16x2(g0, g1);
    }
  }
}

__device__ __forceinline__ void store_row_bf16_128(uint32_t taddr, bf16* dst, bool valid, float mul) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
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

// Context-parallel shard: where the key tiles come from (attn_common.cuh) and where the gradients of keys that
// other ranks own go: fp32 return blocks in the owners' memory, [B, rows, 2*Hkv*128] with K in the first Hkv*128
// columns, added to with reductions over NVLink; the owner folds them into its own dK / dV afterwards.
struct CpBwdSources {
  CpSources src;
  int n_sum_src;                  // summary sources; the last one is this rank's own
  float* ret_text;                // return block of the halo's owner (its last `halo` text rows)
  float* ret_sum[kCpMaxSum];      // return blocks of the owners of the older summaries
  long long ret_rs, ret_text_bs, ret_sum_bs;   // row stride and batch strides, elements
};

template <bool kCp>
__device__ __forceinline__ void attn_bwd_fused_body(const CUtensorMap& tmQ, const CUtensorMap& tmdO,
                                                    const CUtensorMap& tmK, const CUtensorMap& tmV,
                                                    const CUtensorMap& tmKs, const CUtensorMap& tmVs,
                                                    const CUtensorMap& tmDq, const FbParams& p,
                                                    const CpBwdSources* cp) {
  using S = FbSmem;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + S::kTile;
  uint8_t* sRing = smem + S::kOffRing;
  uint8_t* sDs = smem + S::kOffDs;
  uint8_t* sStats = smem + S::kOffStats;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kOffBar);
  uint64_t* kv_full = bars;                      // 1
  uint64_t* st_full = bars + 1;                  // kFbStages
  uint64_t* st_empty = st_full + kFbStages;      // kFbStages
  uint64_t* sp_full = st_empty + kFbStages;      // S^T and dP^T of a step are in TMEM (first of two slots used)
  uint64_t* pds_full = sp_full + 2;              // 2: P^T_h and dS^T_h are written (TMEM and smem)
  uint64_t* dq_full = pds_full + 2;              // 2: dQ^T_h is in TMEM
  uint64_t* dq_drained = dq_full + 2;            // 2: dQ^T_h has been read out
  uint64_t* acc_full = dq_drained + 2;           // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};
  const AttnShape& sh = p.s;
  // The swizzled tiles need a 1024-byte aligned base and the budget has no room for padding.
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (int)kBadArgument);
    return;
  }
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
    qr.first = max(qr.first, seg * kFbSumSeg);
    qr.last = min(qr.last, seg * kFbSumSeg + kFbSumSeg - 1);
  }
  const int n_q = qr.last >= qr.first ? (qr.last - qr.first + 1) : 0;
  const int total = n_q * G;          // steps: one 128-query tile of one head each
  const bool atomic_out = is_sum && n_seg > 1;
  // context parallel: source of this key tile, its first row there, and whether another rank owns it
  int cp_src = 0, cp_row = kt * 128;
  bool remote = false;
  if (kCp) {
    cp_src = is_sum ? (kt * 128) / cp->src.nsl : (kt * 128 < cp->src.halo ? 0 : 1);
    cp_row = is_sum ? (kt * 128) % cp->src.nsl : (cp_src == 0 ? kt * 128 : kt * 128 - cp->src.halo);
    remote = is_sum ? cp_src < cp->n_sum_src - 1 : cp_src == 0;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kFbStages; ++i) { mbar_init(&st_full[i], 1); mbar_init(&st_empty[i], 1); }
    mbar_init(&sp_full[0], 1);
    for (int h = 0; h < 2; ++h) {
      mbar_init(&pds_full[h], 128);
      mbar_init(&dq_full[h], 1);
      mbar_init(&dq_drained[h], 128);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 2) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && total > 0) {
      const CUtensorMap* mk = is_sum ? &tmKs : &tmK;
      const CUtensorMap* mv = is_sum ? &tmVs : &tmV;
      bool src_ok = true;
      if (kCp) {
        mk = is_sum ? &cp->src.ks[cp_src] : &cp->src.kt[cp_src];
        mv = is_sum ? &cp->src.vs[cp_src] : &cp->src.vt[cp_src];
        const uint32_t* flag = is_sum ? cp->src.sum_flag[cp_src] : cp->src.text_flag[cp_src];
        if (flag != nullptr && !flag_wait_ge(flag, cp->src.flag_target, p.status, kTimeoutPeerFlag, true)) {
          *abort_flag = 1;
          src_ok = false;
        }
      }
      mbar_expect_tx(kv_full, 2 * S::kTile);
      for (int hh = 0; hh < 2 && src_ok; ++hh) {
        tma_load_4d(sK + hh * 16384, mk, hh * 64, cp_row, kv_head, b, kv_full);
        tma_load_4d(sV + hh * 16384, mv, hh * 64, cp_row, kv_head, b, kv_full);
      }
      const long long plane = (long long)sh.B * sh.Hq * p.lq_pad;
      for (int j = 0; j < total && src_ok; ++j) {
        const int stage = j % kFbStages;
        if (!mbar_wait(&st_empty[stage], ((j / kFbStages) & 1) ^ 1, guard, kTimeoutStageEmpty)) break;
        const int qt = qr.first + j / G, head = kv_head * G + j % G;
        const int row0 = qt * 128;
        uint8_t* dst = sRing + stage * S::kStage;
        mbar_expect_tx(&st_full[stage], S::kStageBytes);
        for (int hh = 0; hh < 2; ++hh) {
          tma_load_4d(dst + hh * 16384, &tmQ, hh * 64, row0, head, b, &st_full[stage]);
          tma_load_4d(dst + S::kTile + hh * 16384, &tmdO, hh * 64, row0, head, b, &st_full[stage]);
        }
        const float* src = p.stats + ((long long)b * sh.Hq + head) * p.lq_pad + row0;
        bulk_load(sStats + stage * 1024, src, 512, &st_full[stage]);
        bulk_load(sStats + stage * 1024 + 512, src + plane, 512, &st_full[stage]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && total > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);    // S^T, dP^T: all 128 queries of the step at once
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);  // dV, dK: A from TMEM, B MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 64, 1, 1);    // dQ^T_h: A = K^T, B = dS^T_h, both MN-major
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      auto stage_addr = [&](int j) { return smem_u32(sRing + (j % kFbStages) * S::kStage); };
      // A product whose A operand comes from shared memory takes the time of reading its 128 x 16 A block however
      // narrow it is, so S^T and dP^T are issued 128 columns wide (both halves of the query tile in one product).
      auto issue_s = [&](int j) {
        const uint32_t qa = stage_addr(j);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tS, smem_desc_kmajor_sw128(ka + (kk / 4) * 16384 + (kk % 4) * 32),
                  smem_desc_kmajor_sw128(qa + (kk / 4) * 16384 + (kk % 4) * 32), idesc_s, kk != 0);
      };
      auto issue_dp = [&](int j) {
        const uint32_t doa = stage_addr(j) + S::kTile;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tdP, smem_desc_kmajor_sw128(va + (kk / 4) * 16384 + (kk % 4) * 32),
                  smem_desc_kmajor_sw128(doa + (kk / 4) * 16384 + (kk % 4) * 32), idesc_s, kk != 0);
      };
      bool ok = mbar_wait(kv_full, 0, guard, kTimeoutTmaFull);
      if (ok) ok = mbar_wait(&st_full[0], 0, guard, kTimeoutTmaFull);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
        umma_commit(&sp_full[0]);
      }
      for (int j = 0; j < total && ok; ++j) {
        const uint32_t qa = stage_addr(j), doa = qa + S::kTile;
        for (int h = 0; h < 2 && ok; ++h) {
          const uint32_t dsa = smem_u32(sDs + h * S::kHalfTile);
          if (!mbar_wait(&pds_full[h], j & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
          tc_fence_after();
          // dQ^T_h first: it replaces dP^T_h, which the warpgroup has consumed, and its read-out then overlaps dV / dK.
          // (One 128-column product for both halves was measured too: no faster, and it makes half 0 wait for half 1.)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tdP + h * 64, smem_desc_mnmajor_sw128(ka + kk * 2048, 16384),
                    smem_desc_mnmajor_sw128(dsa + kk * 2048, 8192), idesc_dq, kk != 0);
          umma_commit(&dq_full[h]);
          // dV += P_h^T dO_h, dK += dS_h^T Q_h: the half's 64 query rows of the stage's tiles, 16 per product
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_ts(tdV, tS + h * 64 + k4 * 8, smem_desc_mnmajor_sw128(doa + h * 8192 + k4 * 2048, 16384), idesc_acc,
                    (j | h | k4) != 0);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_ts(tdK, tS + h * 64 + 32 + k4 * 8, smem_desc_mnmajor_sw128(qa + h * 8192 + k4 * 2048, 16384), idesc_acc,
                    (j | h | k4) != 0);
        }
        if (!ok) break;
        umma_commit(&st_empty[j % kFbStages]);
        if (j + 1 < total) {
          if (!mbar_wait(&st_full[(j + 1) % kFbStages], ((j + 1) / kFbStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);       // behind dV / dK in the pipe, which were the last readers of P^T and dS^T in TMEM
          if (!mbar_wait(&dq_drained[0], j & 1, guard, kTimeoutAccEmpty)) { ok = false; break; }
          if (!mbar_wait(&dq_drained[1], j & 1, guard, kTimeoutAccEmpty)) { ok = false; break; }
          tc_fence_after();
          issue_dp(j + 1);
          umma_commit(&sp_full[0]);
        }
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;          // key row of the tile; head-dim index when dQ^T_h is read out
    const int k_local = kt * 128 + r;
    const bool valid = k_local < (is_sum ? sh.Ns : sh.Lk);
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t tSh = tS + lane_addr + half * 64, tdPh = tdP + lane_addr + half * 64;
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
    uint8_t* ds_row = sDs + half * S::kHalfTile + r * 128;   // this key's row of dS^T_h (64 bf16, swizzled 16-byte chunks)
    const int sw = r & 7;
    bool ok = true;
    for (int j = 0; j < total; ++j) {
      const int stage = j % kFbStages;
      const int qt = qr.first + j / G, head = kv_head * G + j % G;
      if (!mbar_wait(&sp_full[0], j & 1, guard, kTimeoutAccFull)) { ok = false; break; }
      // the row statistics arrived with the stage; waiting on its barrier makes them visible to this thread
      if (!mbar_wait(&st_full[stage], (j / kFbStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
      tc_fence_after();
      const float* st = reinterpret_cast<const float*>(sStats + stage * 1024) + half * 64;   // -LSE * log2e
      const float* sd = st + 128;                                                              // -delta
      const long long tq0 = (long long)sh.q_off + qt * 128 + half * 64;
      int lo = (int)max(t_lo - tq0, 0LL);
      const int hi = (int)min(t_hi - tq0, 63LL);
      unsigned span;
      if (hi < lo) { lo = 64; span = 0; } else { span = (unsigned)(hi - lo); }
      const bool masked = !__all_sync(0xffffffffu, lo == 0 && hi >= 63);
      uint32_t s0[32], s1[32], d[32], pk[16], dk[16];
      tmem_ld32(tSh, s0);
      tmem_ld32(tSh + 32, s1);
      tmem_ld32(tdPh, d);
      tmem_wait_ld();
      softmax_grad_32(s0, d, st, sd, p.scale_log2, masked, 0, lo, span, pk, dk);
      tmem_ld32(tdPh + 32, d);
      tmem_st16(tSh, pk);
      tmem_st16(tSh + 32, dk);
      // This warp's 32 rows of dS^T_h (4 KB) are also where it stages its slab of the previous step's dQ^T_h: its own
      // reductions must have read them.  Every warp stages and reduces its own 32 head dimensions, so the hand-offs
      // inside the drain are warp-wide, not warpgroup-wide.
      if (lane == 0) tma_store_wait_read0();
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(ds_row + ((c ^ sw) << 4)) = make_uint4(dk[4 * c], dk[4 * c + 1], dk[4 * c + 2], dk[4 * c + 3]);
      tmem_wait_ld();
      softmax_grad_32(s1, d, st + 32, sd + 32, p.scale_log2, masked, 32, lo, span, pk, dk);
      tmem_st16(tSh + 16, pk);
      tmem_st16(tSh + 48, dk);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(ds_row + (((c + 4) ^ sw) << 4)) = make_uint4(dk[4 * c], dk[4 * c + 1], dk[4 * c + 2], dk[4 * c + 3]);
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&pds_full[half]);
      // dQ^T_h: lane = head-dim index r, 64 query columns
      if (!mbar_wait(&dq_full[half], j & 1, guard, kTimeoutAccFull)) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(tdPh, s0);
      tmem_ld32(tdPh + 32, s1);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&dq_drained[half]);
      // Stage 32 query rows at a time as [query][this warp's 32 head dimensions] fp32 (128-byte rows, 4 KB) in the
      // warp's part of the dS^T_h buffer, which the dQ product has finished reading, and add them to the global fp32
      // dQ with one TMA reduction each; rows past Lq are clipped by the tensor map.
      const int q0 = qt * 128 + half * 64;
      float* stg = reinterpret_cast<float*>(sDs + half * S::kHalfTile + quad * 4096);
#pragma unroll
      for (int c = 0; c < 32; ++c) stg[c * 32 + lane] = __uint_as_float(s0[c]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (q0 < sh.Lq) tma_reduce_add_4d(&tmDq, stg, quad * 32, head, q0, b);
        tma_store_commit();
        tma_store_wait_read0();
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 32; ++c) stg[c * 32 + lane] = __uint_as_float(s1[c]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        if (q0 + 32 < sh.Lq) tma_reduce_add_4d(&tmDq, stg, quad * 32, head, q0 + 32, b);
        tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait0();   // this warp's last reductions have left shared memory and reached global memory
    // Epilogue: warpgroup 0 stores dV, warpgroup 1 stores dK (times the softmax scale).
    const bool do_k = half == 1;
    const float mul = do_k ? p.scale : 1.f;
    const uint32_t t_acc = (do_k ? tdK : tdV) + lane_addr;
    if (kCp && remote) {
      // keys of another rank: add this shard's contribution into the owner's fp32 return block over NVLink
      if (total > 0) {
        if (ok) ok = mbar_wait(acc_full, 0, guard, kTimeoutAccFull);
        if (ok) {
          tc_fence_after();
          float* blk = is_sum ? cp->ret_sum[cp_src] : cp->ret_text;
          const long long bs = is_sum ? cp->ret_sum_bs : cp->ret_text_bs;
          float* base = blk + (long long)b * bs + (long long)(cp_row + r) * cp->ret_rs + (do_k ? 0 : sh.Hkv * 128) + kv_head * 128;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(t_acc + c * 32, o);
            tmem_wait_ld();
            if (valid) {
#pragma unroll
              for (int i = 0; i < 32; ++i) atomicAdd(base + c * 32 + i, __uint_as_float(o[i]) * mul);
            }
          }
        }
      }
    } else if (atomic_out) {
      if (total > 0) {
        if (ok) ok = mbar_wait(acc_full, 0, guard, kTimeoutAccFull);
        if (ok) {
          tc_fence_after();
          float* base = (do_k ? p.dks32 : p.dvs32) + (((long long)b * sh.Ns + k_local) * sh.Hkv + kv_head) * 128;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(t_acc + c * 32, o);
            tmem_wait_ld();
            if (valid) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                atomicAdd(reinterpret_cast<float4*>(base + c * 32 + i),
                          make_float4(__uint_as_float(o[i]) * mul, __uint_as_float(o[i + 1]) * mul,
                                      __uint_as_float(o[i + 2]) * mul, __uint_as_float(o[i + 3]) * mul));
            }
          }
        }
      }
    } else {
      bf16* gbase = is_sum ? (do_k ? p.dks : p.dvs) : (do_k ? p.dk : p.dv);
      const long long rs = is_sum ? (do_k ? p.dks_row_stride : p.dvs_row_stride) : (do_k ? p.dk_row_stride : p.dv_row_stride);
      const long long bs = is_sum ? (do_k ? p.dks_batch_stride : p.dvs_batch_stride)
                                  : (do_k ? p.dk_batch_stride : p.dv_batch_stride);
      bf16* dst = gbase + (long long)b * bs + (long long)k_local * rs + (long long)kv_head * 128;
      if (total == 0) {
        if (valid) {
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < 16; ++i) reinterpret_cast<uint4*>(dst)[i] = z;
        }
      } else {
        if (ok) ok = mbar_wait(acc_full, 0, guard, kTimeoutAccFull);
        if (ok) {
          tc_fence_after();
          store_row_bf16_128(t_acc, dst, valid, mul);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

__global__ void __launch_bounds__(kFbThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmKs, const __grid_constant__ CUtensorMap tmVs,
                      const __grid_constant__ CUtensorMap tmDq, FbParams p) {
  attn_bwd_fused_body<false>(tmQ, tmdO, tmK, tmV, tmKs, tmVs, tmDq, p, nullptr);
}

__global__ void __launch_bounds__(kFbThreads, 1)
attn_bwd_fused_cp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                         const __grid_constant__ CUtensorMap tmDq, const __grid_constant__ CpBwdSources cp, FbParams p) {
  attn_bwd_fused_body<true>(tmQ, tmdO, cp.src.kt[1], cp.src.vt[1], cp.src.ks[0], cp.src.vs[0], tmDq, p, &cp);
}

// Preparation: one warp per (batch, head, query row of the padded length).  Writes -LSE*log2e and
// -delta = -rowsum(O * dO) into the two planes of `stats` (rows past Lq: -inf and 0, so that P = 0 there) and
// zeroes the row of the fp32 dQ buffer.
__global__ void attn_bwd_prep_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, long long o_rs,
                                     long long o_bs, const float* __restrict__ lse, float* __restrict__ stats,
                                     float* __restrict__ dq32, int B, int Hq, int Lq, int lq_pad) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)B * Hq * lq_pad;
  if (w >= rows) return;
  const int q = (int)(w % lq_pad);
  const int head = (int)((w / lq_pad) % Hq);
  const int b = (int)(w / ((long long)lq_pad * Hq));
  float nl = -INFINITY, nd = 0.f;
  if (q < Lq) {
    const long long off = (long long)b * o_bs + (long long)q * o_rs + (long long)head * 128 + lane * 4;
    const uint2 a = *reinterpret_cast<const uint2*>(o + off);
    const uint2 g = *reinterpret_cast<const uint2*>(d_o + off);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
    const float part = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
    nd = -warp_sum(part);
    const float l = lse[((long long)b * Hq + head) * Lq + q];
    nl = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
    // a query row without any visible key has LSE = -inf: P must be 0, not exp2(+inf)
    if (l == -INFINITY) nl = -INFINITY;
    *reinterpret_cast<float4*>(dq32 + (((long long)b * Lq + q) * Hq + head) * 128 + lane * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (lane == 0) {
    stats[w] = nl;
    stats[rows + w] = nd;
  }
}

// Conversion: dq = bf16(dq32 * scale).  One thread per 8 elements.
__global__ void attn_bwd_dq_convert_kernel(const float* __restrict__ dq32, bf16* __restrict__ dq, long long dq_rs,
                                           long long dq_bs, int B, int Lq, int Hq, float scale) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // over B * Lq * Hq * 16
  const long long n = (long long)B * Lq * Hq * 16;
  if (idx >= n) return;
  const int c = (int)(idx & 15);
  const long long row = idx >> 4;          // (b * Lq + q) * Hq + head
  const int head = (int)(row % Hq);
  const long long bq = row / Hq;
  const int q = (int)(bq % Lq);
  const int b = (int)(bq / Lq);
  const float4 x = *reinterpret_cast<const float4*>(dq32 + row * 128 + c * 8);
  const float4 y = *reinterpret_cast<const float4*>(dq32 + row * 128 + c * 8 + 4);
  uint4 v;
  v.x = pack_bf16x2(x.x * scale, x.y * scale);
  v.y = pack_bf16x2(x.z * scale, x.w * scale);
  v.z = pack_bf16x2(y.x * scale, y.y * scale);
  v.w = pack_bf16x2(y.z * scale, y.w * scale);
  *reinterpret_cast<uint4*>(dq + (long long)b * dq_bs + (long long)q * dq_rs + (long long)head * 128 + c * 8) = v;
}

static int make_head_tmap_rows(CUtensorMap* m, const void* base, long long T, int H, int B, long long row_stride,
                               long long batch_stride, int box_rows) {
  uint64_t dims[4] = {128, (uint64_t)(T > 0 ? T : 1), (uint64_t)H, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)row_stride * 2, 128 * 2, (uint64_t)batch_stride * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap(m, base, 2, 4, dims, str, box, true);
}

}  // namespace ksa

// Padded query length of the `stats` workspace of ksa_attn_bwd_fused.
KSA_API int ksa_attn_bwd_fused_lq_pad(int Lq) { return (Lq + 127) / 128 * 128; }

// Backward of ksa_attn_fwd for head dim 128 as one key-stationary kernel plus a preparation and a conversion pass.
// Same tensors as ksa_attn_bwd; the workspaces are `stats` (fp32, 2 * B * Hq * ksa_attn_bwd_fused_lq_pad(Lq)
// elements) and `dq32` (fp32, B * Lq * Hq * 128 elements), both written before they are read.  dQ is accumulated with
// floating-point reductions whose order varies from run to run: results agree to rounding, not bit for bit
// (ksa_attn_bwd is the reproducible form).
KSA_API int ksa_attn_bwd_fused(const void* q, const void* k, const void* v, const void* ks, const void* vs,
                               const void* o, const void* d_o, const void* lse, void* stats, void* dq32, void* dq,
                               void* dk, void* dv, void* dks, void* dvs, int B, int Hq, int Hkv, int HD, int Lq, int Lk,
                               int Ns, long long q_rs, long long q_bs, long long k_rs, long long k_bs, long long v_rs,
                               long long v_bs, long long ks_rs, long long ks_bs, long long vs_rs, long long vs_bs,
                               long long o_rs, long long o_bs, long long dq_rs, long long dq_bs, long long dk_rs,
                               long long dk_bs, long long dv_rs, long long dv_bs, long long dks_rs, long long dks_bs,
                               long long dvs_rs, long long dvs_bs, int q_off, int k_off, int s_off, int chunk,
                               int n_sum, int window, int tok_window, float scale, void* dks32, void* dvs32,
                               const void* q_doc_start, const void* k_doc_end, void* stream) {
  KSA_ENTER(q);
  using namespace ksa;
  KSA_REQUIRE(HD == 128, "attn_bwd_fused: head_dim %d unsupported (128 only)", HD);
  KSA_REQUIRE(Hq % Hkv == 0, "attn_bwd_fused: Hq %% Hkv != 0");
  KSA_REQUIRE(o_rs % 8 == 0 && dq_rs % 8 == 0 && dk_rs % 8 == 0 && dv_rs % 8 == 0,
              "attn_bwd_fused: row strides must be multiples of 8");
  KSA_REQUIRE(stats != nullptr && dq32 != nullptr, "attn_bwd_fused: the stats and dq32 workspaces are required");
  if (B == 0 || Lq == 0) return 0;
  const int lq_pad = ksa_attn_bwd_fused_lq_pad(Lq);
  CUtensorMap tq, tdo, tk, tv, tks, tvs;
  int rc;
  if ((rc = make_head_tmap_rows(&tq, q, Lq, Hq, B, q_rs, q_bs, 128))) return rc;
  if ((rc = make_head_tmap_rows(&tdo, d_o, Lq, Hq, B, o_rs, o_bs, 128))) return rc;
  if ((rc = make_head_tmap_rows(&tk, k, Lk, Hkv, B, k_rs, k_bs, 128))) return rc;
  if ((rc = make_head_tmap_rows(&tv, v, Lk, Hkv, B, v_rs, v_bs, 128))) return rc;
  if (Ns > 0) {
    if ((rc = make_head_tmap_rows(&tks, ks, Ns, Hkv, B, ks_rs, ks_bs, 128))) return rc;
    if ((rc = make_head_tmap_rows(&tvs, vs, Ns, Hkv, B, vs_rs, vs_bs, 128))) return rc;
  } else {
    tks = tk;
    tvs = tv;
  }
  FbParams p;
  p.s = AttnShape{B, Hq, Hkv, Lq, Lk, Ns, q_off, k_off, s_off, chunk, n_sum > 0 ? n_sum : 1, window, tok_window,
                  (const int*)q_doc_start, (const int*)k_doc_end};
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.stats = (const float*)stats;
  p.lq_pad = lq_pad;
  p.dq32 = (float*)dq32;
  p.dk = (bf16*)dk; p.dv = (bf16*)dv;
  p.dk_row_stride = dk_rs; p.dk_batch_stride = dk_bs; p.dv_row_stride = dv_rs; p.dv_batch_stride = dv_bs;
  p.dks = (bf16*)dks; p.dvs = (bf16*)dvs;
  p.dks_row_stride = dks_rs; p.dks_batch_stride = dks_bs; p.dvs_row_stride = dvs_rs; p.dvs_batch_stride = dvs_bs;
  p.dks32 = (float*)dks32; p.dvs32 = (float*)dvs32;
  p.n_seg = (Ns > 0 && dks32 != nullptr && dvs32 != nullptr) ? (((Lq + 127) / 128 + kFbSumSeg - 1) / kFbSumSeg) : 1;
  p.status = status_word();
  KSA_REQUIRE(p.status != nullptr, "could not allocate the status word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSmem::kTotal));
    attr = true;
  }
  {
    const long long warps = (long long)B * Hq * lq_pad;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    attn_bwd_prep_kernel<<<(unsigned)blocks, threads, 0, st>>>((const bf16*)o, (const bf16*)d_o, o_rs, o_bs,
                                                               (const float*)lse, (float*)stats, (float*)dq32, B, Hq,
                                                               Lq, lq_pad);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  CUtensorMap tdq;
  {
    uint64_t dims[4] = {128, (uint64_t)Hq, (uint64_t)Lq, (uint64_t)B};
    uint64_t str[4] = {4, 512, (uint64_t)Hq * 512, (uint64_t)Lq * Hq * 512};
    uint32_t box[4] = {32, 1, 32, 1};     // one warp's slab: 32 head dimensions x 32 query rows
    if ((rc = make_tmap(&tdq, dq32, 4, 4, dims, str, box, false))) return rc;
  }
  dim3 grid((Lk + 127) / 128 + ((Ns + 127) / 128) * p.n_seg, Hkv, B);
  attn_bwd_fused_kernel<<<grid, kFbThreads, FbSmem::kTotal, st>>>(tq, tdo, tk, tv, tks, tvs, tdq, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  {
    const long long n = (long long)B * Lq * Hq * 16;
    const int threads = 256;
    attn_bwd_dq_convert_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, st>>>(
        (const float*)dq32, (bf16*)dq, dq_rs, dq_bs, B, Lq, Hq, scale);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
}

// Backward of ksa_attn_fwd_cp: the fused key-stationary kernel on one shard of a context-parallel group.  Key tiles
// are read where they are (sources as in ksa_attn_fwd_cp).  dK / dV of this rank's own rows go to `dk` / `dv`
// ([B, local_rows, Hkv, 128]) and `dks` / `dvs` ([B, nsl, Hkv, 128]); dK / dV of the halo and of older summaries are
// ADDED, in fp32, into the owners' return blocks over NVLink (`ret_text`: [B, halo, 2*Hkv*128] of the previous rank,
// `ret_sum[s]`: [B, nsl, 2*Hkv*128] of rank s; row stride `ret_rs`), which the owners fold into their gradients
// (ksa_cp_fold_return).  `dks32` / `dvs32`: fp32 partial sums [B, n_sum_src*nsl, Hkv, 128] for this rank's own summary
// tiles when their query range is split (as in ksa_attn_bwd_fused), zeroed by the caller.
KSA_API int ksa_attn_bwd_fused_cp(const void* q, const void* o, const void* d_o, const void* lse, void* stats,
                                  void* dq32, void* dq, void* dk, void* dv, void* dks, void* dvs, int B, int Hq, int Hkv,
                                  int HD, int Lq, long long q_rs, long long q_bs, long long o_rs, long long o_bs,
                                  long long dq_rs, long long dq_bs, long long dk_rs, long long dk_bs, long long dv_rs,
                                  long long dv_bs, long long dks_rs, long long dks_bs, long long dvs_rs, long long dvs_bs,
                                  const void* const* text_src, int halo, int local_rows, const void* const* sum_src,
                                  int n_sum_src, int nsl, long long src_rs, long long text_bs, long long sum_bs,
                                  const void* const* text_flags, const void* const* sum_flags, unsigned flag_target,
                                  void* ret_text, void* const* ret_sum, long long ret_rs, long long ret_text_bs,
                                  long long ret_sum_bs, int q_off, int k_off, int chunk, int n_sum, int window,
                                  int tok_window, float scale, void* dks32, void* dvs32, void* stream) {
  KSA_ENTER(q);
  using namespace ksa;
  KSA_REQUIRE(HD == 128, "attn_bwd_fused_cp: head_dim %d unsupported (128 only)", HD);
  KSA_REQUIRE(Hq % Hkv == 0 && chunk > 0, "attn_bwd_fused_cp: bad head counts / chunk");
  KSA_REQUIRE(halo >= 0 && halo % 128 == 0, "attn_bwd_fused_cp: halo %d must be a multiple of 128", halo);
  KSA_REQUIRE(n_sum_src >= 0 && n_sum_src <= kCpMaxSum, "attn_bwd_fused_cp: %d summary sources (max %d)", n_sum_src, kCpMaxSum);
  KSA_REQUIRE(n_sum_src <= 1 || nsl % 128 == 0, "attn_bwd_fused_cp: %d summary rows per rank must be a multiple of 128", nsl);
  KSA_REQUIRE(o_rs % 8 == 0 && dq_rs % 8 == 0 && dk_rs % 8 == 0 && dv_rs % 8 == 0, "attn_bwd_fused_cp: row strides must be multiples of 8");
  KSA_REQUIRE(stats != nullptr && dq32 != nullptr, "attn_bwd_fused_cp: the stats and dq32 workspaces are required");
  KSA_REQUIRE(halo == 0 || ret_text != nullptr, "attn_bwd_fused_cp: a halo needs the return block of its owner");
  if (B == 0 || Lq == 0) return 0;
  const int lq_pad = ksa_attn_bwd_fused_lq_pad(Lq);
  const int Ns = n_sum_src * nsl;
  CUtensorMap tq, tdo, tdq;
  CpBwdSources cp;
  memset(&cp, 0, sizeof(cp));
  int rc;
  if ((rc = make_head_tmap_rows(&tq, q, Lq, Hq, B, q_rs, q_bs, 128))) return rc;
  if ((rc = make_head_tmap_rows(&tdo, d_o, Lq, Hq, B, o_rs, o_bs, 128))) return rc;
  const long long voff = (long long)Hkv * 128;
  for (int s = 0; s < 2; ++s) {
    const int rows = s == 0 ? halo : local_rows;
    const bf16* base = static_cast<const bf16*>(text_src[rows > 0 ? s : 1]);
    if ((rc = make_head_tmap_rows(&cp.src.kt[s], base, rows > 0 ? rows : 1, Hkv, B, src_rs, text_bs, 128))) return rc;
    if ((rc = make_head_tmap_rows(&cp.src.vt[s], base + voff, rows > 0 ? rows : 1, Hkv, B, src_rs, text_bs, 128))) return rc;
    cp.src.text_flag[s] = text_flags ? static_cast<const uint32_t*>(text_flags[s]) : nullptr;
  }
  for (int s = 0; s < kCpMaxSum; ++s) {
    const int src = s < n_sum_src ? s : (n_sum_src > 0 ? n_sum_src - 1 : -1);
    const bf16* base = src >= 0 ? static_cast<const bf16*>(sum_src[src]) : static_cast<const bf16*>(text_src[1]);
    if ((rc = make_head_tmap_rows(&cp.src.ks[s], base, nsl > 0 ? nsl : 1, Hkv, B, src_rs, sum_bs, 128))) return rc;
    if ((rc = make_head_tmap_rows(&cp.src.vs[s], base + voff, nsl > 0 ? nsl : 1, Hkv, B, src_rs, sum_bs, 128))) return rc;
    cp.src.sum_flag[s] = (sum_flags && s < n_sum_src) ? static_cast<const uint32_t*>(sum_flags[s]) : nullptr;
    cp.ret_sum[s] = (ret_sum && s < n_sum_src - 1) ? static_cast<float*>(ret_sum[s]) : nullptr;
    KSA_REQUIRE(s >= n_sum_src - 1 || cp.ret_sum[s] != nullptr, "attn_bwd_fused_cp: summary source %d has no return block", s);
  }
  cp.src.flag_target = flag_target;
  cp.src.halo = halo;
  cp.src.nsl = nsl > 0 ? nsl : 128;
  cp.n_sum_src = n_sum_src;
  cp.ret_text = static_cast<float*>(ret_text);
  cp.ret_rs = ret_rs; cp.ret_text_bs = ret_text_bs; cp.ret_sum_bs = ret_sum_bs;
  FbParams p;
  p.s = AttnShape{B, Hq, Hkv, Lq, halo + local_rows, Ns, q_off, k_off, 0, chunk, n_sum > 0 ? n_sum : 1, window, tok_window,
                  nullptr, nullptr};
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.stats = (const float*)stats;
  p.lq_pad = lq_pad;
  p.dq32 = (float*)dq32;
  // the kernel addresses key rows by their index in [halo | own rows] and [older summaries | own summaries]
  p.dk = (bf16*)dk - (long long)halo * dk_rs; p.dv = (bf16*)dv - (long long)halo * dv_rs;
  p.dk_row_stride = dk_rs; p.dk_batch_stride = dk_bs; p.dv_row_stride = dv_rs; p.dv_batch_stride = dv_bs;
  const long long own_sum0 = (long long)(n_sum_src > 0 ? n_sum_src - 1 : 0) * nsl;
  p.dks = dks ? (bf16*)dks - own_sum0 * dks_rs : nullptr; p.dvs = dvs ? (bf16*)dvs - own_sum0 * dvs_rs : nullptr;
  p.dks_row_stride = dks_rs; p.dks_batch_stride = dks_bs; p.dvs_row_stride = dvs_rs; p.dvs_batch_stride = dvs_bs;
  p.dks32 = (float*)dks32; p.dvs32 = (float*)dvs32;
  p.n_seg = (Ns > 0 && dks32 != nullptr && dvs32 != nullptr) ? (((Lq + 127) / 128 + kFbSumSeg - 1) / kFbSumSeg) : 1;
  p.status = status_word();
  KSA_REQUIRE(p.status != nullptr, "could not allocate the status word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(attn_bwd_fused_cp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSmem::kTotal));
    attr = true;
  }
  {
    const long long warps = (long long)B * Hq * lq_pad;
    const int threads = 256;
    attn_bwd_prep_kernel<<<(unsigned)((warps * 32 + threads - 1) / threads), threads, 0, st>>>(
        (const bf16*)o, (const bf16*)d_o, o_rs, o_bs, (const float*)lse, (float*)stats, (float*)dq32, B, Hq, Lq, lq_pad);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  {
    uint64_t dims[4] = {128, (uint64_t)Hq, (uint64_t)Lq, (uint64_t)B};
    uint64_t str[4] = {4, 512, (uint64_t)Hq * 512, (uint64_t)Lq * Hq * 512};
    uint32_t box[4] = {32, 1, 32, 1};     // one warp's slab: 32 head dimensions x 32 query rows
    if ((rc = make_tmap(&tdq, dq32, 4, 4, dims, str, box, false))) return rc;
  }
  dim3 grid((halo + local_rows + 127) / 128 + ((Ns + 127) / 128) * p.n_seg, Hkv, B);
  attn_bwd_fused_cp_kernel<<<grid, kFbThreads, FbSmem::kTotal, st>>>(tq, tdo, tdq, cp, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  {
    const long long n = (long long)B * Lq * Hq * 16;
    const int threads = 256;
    attn_bwd_dq_convert_kernel<<<(unsigned)((n + threads - 1) / threads), threads, 0, st>>>(
        (const float*)dq32, (bf16*)dq, dq_rs, dq_bs, B, Lq, Hq, scale);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
}
