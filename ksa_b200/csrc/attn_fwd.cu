// Forward attention for text queries on tcgen05 tensor cores: Kwai Summary
// Attention (sliding chunk window + old-chunk summaries), plain causal attention
// and token-sliding-window attention share this kernel.
//
// A work item is one tile of 128 query rows for TWO query heads of the same KV
// group ("slots"), so every K/V tile fetched by TMA feeds two S = Q K^T and two
// O += P V products and the two softmax warpgroups ping-pong against the tensor
// pipe.  Key tiles come from a closed-form range (attn_common.cuh): summary-key
// tiles first, then the text-key tiles of the window up to the diagonal.
// The grid is persistent: one CTA per SM walks the items (longest first) with
// barrier phases that run on across items, so the loads and the first S product
// of the next item overlap the epilogue of the current one.
//
//   warps 0-3   softmax + correction + epilogue for slot 0 (thread = query row)
//   warps 4-7   the same for slot 1
//   warp 8      TMA producer (Q once, then K_j / V_j through a 5-stage ring)
//   warp 9      MMA issuer (one elected thread);  warps 10-11 only give their registers away
// The three warpgroups re-divide the register file at entry (setmaxnreg): 224 registers per softmax thread, which
// holds a whole 128-column score row without spilling, 56 for the producer / issuer warpgroup.
//
// TMEM: S0 @0, S1 @128 (fp32 scores; P, packed bf16, overwrites S in place and is
// the A operand of the second product), O0 @256, O1 @256+HD.
//
// Bar: FlashAttentionForwardSm100 + block-sparse lists in the reference wheel
// (flash_attn/cute/flash_fwd_sm100.py:68 in the flash_attn_cute wheel, summary_attn/interface.py:77-82 in the
// summary_attn wheel).
#include "attn_common.cuh"
#include "host.h"
#include <string.h>

namespace ksa {

constexpr int kFwdThreads = 384;
constexpr int kKvStages = 5;
template <int HD>
struct FwdSmem {
  static constexpr int kTile = 128 * HD * 2;  // bytes of one 128-row tile
  static constexpr int kQ = 2 * kTile;
  static constexpr int kRing = kKvStages * kTile;
  static constexpr int kBar = 256;
  static constexpr int kTotal = kQ + kRing + kBar + 1024;
};

struct FwdParams {
  AttnShape s;
  float scale_log2;
  bf16* o;  // [B, Lq, Hq, HD]
  long long o_row_stride, o_batch_stride;
  float* lse;  // [B, Hq, Lq], natural log
  int nslot;   // query heads per CTA (2 when Hq/Hkv is even, else 1)
  int* status;
};

// Load a [128 x HD] tile (row = token) of head `h`, batch `b` starting at token `row0`.
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, int row0, int h, int b, uint64_t* bar) {
#pragma unroll
  for (int half = 0; half < HD / 64; ++half) tma_load_4d(dst + half * 16384, m, half * 64, row0, h, b, bar);
}

template <int HD, bool kCp>
__device__ __forceinline__ void attn_fwd_body(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                              const CUtensorMap& tmKs, const CUtensorMap& tmVs, const FwdParams& p,
                                              const CpSources* cps) {
  using S = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + S::kQ;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kQ + S::kRing);
  uint64_t* q_full = bars;                 // Q of the current work item has landed
  uint64_t* q_empty = bars + 1;            // every S product of the item has read Q
  uint64_t* kv_full = bars + 2;            // kKvStages
  uint64_t* kv_empty = kv_full + kKvStages;
  uint64_t* s_full = kv_empty + kKvStages;  // 2
  uint64_t* p_full = s_full + 2;            // 4: slot t, keys 0-63 and 64-127 of the tile
  uint64_t* o_full = p_full + 4;            // 2
  uint64_t* o_free = o_full + 2;            // 2: the epilogue has copied O of the finished item into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};
  const AttnShape& sh = p.s;

  // Work items: (query tile, head group, batch), late (long) query tiles first; CTA c takes items c, c + grid, ...
  const int n_qtiles = (sh.Lq + 127) / 128;
  const int heads_per_cta = p.nslot;
  const int n_groups = sh.Hq / heads_per_cta;
  const int per_q = n_groups * sh.B;
  const int n_items = n_qtiles * per_q;
  // round k hands CTA c item k * grid + c, odd rounds in reverse CTA order, which evens out the causal lengths
  auto item_of_round = [&](int k) {
    const int base = k * (int)gridDim.x;
    return base + ((k & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto decode = [&](int item, int& q_tile, int& head0, int& b) {
    const int qi = item / per_q, r = item - qi * per_q;
    q_tile = n_qtiles - 1 - qi;
    b = r / n_groups;
    head0 = (r - b * n_groups) * heads_per_cta;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < kKvStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[2 * i], 128);
      mbar_init(&p_full[2 * i + 1], 128);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_free[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 8) {
      // -------------------------------------------------------------- TMA producer
      if (lane == 0) {
        int n = 0, it = 0;
        bool ok = true;
        uint32_t waited = 0;   // context parallel: sources whose flag has been seen (bit s: text, bit 2 + s: summary)
        for (int k = 0; k < n_rounds && ok; ++k) {
          const int item = item_of_round(k);
          if (item >= n_items) continue;
          int q_tile, head0, b;
          decode(item, q_tile, head0, b);
          const int kv_head = head0 / (sh.Hq / sh.Hkv);
          const TileRange tr = key_tiles_for_query_tile(sh, q_tile, b);
          const int total = tr.total();
          // Q can only be replaced once the previous item's last S product has read it; the first K / V tiles of
          // this item do not have to wait for that, so they are requested first and cross the item boundary in flight
          bool q_loaded = false;
          auto load_q = [&]() {
            if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1, guard, kTimeoutStageEmpty)) return false;
            ++it;
            mbar_expect_tx(q_full, heads_per_cta * S::kTile);
            for (int t = 0; t < heads_per_cta; ++t)
              load_tile<HD>(sQ + t * S::kTile, &tmQ, q_tile * 128, head0 + t, b, q_full);
            q_loaded = true;
            return true;
          };
          if (it == 0 && !load_q()) break;
          for (int j = 0; j < total && ok; ++j) {
            if (!q_loaded && j == 2 && !load_q()) { ok = false; break; }
            const bool is_sum = j < tr.n_sum_tiles;
            const int kt = is_sum ? j : tr.text_first + (j - tr.n_sum_tiles);
            const CUtensorMap* mk = is_sum ? &tmKs : &tmK;
            const CUtensorMap* mv = is_sum ? &tmVs : &tmV;
            int row = kt * 128;
            if (kCp) {
              const int src = is_sum ? (kt * 128) / cps->nsl : (kt * 128 < cps->halo ? 0 : 1);
              row = is_sum ? (kt * 128) % cps->nsl : (src == 0 ? kt * 128 : kt * 128 - cps->halo);
              mk = is_sum ? &cps->ks[src] : &cps->kt[src];
              mv = is_sum ? &cps->vs[src] : &cps->vt[src];
              const uint32_t bit = 1u << (is_sum ? 2 + src : src);
              const uint32_t* flag = is_sum ? cps->sum_flag[src] : cps->text_flag[src];
              if (flag != nullptr && !(waited & bit)) {
                if (!flag_wait_ge(flag, cps->flag_target, p.status, kTimeoutPeerFlag, true)) {
                  *abort_flag = 1;
                  ok = false;
                  break;
                }
                waited |= bit;
              }
            }
            for (int kv = 0; kv < 2; ++kv, ++n) {
              const int stage = n % kKvStages;
              const uint32_t phase = (n / kKvStages) & 1;
              if (!mbar_wait(&kv_empty[stage], phase ^ 1, guard, kTimeoutStageEmpty)) { ok = false; break; }
              mbar_expect_tx(&kv_full[stage], S::kTile);
              load_tile<HD>(sKV + stage * S::kTile, kv == 0 ? mk : mv, row, kv_head, b, &kv_full[stage]);
            }
          }
          if (ok && !q_loaded && !load_q()) ok = false;
        }
      }
    } else if (warp == 9) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
        constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
        auto issue_s = [&](int t, int stage) {
          const uint32_t qa = smem_u32(sQ + t * S::kTile), ka = smem_u32(sKV + stage * S::kTile);
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
            umma_ss(tmem_base + t * 128, smem_desc_kmajor_sw128(qa + off), smem_desc_kmajor_sw128(ka + off), idesc_s,
                    kk != 0);
          }
          umma_commit(&s_full[t]);
        };
        int n0 = 0;    // ring slots used by earlier items
        int g = 0;     // key tiles of earlier items (phase of s_full / p_full / o_full)
        int it = 0, it_o = 0;   // items seen; items that produced an output tile
        bool ok = true;
        for (int k = 0; k < n_rounds && ok; ++k) {
          const int item = item_of_round(k);
          if (item >= n_items) continue;
          int q_tile, head0, b;
          decode(item, q_tile, head0, b);
          const int total = key_tiles_for_query_tile(sh, q_tile, b).total();
          ok = mbar_wait(q_full, it & 1, guard, kTimeoutTmaFull);
          if (ok && total > 0) {
            ok = mbar_wait(&kv_full[n0 % kKvStages], (n0 / kKvStages) & 1, guard, kTimeoutTmaFull);
            if (ok) {
              tc_fence_after();
              for (int t = 0; t < heads_per_cta; ++t) issue_s(t, n0 % kKvStages);
              umma_commit(&kv_empty[n0 % kKvStages]);
            }
          }
          for (int j = 0; j < total && ok; ++j) {
            const int nv = n0 + 2 * j + 1, nk = n0 + 2 * j + 2;
            const int st_v = nv % kKvStages, st_k = nk % kKvStages;
            if (!mbar_wait(&kv_full[st_v], (nv / kKvStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
            const bool more = (j + 1 < total);
            for (int t = 0; t < heads_per_cta && ok; ++t) {
              if (!mbar_wait(&p_full[2 * t], (g + j) & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
              // the first product of an item overwrites O: the previous item's epilogue must have read it
              if (j == 0 && it_o > 0 && !mbar_wait(&o_free[t], (it_o - 1) & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
              tc_fence_after();
              const uint32_t va = smem_u32(sKV + st_v * S::kTile);
#pragma unroll
              for (int kk = 0; kk < 8; ++kk) {
                if (kk == 4) {
                  if (!mbar_wait(&p_full[2 * t + 1], (g + j) & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
                  tc_fence_after();
                }
                umma_ts(tmem_base + 256 + t * HD, tmem_base + t * 128 + kk * 8,
                        smem_desc_mnmajor_sw128(va + kk * 2048, 16384), idesc_o, (j | kk) != 0);
              }
              if (!ok) break;
              umma_commit(&o_full[t]);
              if (more) {
                if (t == 0 && !mbar_wait(&kv_full[st_k], (nk / kKvStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
                tc_fence_after();
                issue_s(t, st_k);
              }
            }
            if (ok) {
              umma_commit(&kv_empty[st_v]);
              if (more) umma_commit(&kv_empty[st_k]);
            }
          }
          if (ok) umma_commit(q_empty);   // fires when the S products issued so far have read Q
          n0 += 2 * total;
          g += total;
          if (total > 0) ++it_o;
          ++it;
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int t = warp >> 2;  // slot
    if (t < heads_per_cta) {
      const int quad = warp & 3;
      const int r = quad * 32 + lane;               // row inside the tile
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t tS = tmem_base + lane_addr + t * 128;
      const uint32_t tO = tmem_base + lane_addr + 256 + t * HD;
      int g = 0;
      bool ok = true;
      for (int k = 0; k < n_rounds && ok; ++k) {
        const int item = item_of_round(k);
        if (item >= n_items) continue;
        int q_tile, head0, b;
        decode(item, q_tile, head0, b);
        const TileRange tr = key_tiles_for_query_tile(sh, q_tile, b);
        const int total = tr.total();
        const int q_local = q_tile * 128 + r;
        const int t_glob = sh.q_off + q_local;
        float m_run = -INFINITY, l_run = 0.f;
        const int doc_start = (sh.q_doc_start && q_local < sh.Lq) ? sh.q_doc_start[(long long)b * sh.Lq + q_local] : 0;
        for (int j = 0; j < total; ++j) {
          // what this row may see of the tile does not depend on the scores: worked out before they arrive
          const bool is_sum = j < tr.n_sum_tiles;
          const int kt = is_sum ? j : tr.text_first + (j - tr.n_sum_tiles);
          int lo, hi;
          allowed_columns(sh, t_glob, is_sum, kt, lo, hi, doc_start);
          const bool row_masked = lo > 0 || hi < 127;
          if (!mbar_wait(&s_full[t], (g + j) & 1, guard, kTimeoutAccFull)) { ok = false; break; }
          tc_fence_after();
          uint32_t sreg[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sreg[c]);
          tmem_wait_ld();
          if (row_masked) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = c * 32 + i;
                if (col < lo || col > hi) sreg[c][i] = 0xff800000u;  // -inf; its exponential is an exact 0
              }
          }
          float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              mx0 = max3(mx0, __uint_as_float(sreg[c][i]), __uint_as_float(sreg[c][i + 1]));
              mx1 = max3(mx1, __uint_as_float(sreg[c][i + 2]), __uint_as_float(sreg[c][i + 3]));
            }
          const float mx = fmaxf(mx0, mx1) * p.scale_log2;  // scale > 0
          const float m_new = fmaxf(m_run, mx);
          if (j == 0) {
            m_run = m_new;
          } else {
            const bool need = m_new > m_run + 8.f;
            if (__any_sync(0xffffffffu, need)) {
              if (!mbar_wait(&o_full[t], (g + j - 1) & 1, guard, kTimeoutAccFull)) { ok = false; break; }
              tc_fence_after();
              const float alpha = need ? fast_exp2(m_run - m_new) : 1.f;
#pragma unroll
              for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(tO + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st32(tO + c * 32, o);
              }
              tmem_wait_st();
              l_run *= alpha;
              if (need) m_run = m_new;
            }
          }
          const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
          const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(-m_use, -m_use);
          uint64_t acc0 = f2_pack(0.f, 0.f), acc1 = acc0;
          // P = 2^(S * scale - m) -> bf16 over the first half of the columns of S; the product P V starts on the
          // first 64 keys while the exponentials of the other 64 are still being computed
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float p0, p1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(sreg[c][2 * i]), __uint_as_float(sreg[c][2 * i + 1])), sc2, nm2),
                        p0, p1);
              p0 = fast_exp2(p0);
              p1 = fast_exp2(p1);
              if (i & 1) acc1 = f2_add(acc1, f2_pack(p0, p1)); else acc0 = f2_add(acc0, f2_pack(p0, p1));
              pk[i] = pack_bf16x2(p0, p1);
            }
            tmem_st16(tS + c * 16, pk);
            if (c & 1) {
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(&p_full[t * 2 + (c >> 1)]);
            }
          }
          float lsum, l1;
          f2_unpack(f2_add(acc0, acc1), lsum, l1);
          l_run += lsum + l1;
        }
        if (!ok) break;
        // epilogue: copy O into registers, hand the accumulator back, then O / l -> global and LSE
        const bool valid = q_local < sh.Lq;
        const int head = head0 + t;
        bf16* dst = p.o + (long long)b * p.o_batch_stride + (long long)q_local * p.o_row_stride + (long long)head * HD;
        if (total > 0) {
          if (!mbar_wait(&o_full[t], (g + total - 1) & 1, guard, kTimeoutAccFull)) { ok = false; break; }
          tc_fence_after();
          uint32_t o[HD / 32][32];
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) tmem_ld32(tO + c * 32, o[c]);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(&o_free[t]);
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          if (valid) {
#pragma unroll
            for (int c = 0; c < HD / 32; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(o[c][i]) * inv, __uint_as_float(o[c][i + 1]) * inv);
                v.y = pack_bf16x2(__uint_as_float(o[c][i + 2]) * inv, __uint_as_float(o[c][i + 3]) * inv);
                v.z = pack_bf16x2(__uint_as_float(o[c][i + 4]) * inv, __uint_as_float(o[c][i + 5]) * inv);
                v.w = pack_bf16x2(__uint_as_float(o[c][i + 6]) * inv, __uint_as_float(o[c][i + 7]) * inv);
                *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
              }
          }
        } else if (valid) {
#pragma unroll
          for (int i = 0; i < HD; i += 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
        }
        if (valid && p.lse)
          p.lse[((long long)b * sh.Hq + head) * sh.Lq + q_local] =
              (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
        g += total;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmKs,
                const __grid_constant__ CUtensorMap tmVs, FwdParams p) {
  attn_fwd_body<HD, false>(tmQ, tmK, tmV, tmKs, tmVs, p, nullptr);
}

// The same kernel for one shard of a context-parallel group: keys and values come from the sources in `cps`.
template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_cp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CpSources cps, FwdParams p) {
  attn_fwd_body<HD, true>(tmQ, cps.kt[1], cps.vt[1], cps.ks[0], cps.vs[0], p, &cps);
}

// [B, T, H, HD] view -> 4-D tensor map {HD, T, H, B}, box {64, 128, 1, 1}, 128-byte swizzle.
static int make_head_tmap(CUtensorMap* m, const void* base, int HD, long long T, int H, int B, long long row_stride,
                          long long batch_stride) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)(T > 0 ? T : 1), (uint64_t)H, (uint64_t)B};
  uint64_t str[4] = {2, (uint64_t)row_stride * 2, (uint64_t)HD * 2, (uint64_t)batch_stride * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap(m, base, 2, 4, dims, str, box, true);
}

static int sm_count() {
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  }
  return num_sms;
}

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tks,
                      const CUtensorMap& tvs, const FwdParams& p, cudaStream_t st) {
  auto kern = attn_fwd_kernel<HD>;
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<HD>::kTotal));
    attr = true;
  }
  const int items = ((p.s.Lq + 127) / 128) * (p.s.Hq / p.nslot) * p.s.B;
  int sms = sm_count();
  if (sms <= 0) return 1;
  dim3 grid(items < sms ? items : sms);
  kern<<<grid, kFwdThreads, FwdSmem<HD>::kTotal, st>>>(tq, tk, tv, tks, tvs, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

template <int HD>
static int launch_fwd_cp(const CUtensorMap& tq, const CpSources& cps, const FwdParams& p, cudaStream_t st) {
  auto kern = attn_fwd_cp_kernel<HD>;
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<HD>::kTotal));
    attr = true;
  }
  const int items = ((p.s.Lq + 127) / 128) * (p.s.Hq / p.nslot) * p.s.B;
  int sms = sm_count();
  if (sms <= 0) return 1;
  dim3 grid(items < sms ? items : sms);
  kern<<<grid, kFwdThreads, FwdSmem<HD>::kTotal, st>>>(tq, cps, p);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace ksa

// Text-query attention forward of ONE SHARD of a context-parallel group, reading keys and values where they are.
// q, o, lse: this rank's queries and outputs as in ksa_attn_fwd.  Keys / values: `text_src[0]` = first halo row in the
// previous rank's exchange slot (ignored when halo = 0), `text_src[1]` = this rank's own text rows, `sum_src[s]` =
// the summary rows of rank s (s < n_sum_src - 1: peers; the last one: this rank); every source is a [B, rows, 2*Hkv*HD]
// block, K in the first Hkv*HD columns and V in the rest, row stride `src_rs`, batch strides `text_bs` / `sum_bs`
// (elements).  `halo` and `nsl` (summary rows per rank) must be multiples of 128 unless there is no halo / a single
// summary source.  `text_flags[s]` / `sum_flags[s]`: address of a flag in this rank's memory that the owner of the
// source raises to `flag_target` when its slot is filled, or null for sources that need no wait.
// Peer memory is only ever read with TMA loads issued by this kernel's own CTAs (no multicast).
KSA_API int ksa_attn_fwd_cp(const void* q, void* o, void* lse, int B, int Hq, int Hkv, int HD, int Lq, long long q_rs,
                            long long q_bs, long long o_rs, long long o_bs, const void* const* text_src, int halo,
                            int local_rows, const void* const* sum_src, int n_sum_src, int nsl, long long src_rs,
                            long long text_bs, long long sum_bs, const void* const* text_flags,
                            const void* const* sum_flags, unsigned flag_target, int q_off, int k_off, int chunk,
                            int n_sum, int window, int tok_window, float scale, void* stream) {
  KSA_ENTER(q);
  using namespace ksa;
  KSA_REQUIRE(HD == 128 || HD == 64, "attn_fwd_cp: head_dim %d unsupported (64 or 128)", HD);
  KSA_REQUIRE(Hq % Hkv == 0 && chunk > 0, "attn_fwd_cp: bad head counts / chunk");
  KSA_REQUIRE(halo >= 0 && halo % 128 == 0, "attn_fwd_cp: halo %d must be a multiple of 128", halo);
  KSA_REQUIRE(n_sum_src >= 0 && n_sum_src <= kCpMaxSum, "attn_fwd_cp: %d summary sources (max %d)", n_sum_src, kCpMaxSum);
  KSA_REQUIRE(n_sum_src <= 1 || nsl % 128 == 0, "attn_fwd_cp: %d summary rows per rank must be a multiple of 128", nsl);
  KSA_REQUIRE(o_rs % 8 == 0, "attn_fwd_cp: output row stride must be a multiple of 8");
  if (B == 0 || Lq == 0) return 0;
  CUtensorMap tq;
  CpSources cps;
  memset(&cps, 0, sizeof(cps));
  int rc;
  if ((rc = make_head_tmap(&tq, q, HD, Lq, Hq, B, q_rs, q_bs))) return rc;
  const long long voff = (long long)Hkv * HD;
  for (int s = 0; s < 2; ++s) {
    const int rows = s == 0 ? halo : local_rows;
    const bf16* base = static_cast<const bf16*>(text_src[rows > 0 ? s : 1]);
    if ((rc = make_head_tmap(&cps.kt[s], base, HD, rows > 0 ? rows : 1, Hkv, B, src_rs, text_bs))) return rc;
    if ((rc = make_head_tmap(&cps.vt[s], base + voff, HD, rows > 0 ? rows : 1, Hkv, B, src_rs, text_bs))) return rc;
    cps.text_flag[s] = text_flags ? static_cast<const uint32_t*>(text_flags[s]) : nullptr;
  }
  for (int s = 0; s < kCpMaxSum; ++s) {
    const int src = s < n_sum_src ? s : (n_sum_src > 0 ? n_sum_src - 1 : -1);
    const bf16* base = src >= 0 ? static_cast<const bf16*>(sum_src[src]) : static_cast<const bf16*>(text_src[1]);
    if ((rc = make_head_tmap(&cps.ks[s], base, HD, nsl > 0 ? nsl : 1, Hkv, B, src_rs, sum_bs))) return rc;
    if ((rc = make_head_tmap(&cps.vs[s], base + voff, HD, nsl > 0 ? nsl : 1, Hkv, B, src_rs, sum_bs))) return rc;
    cps.sum_flag[s] = (sum_flags && s < n_sum_src) ? static_cast<const uint32_t*>(sum_flags[s]) : nullptr;
  }
  cps.flag_target = flag_target;
  cps.halo = halo;
  cps.nsl = nsl > 0 ? nsl : 128;
  FwdParams p;
  p.s = AttnShape{B, Hq, Hkv, Lq, halo + local_rows, n_sum_src * nsl, q_off, k_off, 0, chunk, n_sum > 0 ? n_sum : 1,
                  window, tok_window, nullptr, nullptr};
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = (bf16*)o;
  p.o_row_stride = o_rs;
  p.o_batch_stride = o_bs;
  p.lse = (float*)lse;
  p.nslot = ((Hq / Hkv) % 2 == 0) ? 2 : 1;
  p.status = status_word();
  KSA_REQUIRE(p.status != nullptr, "could not allocate the status word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return HD == 128 ? launch_fwd_cp<128>(tq, cps, p, st) : launch_fwd_cp<64>(tq, cps, p, st);
}

// Text-query attention forward.  All tensors are bf16 with the head dimension contiguous:
//   q  [B, Lq, Hq, HD]   (row stride q_rs elements, batch stride q_bs)
//   k,v  [B, Lk, Hkv, HD]  text keys;   ks,vs [B, Ns, Hkv, HD] summary keys (Ns may be 0)
//   o  [B, Lq, Hq, HD];  lse [B, Hq, Lq] fp32 (natural log) or null
// window >= 2^29 disables the chunk window (plain causal); tok_window > 0 adds a token sliding window.
// q_doc_start / k_doc_end (int32 [B, Lq] / [B, Lk], both or neither): packed documents, see AttnShape.
KSA_API int ksa_attn_fwd(const void* q, const void* k, const void* v, const void* ks, const void* vs, void* o,
                         void* lse, int B, int Hq, int Hkv, int HD, int Lq, int Lk, int Ns, long long q_rs,
                         long long q_bs, long long k_rs, long long k_bs, long long v_rs, long long v_bs,
                         long long ks_rs, long long ks_bs, long long vs_rs, long long vs_bs, long long o_rs,
                         long long o_bs, int q_off, int k_off, int s_off, int chunk, int n_sum, int window,
                         int tok_window, float scale, const void* q_doc_start, const void* k_doc_end, void* stream) {
  KSA_ENTER(q);
  using namespace ksa;
  KSA_REQUIRE(HD == 128 || HD == 64, "attn_fwd: head_dim %d unsupported (64 or 128)", HD);
  KSA_REQUIRE(Hq % Hkv == 0, "attn_fwd: Hq %% Hkv != 0");
  KSA_REQUIRE(chunk > 0 && n_sum >= 0, "attn_fwd: bad chunk/n_sum");
  KSA_REQUIRE(o_rs % 8 == 0, "attn_fwd: output row stride must be a multiple of 8");
  if (B == 0 || Lq == 0) return 0;
  CUtensorMap tq, tk, tv, tks, tvs;
  int rc;
  if ((rc = make_head_tmap(&tq, q, HD, Lq, Hq, B, q_rs, q_bs))) return rc;
  if ((rc = make_head_tmap(&tk, k, HD, Lk, Hkv, B, k_rs, k_bs))) return rc;
  if ((rc = make_head_tmap(&tv, v, HD, Lk, Hkv, B, v_rs, v_bs))) return rc;
  if (Ns > 0) {
    if ((rc = make_head_tmap(&tks, ks, HD, Ns, Hkv, B, ks_rs, ks_bs))) return rc;
    if ((rc = make_head_tmap(&tvs, vs, HD, Ns, Hkv, B, vs_rs, vs_bs))) return rc;
  } else {
    tks = tk;
    tvs = tv;
  }
  FwdParams p;
  p.s = AttnShape{B, Hq, Hkv, Lq, Lk, Ns, q_off, k_off, s_off, chunk, n_sum > 0 ? n_sum : 1, window, tok_window,
                  (const int*)q_doc_start, (const int*)k_doc_end};
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = (bf16*)o;
  p.o_row_stride = o_rs;
  p.o_batch_stride = o_bs;
  p.lse = (float*)lse;
  p.nslot = ((Hq / Hkv) % 2 == 0) ? 2 : 1;
  p.status = status_word();
  KSA_REQUIRE(p.status != nullptr, "could not allocate the status word");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return HD == 128 ? launch_fwd<128>(tq, tk, tv, tks, tvs, p, st) : launch_fwd<64>(tq, tk, tv, tks, tvs, p, st);
}
