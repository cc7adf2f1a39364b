// Forward attention for text queries on tcgen05 tensor cores: Kwai Summary
// Attention (sliding chunk window + old-chunk summaries), plain causal attention
// and token-sliding-window attention share this kernel.
//
// One CTA owns one tile of 128 query rows for TWO query heads of the same KV
// group ("slots"), so every K/V tile fetched by TMA feeds two S = Q K^T and two
// O += P V products and the two softmax warpgroups ping-pong against the tensor
// pipe.  Key tiles come from a closed-form range (attn_common.cuh): summary-key
// tiles first, then the text-key tiles of the window up to the diagonal.
//
//   warp 0      TMA producer (Q once, then K_j / V_j through a 4-stage ring)
//   warp 1      MMA issuer (one elected thread)
//   warps 2-5   softmax + correction + epilogue for slot 0 (thread = query row)
//   warps 6-9   the same for slot 1
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

constexpr int kFwdThreads = 320;
constexpr int kKvStages = 4;

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
  uint64_t* q_full = bars;                 // 1
  uint64_t* kv_full = bars + 1;            // kKvStages
  uint64_t* kv_empty = kv_full + kKvStages;
  uint64_t* s_full = kv_empty + kKvStages;  // 2
  uint64_t* p_full = s_full + 2;            // 2
  uint64_t* o_full = p_full + 2;            // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitGuard guard{abort_flag, p.status};
  const AttnShape& sh = p.s;

  const int n_qtiles = (sh.Lq + 127) / 128;
  const int q_tile = n_qtiles - 1 - (int)blockIdx.x;  // heavy (late) tiles first
  const int heads_per_cta = p.nslot;
  const int head0 = blockIdx.y * heads_per_cta;
  const int kv_head = head0 / (sh.Hq / sh.Hkv);
  const int b = blockIdx.z;
  const TileRange tr = key_tiles_for_query_tile(sh, q_tile, b);
  const int total = tr.total();

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kKvStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128); mbar_init(&o_full[i], 1); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 2) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, heads_per_cta * S::kTile);
      for (int t = 0; t < heads_per_cta; ++t) load_tile<HD>(sQ + t * S::kTile, &tmQ, q_tile * 128, head0 + t, b, q_full);
      int n = 0;
      bool ok = true;
      uint32_t waited = 0;     // context parallel: sources whose flag has been seen (bit s: text, bit 2 + s: summary)
      for (int j = 0; j < total && ok; ++j) {
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
            if (!flag_wait_ge(flag, cps->flag_target, p.status, kTimeoutPeerFlag, true)) { *abort_flag = 1; ok = false; break; }
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
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
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
      bool ok = mbar_wait(q_full, 0, guard, kTimeoutTmaFull);
      if (ok) ok = mbar_wait(&kv_full[0], 0, guard, kTimeoutTmaFull);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < heads_per_cta; ++t) issue_s(t, 0);
        umma_commit(&kv_empty[0]);
      }
      for (int j = 0; j < total && ok; ++j) {
        const int nv = 2 * j + 1, nk = 2 * j + 2;
        const int st_v = nv % kKvStages, st_k = nk % kKvStages;
        if (!mbar_wait(&kv_full[st_v], (nv / kKvStages) & 1, guard, kTimeoutTmaFull)) { ok = false; break; }
        const bool more = (j + 1 < total);
        for (int t = 0; t < heads_per_cta && ok; ++t) {
          if (!mbar_wait(&p_full[t], j & 1, guard, kTimeoutSoftmax)) { ok = false; break; }
          tc_fence_after();
          const uint32_t va = smem_u32(sKV + st_v * S::kTile);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            umma_ts(tmem_base + 256 + t * HD, tmem_base + t * 128 + kk * 8,
                    smem_desc_mnmajor_sw128(va + kk * 2048, 16384), idesc_o, (j | kk) != 0);
          }
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
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int t = (warp - 2) >> 2;  // slot
    if (t < heads_per_cta) {
      const int quad = warp & 3;
      const int r = quad * 32 + lane;               // row inside the tile
      const int q_local = q_tile * 128 + r;
      const int t_glob = sh.q_off + q_local;
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t tS = tmem_base + lane_addr + t * 128;
      const uint32_t tO = tmem_base + lane_addr + 256 + t * HD;
      float m_run = -INFINITY, l_run = 0.f;
      const int doc_start = (sh.q_doc_start && q_local < sh.Lq) ? sh.q_doc_start[(long long)b * sh.Lq + q_local] : 0;
      bool ok = true;
      for (int j = 0; j < total; ++j) {
        if (!mbar_wait(&s_full[t], j & 1, guard, kTimeoutAccFull)) { ok = false; break; }
        tc_fence_after();
        uint32_t sreg[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, sreg[c]);
        tmem_wait_ld();
        const bool is_sum = j < tr.n_sum_tiles;
        const int kt = is_sum ? j : tr.text_first + (j - tr.n_sum_tiles);
        int lo, hi;
        allowed_columns(sh, t_glob, is_sum, kt, lo, hi, doc_start);
        float mx = -INFINITY;
        if (lo > 0 || hi < 127) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = c * 32 + i;
              float v = (col >= lo && col <= hi) ? __uint_as_float(sreg[c][i]) : -INFINITY;
              sreg[c][i] = __float_as_uint(v);
              mx = fmaxf(mx, v);
            }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sreg[c][i]));
        }
        mx *= p.scale_log2;  // scale > 0
        const float m_new = fmaxf(m_run, mx);
        if (j == 0) {
          m_run = m_new;
        } else {
          const bool need = m_new > m_run + 8.f;
          if (__any_sync(0xffffffffu, need)) {
            if (!mbar_wait(&o_full[t], (j - 1) & 1, guard, kTimeoutAccFull)) { ok = false; break; }
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
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sreg[c][2 * i]), p.scale_log2, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sreg[c][2 * i + 1]), p.scale_log2, -m_use));
            lsum += p0 + p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st16(tS + c * 16, pk);
        }
        l_run += lsum;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
      }
      // epilogue: O / l  -> global, LSE
      if (ok && total > 0) ok = mbar_wait(&o_full[t], (total - 1) & 1, guard, kTimeoutAccFull);
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const int head = head0 + t;
        const bool valid = q_local < sh.Lq;
        bf16* dst = p.o + (long long)b * p.o_batch_stride + (long long)q_local * p.o_row_stride + (long long)head * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
            }
          }
        }
        if (valid && p.lse)
          p.lse[((long long)b * sh.Hq + head) * sh.Lq + q_local] =
              (l_run > 0.f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
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

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tks,
                      const CUtensorMap& tvs, const FwdParams& p, cudaStream_t st) {
  auto kern = attn_fwd_kernel<HD>;
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<HD>::kTotal));
    attr = true;
  }
  dim3 grid((p.s.Lq + 127) / 128, p.s.Hq / p.nslot, p.s.B);
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
  dim3 grid((p.s.Lq + 127) / 128, p.s.Hq / p.nslot, p.s.B);
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
