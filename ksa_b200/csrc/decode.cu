// Decode-time attention over the contiguous ring-buffer KV cache, and the cache update kernels.
//
// A decode step has 1 query token per sequence (or 1 + S at a chunk boundary: the last text token of the chunk and
// its S summary tokens).  Every query attends ONE contiguous slice [start, start + len) of its sequence's cache
// (layout [scratch | current chunk | sliding-chunk ring | summaries | headroom], keys cached after RoPE, so physical
// order does not matter and no mask is needed inside the slice).  The work is bound by reading K and V once:
//   * grid (splits, KV heads, batch): a CTA stages 64-key tiles of K and V in shared memory with coalesced 16-byte
//     loads (rows padded by one word -> conflict-free "thread = key" reads) and serves all G * Tq queries that share
//     the KV head from the same tile (GQA heads are never re-read or materialised);
//   * partial (max, sum, out) per split go to a scratch buffer; a second kernel merges the splits.
// Slices, slot indices and enable flags are device tensors, so one captured launch serves every step.
//
// Replaces SDPA over a repeat_kv-expanded slice plus copy_ ops in the reference's HF model
// (examples/pretrain/hf_template/modeling_qwen3sa.py:306-434, :591-612, :816-876).
#include "common.cuh"
#include "host.h"

namespace ksa {

constexpr int kDecThreads = 128;
constexpr int kDecTile = 64;       // keys per shared-memory tile
constexpr int kDecMaxQ = 16;       // queries (G * Tq) served per CTA
constexpr int kDecMaxSplits = 64;  // splits of the key range when the last split merges them itself

struct DecodeArgs {
  const bf16* q;        // [B, Tq, Hq, D]
  const bf16* k_cache;  // [B, Hkv, cap, D]
  const bf16* v_cache;
  const int* start;     // [B, Tq]
  const int* len;       // [B, Tq]
  float* part_o;        // [B, Tq, Hq, splits, D]
  float* part_ml;       // [B, Tq, Hq, splits, 2]
  bf16* out;            // [B, Tq, Hq, D]
  int B, Tq, Hq, Hkv, D, cap, splits, keys_per_split;
  float scale;
  int* counters;        // [B * Hkv] zeros, or null: with counters the last split of a KV group to finish merges the
                        // splits itself (and puts the counter back to zero); without, decode_combine_kernel does
};

// Called by every thread of a CTA after it has written its split's partial results.  The CTA that finishes last for
// its (batch, KV head) merges all splits of the group's nq = G * Tq queries into `out`.
__device__ __forceinline__ void combine_if_last(const DecodeArgs& a, int b, int kvh, int nq, int G) {
  if (a.counters == nullptr) return;
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&a.counters[b * a.Hkv + kvh], 1);
    s_last = prev == a.splits - 1;
    if (s_last) a.counters[b * a.Hkv + kvh] = 0;      // ready for the next launch on this stream
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // weights of the splits: stage (max, sum) of every (query, split), then one thread per query turns them into
  // exp(m_split - m) / l; the outputs are then plain weighted sums with independent loads
  __shared__ float s_w[kDecMaxQ][kDecMaxSplits], s_ls[kDecMaxQ][kDecMaxSplits];
  const int D = a.D, S = a.splits;
  for (int i = threadIdx.x; i < nq * S; i += blockDim.x) {
    const int q = i / S, sp = i - q * S;
    const long long row = ((long long)b * a.Tq + q / G) * a.Hq + kvh * G + q % G;
    s_w[q][sp] = __ldcg(a.part_ml + (row * S + sp) * 2);
    s_ls[q][sp] = __ldcg(a.part_ml + (row * S + sp) * 2 + 1);
  }
  __syncthreads();
  if (threadIdx.x < nq) {
    const int q = threadIdx.x;
    float m = -INFINITY, l = 0.f;
    for (int sp = 0; sp < S; ++sp) m = fmaxf(m, s_w[q][sp]);
    for (int sp = 0; sp < S; ++sp) {
      const float f = s_w[q][sp] == -INFINITY ? 0.f : __expf(s_w[q][sp] - m);
      s_w[q][sp] = f;
      l += s_ls[q][sp] * f;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int sp = 0; sp < S; ++sp) s_w[q][sp] *= inv;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nq * D; i += blockDim.x) {
    const int q = i / D, d = i - q * D;
    const long long row = ((long long)b * a.Tq + q / G) * a.Hq + kvh * G + q % G;
    const float* po = a.part_o + row * S * D + d;
    float o = 0.f;
    int sp = 0;
    for (; sp + 8 <= S; sp += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + (long long)(sp + u) * D);
#pragma unroll
      for (int u = 0; u < 8; ++u) o = fmaf(v[u], s_w[q][sp + u], o);
    }
    for (; sp < S; ++sp) o = fmaf(__ldcg(po + (long long)sp * D), s_w[q][sp], o);
    a.out[row * D + d] = __float2bfloat16(o);
  }
}

template <int D>
__global__ void __launch_bounds__(kDecThreads) decode_attn_kernel(DecodeArgs a) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  constexpr int ROW_W = D / 2 + 1;  // 32-bit words per padded row
  __shared__ uint32_t k_s[kDecTile * ROW_W];
  __shared__ uint32_t v_s[kDecTile * ROW_W];
  __shared__ float q_s[kDecMaxQ * D];
  __shared__ float p_s[kDecMaxQ * kDecTile];
  __shared__ float m_s[kDecMaxQ], l_s[kDecMaxQ], corr_s[kDecMaxQ];
  __shared__ int s_start[kDecMaxQ], s_end[kDecMaxQ];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int nq = G * a.Tq;  // query index qi = t * G + g
  const int tid = threadIdx.x;
  for (int i = tid; i < nq * D; i += kDecThreads) {
    const int qi = i / D, d = i % D, t = qi / G, g = qi % G;
    q_s[i] = __bfloat162float(a.q[(((long long)b * a.Tq + t) * a.Hq + kvh * G + g) * D + d]) * a.scale;
  }
  if (tid < nq) {
    const int t = tid / G;
    const int st = a.start[b * a.Tq + t];
    s_start[tid] = st;
    s_end[tid] = st + a.len[b * a.Tq + t];
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  __syncthreads();
  int lo = a.cap, hi = 0;
  for (int qi = 0; qi < nq; ++qi) { lo = min(lo, s_start[qi]); hi = max(hi, s_end[qi]); }
  const int k0 = lo + split * a.keys_per_split;
  const int k1 = min(hi, k0 + a.keys_per_split);
  // output accumulators: thread owns dims d = tid, tid + 128, ... for every query
  constexpr int DPT = (D + kDecThreads - 1) / kDecThreads;
  float acc[kDecMaxQ][DPT];
#pragma unroll
  for (int qi = 0; qi < kDecMaxQ; ++qi)
#pragma unroll
    for (int j = 0; j < DPT; ++j) acc[qi][j] = 0.f;
  const bf16* kb = a.k_cache + ((long long)b * a.Hkv + kvh) * a.cap * D;
  const bf16* vb = a.v_cache + ((long long)b * a.Hkv + kvh) * a.cap * D;
  for (int kt = k0; kt < k1; kt += kDecTile) {
    const int nkeys = min(kDecTile, k1 - kt);
    __syncthreads();
    for (int i = tid; i < nkeys * (D / 8); i += kDecThreads) {
      const int r = i / (D / 8), v = i % (D / 8);
      const uint4 ku = *reinterpret_cast<const uint4*>(kb + (long long)(kt + r) * D + v * 8);
      const uint4 vu = *reinterpret_cast<const uint4*>(vb + (long long)(kt + r) * D + v * 8);
      uint32_t* kd = k_s + r * ROW_W + v * 4;
      uint32_t* vd = v_s + r * ROW_W + v * 4;
      kd[0] = ku.x; kd[1] = ku.y; kd[2] = ku.z; kd[3] = ku.w;
      vd[0] = vu.x; vd[1] = vu.y; vd[2] = vu.z; vd[3] = vu.w;
    }
    __syncthreads();
    // scores: thread -> (key = tid % 64, queries qi = tid / 64, +2, ...)
    {
      const int r = tid % kDecTile;
      for (int qi = tid / kDecTile; qi < nq; qi += kDecThreads / kDecTile) {
        float s = -INFINITY;
        const int key = kt + r;
        if (r < nkeys && key >= s_start[qi] && key < s_end[qi]) {
          s = 0.f;
          const uint32_t* row = k_s + r * ROW_W;
          const float* qv = q_s + qi * D;
#pragma unroll 8
          for (int w = 0; w < D / 2; ++w) {
            const float2 f = unpack_bf16x2(row[w]);
            s += qv[2 * w] * f.x + qv[2 * w + 1] * f.y;
          }
        }
        p_s[qi * kDecTile + r] = s;
      }
    }
    __syncthreads();
    // online softmax state per query: one warp per query (strided)
    for (int qi = tid >> 5; qi < nq; qi += kDecThreads >> 5) {
      const int lane = tid & 31;
      const float s0 = p_s[qi * kDecTile + lane], s1 = p_s[qi * kDecTile + lane + 32];
      const float mx = warp_max(fmaxf(s0, s1));
      const float m_old = m_s[qi];
      const float m_new = fmaxf(m_old, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float p0 = __expf(s0 - m_use), p1 = __expf(s1 - m_use);
      p_s[qi * kDecTile + lane] = p0;
      p_s[qi * kDecTile + lane + 32] = p1;
      const float sum = warp_sum(p0 + p1);
      if (lane == 0) {
        const float c = m_old == -INFINITY ? 0.f : __expf(m_old - m_use);
        corr_s[qi] = c;
        l_s[qi] = l_s[qi] * c + sum;
        m_s[qi] = m_new;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < DPT; ++j) {
      const int d = tid + j * kDecThreads;
      if (d < D) {
        const bf16* vcol = reinterpret_cast<const bf16*>(v_s) + d;
#pragma unroll
        for (int qi = 0; qi < kDecMaxQ; ++qi) {
          if (qi < nq) {
            float o = acc[qi][j] * corr_s[qi];
            const float* pr = p_s + qi * kDecTile;
            for (int r = 0; r < nkeys; ++r) o += pr[r] * __bfloat162float(vcol[r * ROW_W * 2]);
            acc[qi][j] = o;
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int qi = 0; qi < kDecMaxQ; ++qi) {
    if (qi < nq) {
      const int t = qi / G, g = qi % G;
      const long long base = ((((long long)b * a.Tq + t) * a.Hq + kvh * G + g) * a.splits + split);
#pragma unroll
      for (int j = 0; j < DPT; ++j) {
        const int d = tid + j * kDecThreads;
        if (d < D) a.part_o[base * D + d] = acc[qi][j];
      }
      if (tid == 0) {
        a.part_ml[base * 2] = m_s[qi];
        a.part_ml[base * 2 + 1] = l_s[qi];
      }
    }
  }
  combine_if_last(a, b, kvh, nq, G);
}

// ------------------------------------------------------------------------------------------ tensor-core variant
// Same interface and the same split / combine scheme, but a key is read from global memory exactly once and never
// staged in shared memory.  Scores: warp-level mma.sync m16n8k16 with the (up to 16) queries of the KV group as the
// 16-row operand and 8 keys as the 8-column operand; a lane loads 16 contiguous bytes of a key (and of a query) and
// hands them to two MMAs as k slots {2t, 2t+1, 2t+8, 2t+9}, a permutation of the head dimension that is the same on
// both sides.  Probabilities go through a 1 KB per-warp shared buffer so that the P.V product runs with
// "lane = 4 head dimensions" (V rows are read as 8 bytes per lane, coalesced) on the FMA units.
__device__ __forceinline__ void mma_qk(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NQ>   // queries served per CTA, padded: 4, 8 or 16
__global__ void __launch_bounds__(kDecThreads) decode_attn_mma_kernel(DecodeArgs a) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  constexpr int D = 128, KPI = 16;                 // keys per warp iteration
  __shared__ __align__(16) float s_p[4][KPI][NQ];  // per warp: probabilities, [key][query]
  __shared__ float s_m[4][NQ], s_l[4][NQ];
  __shared__ __align__(16) float s_o[4][NQ][D];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int nq = G * a.Tq;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // per-row (g and g+8) slice bounds, and the CTA's key range
  int st0 = 0, en0 = 0, st1 = 0, en1 = 0, lo = a.cap, hi = 0;
  for (int qi = 0; qi < nq; ++qi) {
    const int s = a.start[b * a.Tq + qi / G], e = s + a.len[b * a.Tq + qi / G];
    lo = min(lo, s); hi = max(hi, e);
    if (qi == g) { st0 = s; en0 = e; }
    if (qi == g + 8) { st1 = s; en1 = e; }
  }
  const int k0 = lo + split * a.keys_per_split;
  const int k1 = min(hi, k0 + a.keys_per_split);
  // query fragments: row g and row g+8, 4 blocks of 32 head dimensions
  uint4 qa[4], qb[4];
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    qa[blk] = make_uint4(0, 0, 0, 0);
    qb[blk] = make_uint4(0, 0, 0, 0);
    if (g < nq) {
      const int tq = g / G, gg = g % G;
      qa[blk] = *reinterpret_cast<const uint4*>(a.q + (((long long)b * a.Tq + tq) * a.Hq + kvh * G + gg) * D + blk * 32 + t * 8);
    }
    if (NQ > 8 && g + 8 < nq) {
      const int tq = (g + 8) / G, gg = (g + 8) % G;
      qb[blk] = *reinterpret_cast<const uint4*>(a.q + (((long long)b * a.Tq + tq) * a.Hq + kvh * G + gg) * D + blk * 32 + t * 8);
    }
  }
  const bf16* kb = a.k_cache + ((long long)b * a.Hkv + kvh) * a.cap * D;
  const bf16* vb = a.v_cache + ((long long)b * a.Hkv + kvh) * a.cap * D;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max / partial sums of rows g and g+8
  float acc[NQ][4];
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[q][i] = 0.f;
  const float sc = a.scale * 1.4426950408889634f;              // scores in log2 units

  for (int kbase = k0 + warp * KPI; kbase < k1; kbase += 4 * KPI) {
    // ---- scores of 16 keys
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int key = min(kbase + j * 8 + g, a.cap - 1);
      const bf16* krow = kb + (long long)key * D + t * 8;
      uint4 kk[4];
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) kk[blk] = *reinterpret_cast<const uint4*>(krow + blk * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        mma_qk(s[j], qa[blk].x, qb[blk].x, qa[blk].y, qb[blk].y, kk[blk].x, kk[blk].y);
        mma_qk(s[j], qa[blk].z, qb[blk].z, qa[blk].w, qb[blk].w, kk[blk].z, kk[blk].w);
      }
    }
    // ---- V rows of the same keys: lane owns head dimensions 4*lane .. 4*lane+3 (requested before the softmax math)
    uint2 vv[KPI];
#pragma unroll
    for (int k = 0; k < KPI; ++k) {
      const int key = min(kbase + k, a.cap - 1);
      vv[k] = *reinterpret_cast<const uint2*>(vb + (long long)key * D + lane * 4);
    }
    // ---- mask, online softmax (rows g and g+8; this lane's columns are keys j*8 + 2t, 2t+1)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = kbase + j * 8 + 2 * t + e;
        const bool in = key < k1;
        s[j][e] = (in && key >= st0 && key < en0) ? s[j][e] * sc : -INFINITY;
        s[j][2 + e] = (in && key >= st1 && key < en1) ? s[j][2 + e] * sc : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float c0 = m0 == -INFINITY ? 0.f : exp2f(m0 - u0), c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - u1);
    m0 = n0; m1 = n1;
    l0 *= c0; l1 *= c1;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p0 = exp2f(s[j][e] - u0), p1 = exp2f(s[j][2 + e] - u1);
        l0 += p0; l1 += p1;
        if (g < NQ) s_p[warp][j * 8 + 2 * t + e][g] = p0;
        if (NQ > 8) s_p[warp][j * 8 + 2 * t + e][g + 8] = p1;
      }
    // correction factors of all queries: row q lives in lanes 4*(q%8) .. +3
    float corr[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) corr[q] = __shfl_sync(0xffffffffu, q < 8 ? c0 : c1, (q & 7) * 4);
    __syncwarp();
    // ---- O += P V on the FMA units
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[q][i] *= corr[q];
#pragma unroll
    for (int k = 0; k < KPI; ++k) {
      const float2 v01 = unpack_bf16x2(vv[k].x), v23 = unpack_bf16x2(vv[k].y);
#pragma unroll
      for (int q4 = 0; q4 < NQ / 4; ++q4) {
        const float4 p = *reinterpret_cast<const float4*>(&s_p[warp][k][q4 * 4]);
        const float pq[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[q4 * 4 + i][0] = fmaf(pq[i], v01.x, acc[q4 * 4 + i][0]);
          acc[q4 * 4 + i][1] = fmaf(pq[i], v01.y, acc[q4 * 4 + i][1]);
          acc[q4 * 4 + i][2] = fmaf(pq[i], v23.x, acc[q4 * 4 + i][2]);
          acc[q4 * 4 + i][3] = fmaf(pq[i], v23.y, acc[q4 * 4 + i][3]);
        }
      }
    }
  }
  // ---- merge the four warps, write this split's partial result
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (t == 0) {
    if (g < NQ) { s_m[warp][g] = m0; s_l[warp][g] = l0; }
    if (NQ > 8) { s_m[warp][g + 8] = m1; s_l[warp][g + 8] = l1; }
  }
#pragma unroll
  for (int q = 0; q < NQ; ++q) *reinterpret_cast<float4*>(&s_o[warp][q][lane * 4]) = make_float4(acc[q][0], acc[q][1], acc[q][2], acc[q][3]);
  __syncthreads();
  for (int i = threadIdx.x; i < nq * D; i += kDecThreads) {
    const int q = i / D, d = i % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, s_m[w][q]);
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = s_m[w][q] == -INFINITY ? 0.f : exp2f(s_m[w][q] - m);
      o += s_o[w][q][d] * f;
      l += s_l[w][q] * f;
    }
    const int tq = q / G, gg = q % G;
    const long long base = ((((long long)b * a.Tq + tq) * a.Hq + kvh * G + gg) * a.splits + split);
    a.part_o[base * D + d] = o;
    if (d == 0) {
      a.part_ml[base * 2] = m == -INFINITY ? -INFINITY : m * 0.6931471805599453f;   // natural-log units for the combine
      a.part_ml[base * 2 + 1] = l;
    }
  }
  combine_if_last(a, b, kvh, nq, G);
}

// one CTA per (b, t, head): merge the splits
__global__ void __launch_bounds__(128) decode_combine_kernel(DecodeArgs a) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const long long row = blockIdx.x;  // (b * Tq + t) * Hq + h
  const float* ml = a.part_ml + row * a.splits * 2;
  float m = -INFINITY;
  for (int s = 0; s < a.splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < a.splits; ++s) l += ml[2 * s] == -INFINITY ? 0.f : ml[2 * s + 1] * __expf(ml[2 * s] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < a.splits; ++s) {
      if (ml[2 * s] == -INFINITY) continue;
      o += a.part_o[(row * a.splits + s) * a.D + d] * __expf(ml[2 * s] - m);
    }
    a.out[row * a.D + d] = __float2bfloat16(o * inv);
  }
}

// cache[b, h, slot[b, t], :] = src[b, t, h, :] for slot >= 0 (K and V together)
__global__ void __launch_bounds__(256)
kv_cache_append_kernel(const bf16* __restrict__ k_new, const bf16* __restrict__ v_new, bf16* __restrict__ k_cache,
                       bf16* __restrict__ v_cache, const int* __restrict__ slots, int B, int T, int H, int D, int cap,
                       long long src_row_stride, long long src_batch_stride) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per = D / 8;
  if (vec >= (long long)B * T * H * per) return;
  const int v = vec % per;
  const int h = (vec / per) % H;
  const int t = (vec / ((long long)per * H)) % T;
  const int b = vec / ((long long)per * H * T);
  const int slot = slots[b * T + t];
  if (slot < 0 || slot >= cap) return;
  const long long src = (long long)b * src_batch_stride + (long long)t * src_row_stride + (long long)h * D + v * 8;
  const long long dst = (((long long)b * H + h) * cap + slot) * D + v * 8;
  *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(k_new + src);
  *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v_new + src);
}

// cache[b, h, dst[b] + r, :] = cache[b, h, src[b] + r, :] for r < rows, for sequences with enable[b] != 0
__global__ void __launch_bounds__(256)
kv_cache_move_kernel(bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, const int* __restrict__ src,
                     const int* __restrict__ dst, const int* __restrict__ enable, int B, int H, int D, int cap,
                     int rows) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per = D / 8;
  if (vec >= (long long)B * H * rows * per) return;
  const int v = vec % per;
  const int r = (vec / per) % rows;
  const int h = (vec / ((long long)per * rows)) % H;
  const int b = vec / ((long long)per * rows * H);
  if (enable && !enable[b]) return;
  const long long base = ((long long)b * H + h) * cap;
  const long long s = (base + src[b] + r) * D + v * 8, d = (base + dst[b] + r) * D + v * 8;
  *reinterpret_cast<uint4*>(k_cache + d) = *reinterpret_cast<const uint4*>(k_cache + s);
  *reinterpret_cast<uint4*>(v_cache + d) = *reinterpret_cast<const uint4*>(v_cache + s);
}

}  // namespace ksa

using namespace ksa;

// Scratch sizes the caller allocates: part_o [B*Tq*Hq*splits*D] fp32, part_ml [B*Tq*Hq*splits*2] fp32.
// counters: B*Hkv int32 zeros that launches on one stream may share (each launch leaves them zero), or null for a
// separate merge kernel.
KSA_API int ksa_decode_attn(const void* q, const void* k_cache, const void* v_cache, const void* start, const void* len,
                            void* part_o, void* part_ml, void* out, int B, int Tq, int Hq, int Hkv, int D, int cap,
                            int splits, int keys_per_split, float scale, void* counters, void* stream) {
  KSA_ENTER(q);
  KSA_REQUIRE(D == 128 || D == 64, "decode_attn: head_dim %d unsupported (64 or 128)", D);
  KSA_REQUIRE(Hq % Hkv == 0 && (Hq / Hkv) * Tq <= kDecMaxQ, "decode_attn: (Hq/Hkv) * Tq = %d exceeds %d queries per CTA",
              (Hq / Hkv) * Tq, kDecMaxQ);
  KSA_REQUIRE(splits >= 1 && keys_per_split >= 1, "decode_attn: bad split configuration");
  KSA_REQUIRE(counters == nullptr || splits <= kDecMaxSplits, "decode_attn: %d splits (at most %d with counters)", splits,
              kDecMaxSplits);
  if (B == 0) return 0;
  DecodeArgs a{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (const int*)start, (const int*)len,
               (float*)part_o, (float*)part_ml, (bf16*)out, B, Tq, Hq, Hkv, D, cap, splits, keys_per_split, scale,
               (int*)counters};
  dim3 grid(splits, Hkv, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int nq = (Hq / Hkv) * Tq;
  const bool dep = dependent_launch_enabled();
  if (D == 128 && nq <= 4) KSA_CHECK_CUDA(launch_kernel(dep, decode_attn_mma_kernel<4>, grid, dim3(kDecThreads), 0, st, a));
  else if (D == 128 && nq <= 8) KSA_CHECK_CUDA(launch_kernel(dep, decode_attn_mma_kernel<8>, grid, dim3(kDecThreads), 0, st, a));
  else if (D == 128) KSA_CHECK_CUDA(launch_kernel(dep, decode_attn_mma_kernel<16>, grid, dim3(kDecThreads), 0, st, a));
  else KSA_CHECK_CUDA(launch_kernel(dep, decode_attn_kernel<64>, grid, dim3(kDecThreads), 0, st, a));
  if (counters == nullptr) KSA_CHECK_CUDA(launch_kernel(dep, decode_combine_kernel, dim3(B * Tq * Hq), dim3(128), 0, st, a));
  return 0;
}

KSA_API int ksa_kv_cache_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const void* slots,
                                int B, int T, int H, int D, int cap, long long src_row_stride,
                                long long src_batch_stride, void* stream) {
  KSA_ENTER(k_new);
  KSA_REQUIRE(D % 8 == 0, "kv_cache_append: head_dim must be a multiple of 8");
  const long long n = (long long)B * T * H * (D / 8);
  if (n == 0) return 0;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), kv_cache_append_kernel, dim3((unsigned)((n + 255) / 256)),
                              dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), (const bf16*)k_new,
                              (const bf16*)v_new, (bf16*)k_cache, (bf16*)v_cache, (const int*)slots, B, T, H, D, cap,
                              src_row_stride, src_batch_stride));
  return 0;
}

KSA_API int ksa_kv_cache_move(void* k_cache, void* v_cache, const void* src, const void* dst, const void* enable, int B,
                              int H, int D, int cap, int rows, void* stream) {
  KSA_ENTER(k_cache);
  const long long n = (long long)B * H * rows * (D / 8);
  if (n == 0) return 0;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), kv_cache_move_kernel, dim3((unsigned)((n + 255) / 256)),
                              dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), (bf16*)k_cache, (bf16*)v_cache,
                              (const int*)src, (const int*)dst, (const int*)enable, B, H, D, cap, rows));
  return 0;
}
