// Attention for the summary-token queries of Kwai Summary Attention.
//
// Summary token j of chunk i attends the C text keys of its own chunk and the
// summary keys (i, j') with j' <= j.  That is one query against C + S keys per
// chunk: matrix-vector work, bound by reading the chunk's K and V once, so it
// runs on the CUDA cores next to the tensor-core kernel that serves the text
// queries.  The reference pushes these rows through the same block-sparse
// kernel as a 128-row tile that is almost entirely masked
// (summary_attn/mask.py:19-31 in the reference's summary_attn wheel).
#include "common.cuh"
#include "host.h"

namespace ksa {

struct SumAttnArgs {
  const bf16* qs; const bf16* k; const bf16* v; const bf16* ks; const bf16* vs;
  long long qs_rs, qs_bs, k_rs, k_bs, v_rs, v_bs, ks_rs, ks_bs, vs_rs, vs_bs;
  bf16* os; long long os_rs, os_bs;   // [B, Nq, Hq, HD]
  float* lse;                         // [B, Hq, Nq]
  int B, Hq, Hkv, HD;
  int Nq;          // local summary query rows (= local chunks * S)
  int L;           // global text length (ragged last chunk)
  int chunk, n_sum;
  int chunk0;      // global chunk index of local summary row 0
  int k_off;       // global text index of local text key row 0
  int s_off;       // global summary index of local summary key row 0
  float scale;
  // backward only
  const bf16* d_os; bf16* dqs; long long dqs_rs, dqs_bs;
  bf16* dk; bf16* dv; bf16* dks; bf16* dvs;
  long long dk_rs, dk_bs, dv_rs, dv_bs, dks_rs, dks_bs, dvs_rs, dvs_bs;
  const float* dks32; const float* dvs32;  // optional fp32 partials [B, Nk_sum, Hkv, HD] that replace the bf16 base
  int Ns_k;                                // rows of the summary key buffer (for the fp32 partial indexing)
};

__device__ __forceinline__ float dot_row(const float* q_s, const bf16* row, int HD) {
  float acc = 0.f;
  for (int d = 0; d < HD; d += 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(row + d);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(w[i]);
      acc += q_s[d + 2 * i] * f.x + q_s[d + 2 * i + 1] * f.y;
    }
  }
  return acc;
}

__device__ __forceinline__ float block_reduce_sum128(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}
__device__ __forceinline__ float block_reduce_max128(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
}

// Key row pointer for key index kk in [0, n_text + j]: text keys first, then the chunk's summary keys.
__device__ __forceinline__ const bf16* key_row(const bf16* text, long long t_rs, const bf16* sum, long long s_rs,
                                               int kk, int n_text, int text0_local, int sum0_local) {
  return kk < n_text ? text + (long long)(text0_local + kk) * t_rs : sum + (long long)(sum0_local + kk - n_text) * s_rs;
}

// grid (local chunks, Hq, B), 128 threads, dynamic smem = (HD + C + S) floats
__global__ void __launch_bounds__(128) summary_attn_fwd_kernel(SumAttnArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[4];
  float* q_s = sm;
  float* sc = sm + a.HD;
  const int ci = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (a.Hq / a.Hkv);
  const int cg = a.chunk0 + ci;
  const int n_text = min(a.chunk, a.L - cg * a.chunk);
  const int text0 = cg * a.chunk - a.k_off;
  const int sum0 = cg * a.n_sum - a.s_off;
  const bf16* kb = a.k + (long long)b * a.k_bs + (long long)kvh * a.HD;
  const bf16* vb = a.v + (long long)b * a.v_bs + (long long)kvh * a.HD;
  const bf16* ksb = a.ks + (long long)b * a.ks_bs + (long long)kvh * a.HD;
  const bf16* vsb = a.vs + (long long)b * a.vs_bs + (long long)kvh * a.HD;
  for (int j = 0; j < a.n_sum; ++j) {
    const int row = ci * a.n_sum + j;
    const bf16* qp = a.qs + (long long)b * a.qs_bs + (long long)row * a.qs_rs + (long long)head * a.HD;
    __syncthreads();
    for (int d = threadIdx.x; d < a.HD; d += 128) q_s[d] = __bfloat162float(qp[d]);
    __syncthreads();
    const int nk = n_text + j + 1;
    float mx = -INFINITY;
    for (int kk = threadIdx.x; kk < nk; kk += 128) {
      const float s = dot_row(q_s, key_row(kb, a.k_rs, ksb, a.ks_rs, kk, n_text, text0, sum0), a.HD) * a.scale;
      sc[kk] = s;
      mx = fmaxf(mx, s);
    }
    mx = block_reduce_max128(mx, red);
    float sum = 0.f;
    for (int kk = threadIdx.x; kk < nk; kk += 128) {
      const float pr = __expf(sc[kk] - mx);
      sc[kk] = pr;
      sum += pr;
    }
    sum = block_reduce_sum128(sum, red);
    const float inv = 1.f / sum;
    for (int d = threadIdx.x; d < a.HD; d += 128) {
      float acc = 0.f;
      for (int kk = 0; kk < nk; ++kk)
        acc += sc[kk] * __bfloat162float(key_row(vb, a.v_rs, vsb, a.vs_rs, kk, n_text, text0, sum0)[d]);
      a.os[(long long)b * a.os_bs + (long long)row * a.os_rs + (long long)head * a.HD + d] = __float2bfloat16(acc * inv);
    }
    if (threadIdx.x == 0 && a.lse) a.lse[((long long)b * a.Hq + head) * a.Nq + row] = mx + __logf(sum);
  }
}

// grid (local chunks, Hkv, B), 128 threads.
// dynamic smem: nq * (2*HD + 2*(C+S)) floats with nq = (Hq/Hkv) * S queries per block.
// dK/dV of the chunk's text keys and summary keys are ADDED to what the text-query backward wrote.
__global__ void __launch_bounds__(128) summary_attn_bwd_kernel(SumAttnArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[4];
  const int G = a.Hq / a.Hkv, S = a.n_sum, HD = a.HD;
  const int nq = G * S;
  const int nkmax = a.chunk + S;
  float* q_s = sm;                  // [nq][HD]
  float* do_s = q_s + nq * HD;      // [nq][HD]
  float* p_s = do_s + nq * HD;      // [nq][nkmax]
  float* ds_s = p_s + nq * nkmax;   // [nq][nkmax]
  const int ci = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int cg = a.chunk0 + ci;
  const int n_text = min(a.chunk, a.L - cg * a.chunk);
  const int text0 = cg * a.chunk - a.k_off;
  const int sum0 = cg * S - a.s_off;
  const bf16* kb = a.k + (long long)b * a.k_bs + (long long)kvh * HD;
  const bf16* vb = a.v + (long long)b * a.v_bs + (long long)kvh * HD;
  const bf16* ksb = a.ks + (long long)b * a.ks_bs + (long long)kvh * HD;
  const bf16* vsb = a.vs + (long long)b * a.vs_bs + (long long)kvh * HD;
  for (int qi = 0; qi < nq; ++qi) {
    const int g = qi / S, j = qi % S;
    const int head = kvh * G + g, row = ci * S + j;
    const long long qoff = (long long)b * a.qs_bs + (long long)row * a.qs_rs + (long long)head * HD;
    const long long ooff = (long long)b * a.os_bs + (long long)row * a.os_rs + (long long)head * HD;
    float part = 0.f;
    for (int d = threadIdx.x; d < HD; d += 128) {
      q_s[qi * HD + d] = __bfloat162float(a.qs[qoff + d]);
      const float g_o = __bfloat162float(a.d_os[ooff + d]);
      do_s[qi * HD + d] = g_o;
      part += g_o * __bfloat162float(a.os[ooff + d]);
    }
    const float delta = block_reduce_sum128(part, red);   // also orders the smem writes above
    const float lse = a.lse[((long long)b * a.Hq + head) * a.Nq + row];
    const int nk = n_text + j + 1;
    for (int kk = threadIdx.x; kk < nkmax; kk += 128) {
      float pr = 0.f, ds = 0.f;
      if (kk < nk) {
        const float s = dot_row(q_s + qi * HD, key_row(kb, a.k_rs, ksb, a.ks_rs, kk, n_text, text0, sum0), HD) * a.scale;
        pr = __expf(s - lse);
        const float dp = dot_row(do_s + qi * HD, key_row(vb, a.v_rs, vsb, a.vs_rs, kk, n_text, text0, sum0), HD);
        ds = pr * (dp - delta) * a.scale;
      }
      p_s[qi * nkmax + kk] = pr;
      ds_s[qi * nkmax + kk] = ds;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < HD; d += 128) {
      float acc = 0.f;
      for (int kk = 0; kk < nk; ++kk)
        acc += ds_s[qi * nkmax + kk] * __bfloat162float(key_row(kb, a.k_rs, ksb, a.ks_rs, kk, n_text, text0, sum0)[d]);
      a.dqs[(long long)b * a.dqs_bs + (long long)row * a.dqs_rs + (long long)head * HD + d] = __float2bfloat16(acc);
    }
  }
  __syncthreads();
  // dK[kk][d] += sum_qi ds[qi][kk] q[qi][d];  dV[kk][d] += sum_qi p[qi][kk] do[qi][d]
  const int nk_all = n_text + S;
  for (int idx = threadIdx.x; idx < nk_all * HD; idx += 128) {
    const int kk = idx / HD, d = idx % HD;
    float gk = 0.f, gv = 0.f;
    for (int qi = 0; qi < nq; ++qi) {
      gk += ds_s[qi * nkmax + kk] * q_s[qi * HD + d];
      gv += p_s[qi * nkmax + kk] * do_s[qi * HD + d];
    }
    bf16 *pk, *pv;
    if (kk < n_text) {
      pk = a.dk + (long long)b * a.dk_bs + (long long)(text0 + kk) * a.dk_rs + (long long)kvh * HD + d;
      pv = a.dv + (long long)b * a.dv_bs + (long long)(text0 + kk) * a.dv_rs + (long long)kvh * HD + d;
    } else {
      pk = a.dks + (long long)b * a.dks_bs + (long long)(sum0 + kk - n_text) * a.dks_rs + (long long)kvh * HD + d;
      pv = a.dvs + (long long)b * a.dvs_bs + (long long)(sum0 + kk - n_text) * a.dvs_rs + (long long)kvh * HD + d;
    }
    float base_k = __bfloat162float(*pk), base_v = __bfloat162float(*pv);
    if (kk >= n_text && a.dks32) {  // the text-query backward left fp32 partial sums instead of bf16 values
      const long long o = (((long long)b * a.Ns_k + (sum0 + kk - n_text)) * a.Hkv + kvh) * HD + d;
      base_k = a.dks32[o];
      base_v = a.dvs32[o];
    }
    *pk = __float2bfloat16(base_k + gk);
    *pv = __float2bfloat16(base_v + gv);
  }
}


// ------------------------------------------------------------------------------------------------
// Fast paths (head dim 128, at most 8 queries per KV group): one CTA per (chunk, KV head) serves all G*S summary
// queries of the group.
// Forward fast path.  grid (local chunks, Hkv, B), 256 threads.  The chunk's V rows are staged in shared memory
// (every output column reads all of them); its K rows are read straight from global memory by the threads that
// compute their dot products (two threads per key, half a row = eight 16-byte loads in flight each), so the K and V
// traffic of a CTA overlaps, shared memory stays near 35 KB and all CTAs of an 8k sequence are resident at once.
// The G*S queries of the group are served together: one pass over a key row yields all their scores, one warp per
// query does the softmax, and the P V product runs with thread = (query, column).
// dynamic smem: V rows [nk_max][HD] bf16 | q[nq][HD] fp32 | p[nq][nk_max] fp32
constexpr int kSumFwdThreads = 256;
constexpr int kSumFwdMaxQ = 8;

template <int HD>
__global__ void __launch_bounds__(kSumFwdThreads) summary_attn_fwd_fast_kernel(SumAttnArgs a, int nk_max) {
  extern __shared__ uint32_t smw[];
  const int G = a.Hq / a.Hkv, S = a.n_sum, nq = G * S;
  bf16* v_s = reinterpret_cast<bf16*>(smw);
  float* q_s = reinterpret_cast<float*>(v_s + (size_t)nk_max * HD);
  float* p_s = q_s + nq * HD;
  const int ci = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int cg = a.chunk0 + ci;
  const int n_text = min(a.chunk, a.L - cg * a.chunk);
  const int text0 = cg * a.chunk - a.k_off, sum0 = cg * S - a.s_off;
  const int nk_all = n_text + S;
  const bf16* kt = a.k + (long long)b * a.k_bs + (long long)kvh * HD;
  const bf16* ks = a.ks + (long long)b * a.ks_bs + (long long)kvh * HD;
  const bf16* vt = a.v + (long long)b * a.v_bs + (long long)kvh * HD;
  const bf16* vs = a.vs + (long long)b * a.vs_bs + (long long)kvh * HD;
  // ---- V rows -> shared memory (requests first, four at a time per thread), queries -> fp32
  constexpr int kVec = HD / 8;
  for (int i0 = threadIdx.x; i0 < nk_all * kVec; i0 += kSumFwdThreads * 4) {
    uint4 u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = i0 + j * kSumFwdThreads;
      if (idx < nk_all * kVec) {
        const int kk = idx / kVec, v = idx % kVec;
        u[j] = *reinterpret_cast<const uint4*>(key_row(vt, a.v_rs, vs, a.vs_rs, kk, n_text, text0, sum0) + v * 8);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = i0 + j * kSumFwdThreads;
      if (idx < nk_all * kVec) *reinterpret_cast<uint4*>(v_s + (size_t)idx * 8) = u[j];
    }
  }
  for (int idx = threadIdx.x; idx < nq * HD; idx += kSumFwdThreads) {
    const int qi = idx / HD, d = idx % HD;
    const int head = kvh * G + qi / S, row = ci * S + qi % S;
    q_s[idx] = __bfloat162float(a.qs[(long long)b * a.qs_bs + (long long)row * a.qs_rs + (long long)head * HD + d]) * a.scale;
  }
  __syncthreads();
  // ---- scores: two threads per key, each half a row
  {
    const int half = threadIdx.x & 1;
    // every thread of a warp runs the same number of rounds (the two halves of a key meet in a shuffle below)
    for (int kk0 = 0; kk0 < nk_all; kk0 += kSumFwdThreads / 2) {
      const int kk = kk0 + (threadIdx.x >> 1);
      const bool valid = kk < nk_all;
      const bf16* row = key_row(kt, a.k_rs, ks, a.ks_rs, valid ? kk : 0, n_text, text0, sum0) + half * (HD / 2);
      uint4 u[HD / 16];
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) u[j] = valid ? *reinterpret_cast<const uint4*>(row + j * 8) : make_uint4(0, 0, 0, 0);
      float acc[kSumFwdMaxQ];
#pragma unroll
      for (int qi = 0; qi < kSumFwdMaxQ; ++qi) acc[qi] = 0.f;
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        const uint32_t w[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = unpack_bf16x2(w[i]);
          const int d = half * (HD / 2) + j * 8 + 2 * i;
#pragma unroll
          for (int qi = 0; qi < kSumFwdMaxQ; ++qi)
            if (qi < nq) acc[qi] += q_s[qi * HD + d] * f.x + q_s[qi * HD + d + 1] * f.y;
        }
      }
#pragma unroll
      for (int qi = 0; qi < kSumFwdMaxQ; ++qi) {
        if (qi < nq) {
          const float sc = acc[qi] + __shfl_xor_sync(0xffffffffu, acc[qi], 1);
          // summary query j sees the chunk's text keys and summary keys 0..j
          if (half == 0 && valid) p_s[qi * nk_max + kk] = kk < n_text + (qi % S) + 1 ? sc : -INFINITY;
        }
      }
    }
  }
  __syncthreads();
  // ---- softmax: one warp per query
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int qi = warp; qi < nq; qi += kSumFwdThreads / 32) {
    float mx = -INFINITY;
    for (int kk = lane; kk < nk_all; kk += 32) mx = fmaxf(mx, p_s[qi * nk_max + kk]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int kk = lane; kk < nk_all; kk += 32) {
      const float pr = __expf(p_s[qi * nk_max + kk] - mx);
      p_s[qi * nk_max + kk] = pr;
      sum += pr;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int kk = lane; kk < nk_all; kk += 32) p_s[qi * nk_max + kk] *= inv;
    if (lane == 0 && a.lse) {
      const int head = kvh * G + qi / S, row = ci * S + qi % S;
      a.lse[((long long)b * a.Hq + head) * a.Nq + row] = mx + __logf(sum);
    }
  }
  __syncthreads();
  // ---- O = P V: thread = (query, pair of columns)
  for (int idx = threadIdx.x; idx < nq * (HD / 2); idx += kSumFwdThreads) {
    const int qi = idx / (HD / 2), d2 = idx % (HD / 2);
    const uint32_t* vcol = reinterpret_cast<const uint32_t*>(v_s) + d2;
    const float* pr = p_s + qi * nk_max;
    float o0 = 0.f, o1 = 0.f;
    for (int kk = 0; kk < nk_all; ++kk) {
      const float2 f = unpack_bf16x2(vcol[(size_t)kk * (HD / 2)]);
      o0 = fmaf(pr[kk], f.x, o0);
      o1 = fmaf(pr[kk], f.y, o1);
    }
    const int head = kvh * G + qi / S, row = ci * S + qi % S;
    *reinterpret_cast<uint32_t*>(a.os + (long long)b * a.os_bs + (long long)row * a.os_rs + (long long)head * HD + 2 * d2) =
        pack_bf16x2(o0, o1);
  }
}

// Backward fast path.  grid (local chunks, Hkv, B), 256 threads, head dim 128.  Only the chunk's K rows are staged
// (padded by 16 bytes per row: "two threads per key" reads of 16-byte vectors and "thread = column" reads of words
// are both conflict-free); V rows are read straight from global memory by the threads that need their dot
// products with dO.  The G*S queries of the group are served together.
// dynamic smem: K rows [nk_max][HD + 8] bf16 | q[nq][HD] | do[nq][HD] | p[nq][nk_max] | ds[nq][nk_max] | delta, lse [2 nq]
constexpr int kSumBwdThreads = 256;
constexpr int kSumBwdMaxQ = 8;

template <int HD>
__global__ void __launch_bounds__(kSumBwdThreads) summary_attn_bwd_fast_kernel(SumAttnArgs a, int nk_max) {
  extern __shared__ uint32_t smw[];
  constexpr int kRowElems = HD + 8;                   // padded K row, bf16 elements
  const int G = a.Hq / a.Hkv, S = a.n_sum, nq = G * S;
  bf16* k_s = reinterpret_cast<bf16*>(smw);
  float* q_s = reinterpret_cast<float*>(k_s + (size_t)nk_max * kRowElems);
  float* do_s = q_s + nq * HD;
  float* p_s = do_s + nq * HD;
  float* ds_s = p_s + nq * nk_max;
  float* dl_s = ds_s + nq * nk_max;                    // delta[nq], lse[nq]
  const int ci = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int cg = a.chunk0 + ci;
  const int n_text = min(a.chunk, a.L - cg * a.chunk);
  const int text0 = cg * a.chunk - a.k_off, sum0 = cg * S - a.s_off;
  const int nk_all = n_text + S;
  const bf16* kt = a.k + (long long)b * a.k_bs + (long long)kvh * HD;
  const bf16* ks = a.ks + (long long)b * a.ks_bs + (long long)kvh * HD;
  const bf16* vt = a.v + (long long)b * a.v_bs + (long long)kvh * HD;
  const bf16* vs = a.vs + (long long)b * a.vs_bs + (long long)kvh * HD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // ---- K rows -> shared memory, four requests in flight per thread
  constexpr int kVec = HD / 8;
  for (int i0 = threadIdx.x; i0 < nk_all * kVec; i0 += kSumBwdThreads * 4) {
    uint4 u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = i0 + j * kSumBwdThreads;
      if (idx < nk_all * kVec)
        u[j] = *reinterpret_cast<const uint4*>(key_row(kt, a.k_rs, ks, a.ks_rs, idx / kVec, n_text, text0, sum0) + (idx % kVec) * 8);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = i0 + j * kSumBwdThreads;
      if (idx < nk_all * kVec) *reinterpret_cast<uint4*>(k_s + (size_t)(idx / kVec) * kRowElems + (idx % kVec) * 8) = u[j];
    }
  }
  // ---- q, dO -> fp32; delta = sum_d dO * O and the log-sum-exp, one warp per query
  for (int qi = warp; qi < nq; qi += kSumBwdThreads / 32) {
    const int head = kvh * G + qi / S, row = ci * S + qi % S;
    const long long qoff = (long long)b * a.qs_bs + (long long)row * a.qs_rs + (long long)head * HD;
    const long long ooff = (long long)b * a.os_bs + (long long)row * a.os_rs + (long long)head * HD;
    float part = 0.f;
    for (int d = lane; d < HD; d += 32) {
      q_s[qi * HD + d] = __bfloat162float(a.qs[qoff + d]);
      const float g_o = __bfloat162float(a.d_os[ooff + d]);
      do_s[qi * HD + d] = g_o;
      part += g_o * __bfloat162float(a.os[ooff + d]);
    }
    part = warp_sum(part);
    if (lane == 0) {
      dl_s[qi] = part;
      dl_s[nq + qi] = a.lse[((long long)b * a.Hq + head) * a.Nq + row];
    }
  }
  __syncthreads();
  // ---- p and dS: two threads per key, each half of the K row (shared memory) and of the V row (global memory);
  // every thread of a warp runs the same number of rounds, the two halves meet in a shuffle
  {
    const int half = threadIdx.x & 1;
    for (int kk0 = 0; kk0 < nk_all; kk0 += kSumBwdThreads / 2) {
      const int kk = kk0 + (threadIdx.x >> 1);
      const bool valid = kk < nk_all;
      const bf16* vrow = key_row(vt, a.v_rs, vs, a.vs_rs, valid ? kk : 0, n_text, text0, sum0) + half * (HD / 2);
      const bf16* krow = k_s + (size_t)(valid ? kk : 0) * kRowElems + half * (HD / 2);
      uint4 uv[HD / 16];
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) uv[j] = valid ? *reinterpret_cast<const uint4*>(vrow + j * 8) : make_uint4(0, 0, 0, 0);
      float sc[kSumBwdMaxQ], dp[kSumBwdMaxQ];
#pragma unroll
      for (int qi = 0; qi < kSumBwdMaxQ; ++qi) { sc[qi] = 0.f; dp[qi] = 0.f; }
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) {
        const uint4 uk = *reinterpret_cast<const uint4*>(krow + j * 8);
        const uint32_t wk[4] = {uk.x, uk.y, uk.z, uk.w}, wv[4] = {uv[j].x, uv[j].y, uv[j].z, uv[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fk = unpack_bf16x2(wk[i]), fv = unpack_bf16x2(wv[i]);
          const int d = half * (HD / 2) + j * 8 + 2 * i;
#pragma unroll
          for (int qi = 0; qi < kSumBwdMaxQ; ++qi)
            if (qi < nq) {
              sc[qi] += q_s[qi * HD + d] * fk.x + q_s[qi * HD + d + 1] * fk.y;
              dp[qi] += do_s[qi * HD + d] * fv.x + do_s[qi * HD + d + 1] * fv.y;
            }
        }
      }
#pragma unroll
      for (int qi = 0; qi < kSumBwdMaxQ; ++qi) {
        if (qi < nq) {
          const float s2 = sc[qi] + __shfl_xor_sync(0xffffffffu, sc[qi], 1);
          const float d2 = dp[qi] + __shfl_xor_sync(0xffffffffu, dp[qi], 1);
          if (half == 0 && valid) {
            const bool seen = kk < n_text + (qi % S) + 1;   // summary query j sees text keys and summary keys 0..j
            const float pr = seen ? __expf(s2 * a.scale - dl_s[nq + qi]) : 0.f;
            p_s[qi * nk_max + kk] = pr;
            ds_s[qi * nk_max + kk] = pr * (d2 - dl_s[qi]) * a.scale;
          }
        }
      }
    }
  }
  __syncthreads();
  // ---- dQ[qi][d] = sum_kk dS[qi][kk] K[kk][d]: thread = (query, pair of columns)
  for (int idx = threadIdx.x; idx < nq * (HD / 2); idx += kSumBwdThreads) {
    const int qi = idx / (HD / 2), d2 = idx % (HD / 2);
    const uint32_t* kcol = reinterpret_cast<const uint32_t*>(k_s) + d2;
    const float* dsr = ds_s + qi * nk_max;
    float g0 = 0.f, g1 = 0.f;
    for (int kk = 0; kk < nk_all; ++kk) {
      const float2 f = unpack_bf16x2(kcol[(size_t)kk * (kRowElems / 2)]);
      g0 = fmaf(dsr[kk], f.x, g0);
      g1 = fmaf(dsr[kk], f.y, g1);
    }
    const int head = kvh * G + qi / S, row = ci * S + qi % S;
    *reinterpret_cast<uint32_t*>(a.dqs + (long long)b * a.dqs_bs + (long long)row * a.dqs_rs + (long long)head * HD + 2 * d2) =
        pack_bf16x2(g0, g1);
  }
  // dK[kk][d] += sum_qi ds[qi][kk] q[qi][d];  dV[kk][d] += sum_qi p[qi][kk] do[qi][d]: eight columns (16 bytes) per
  // thread and read-modify-write, so that the two global round trips per key row are 16 accesses instead of 64
  for (int idx = threadIdx.x; idx < nk_all * kVec; idx += kSumBwdThreads) {
    const int kk = idx / kVec, d = (idx % kVec) * 8;
    float gk[8], gv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { gk[e] = 0.f; gv[e] = 0.f; }
    for (int qi = 0; qi < nq; ++qi) {
      const float dsv = ds_s[qi * nk_max + kk], pv = p_s[qi * nk_max + kk];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        gk[e] += dsv * q_s[qi * HD + d + e];
        gv[e] += pv * do_s[qi * HD + d + e];
      }
    }
    bf16 *pk, *pv;
    if (kk < n_text) {
      pk = a.dk + (long long)b * a.dk_bs + (long long)(text0 + kk) * a.dk_rs + (long long)kvh * HD + d;
      pv = a.dv + (long long)b * a.dv_bs + (long long)(text0 + kk) * a.dv_rs + (long long)kvh * HD + d;
    } else {
      pk = a.dks + (long long)b * a.dks_bs + (long long)(sum0 + kk - n_text) * a.dks_rs + (long long)kvh * HD + d;
      pv = a.dvs + (long long)b * a.dvs_bs + (long long)(sum0 + kk - n_text) * a.dvs_rs + (long long)kvh * HD + d;
    }
    float bk[8], bv[8];
    if (kk >= n_text && a.dks32) {
      const long long o = (((long long)b * a.Ns_k + (sum0 + kk - n_text)) * a.Hkv + kvh) * HD + d;
      const float4 k0 = *reinterpret_cast<const float4*>(a.dks32 + o), k1 = *reinterpret_cast<const float4*>(a.dks32 + o + 4);
      const float4 v0 = *reinterpret_cast<const float4*>(a.dvs32 + o), v1 = *reinterpret_cast<const float4*>(a.dvs32 + o + 4);
      bk[0] = k0.x; bk[1] = k0.y; bk[2] = k0.z; bk[3] = k0.w; bk[4] = k1.x; bk[5] = k1.y; bk[6] = k1.z; bk[7] = k1.w;
      bv[0] = v0.x; bv[1] = v0.y; bv[2] = v0.z; bv[3] = v0.w; bv[4] = v1.x; bv[5] = v1.y; bv[6] = v1.z; bv[7] = v1.w;
    } else {
      const uint4 uk = *reinterpret_cast<const uint4*>(pk), uv = *reinterpret_cast<const uint4*>(pv);
      const uint32_t ku[4] = {uk.x, uk.y, uk.z, uk.w}, vu[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fk = unpack_bf16x2(ku[e]), fv = unpack_bf16x2(vu[e]);
        bk[2 * e] = fk.x; bk[2 * e + 1] = fk.y; bv[2 * e] = fv.x; bv[2 * e + 1] = fv.y;
      }
    }
    uint4 ok, ov;
    ok.x = pack_bf16x2(bk[0] + gk[0], bk[1] + gk[1]); ok.y = pack_bf16x2(bk[2] + gk[2], bk[3] + gk[3]);
    ok.z = pack_bf16x2(bk[4] + gk[4], bk[5] + gk[5]); ok.w = pack_bf16x2(bk[6] + gk[6], bk[7] + gk[7]);
    ov.x = pack_bf16x2(bv[0] + gv[0], bv[1] + gv[1]); ov.y = pack_bf16x2(bv[2] + gv[2], bv[3] + gv[3]);
    ov.z = pack_bf16x2(bv[4] + gv[4], bv[5] + gv[5]); ov.w = pack_bf16x2(bv[6] + gv[6], bv[7] + gv[7]);
    *reinterpret_cast<uint4*>(pk) = ok;
    *reinterpret_cast<uint4*>(pv) = ov;
  }
}

}  // namespace ksa

using namespace ksa;

KSA_API int ksa_summary_attn_fwd(const void* qs, const void* k, const void* v, const void* ks, const void* vs, void* os,
                                 void* lse, int B, int Hq, int Hkv, int HD, int Nq, int L, long long qs_rs,
                                 long long qs_bs, long long k_rs, long long k_bs, long long v_rs, long long v_bs,
                                 long long ks_rs, long long ks_bs, long long vs_rs, long long vs_bs, long long os_rs,
                                 long long os_bs, int chunk, int n_sum, int chunk0, int k_off, int s_off, float scale,
                                 void* stream) {
  KSA_ENTER(qs);
  KSA_REQUIRE(HD % 8 == 0 && Hq % Hkv == 0 && n_sum > 0 && Nq % n_sum == 0, "summary_attn_fwd: bad shape");
  if (B == 0 || Nq == 0) return 0;
  SumAttnArgs a{};
  a.qs = (const bf16*)qs; a.k = (const bf16*)k; a.v = (const bf16*)v; a.ks = (const bf16*)ks; a.vs = (const bf16*)vs;
  a.qs_rs = qs_rs; a.qs_bs = qs_bs; a.k_rs = k_rs; a.k_bs = k_bs; a.v_rs = v_rs; a.v_bs = v_bs;
  a.ks_rs = ks_rs; a.ks_bs = ks_bs; a.vs_rs = vs_rs; a.vs_bs = vs_bs;
  a.os = (bf16*)os; a.os_rs = os_rs; a.os_bs = os_bs; a.lse = (float*)lse;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.HD = HD; a.Nq = Nq; a.L = L; a.chunk = chunk; a.n_sum = n_sum;
  a.chunk0 = chunk0; a.k_off = k_off; a.s_off = s_off; a.scale = scale;
  {
    const int nq = (Hq / Hkv) * n_sum, nk_max = chunk + n_sum;
    const size_t fast_smem = (size_t)nk_max * HD * sizeof(bf16) + (size_t)nq * (HD + nk_max) * sizeof(float);
    if (HD == 128 && nq <= kSumFwdMaxQ && fast_smem <= 100 * 1024 && os_rs % 2 == 0) {
      static bool attr = false;
      if (!attr) {
        KSA_CHECK_CUDA(cudaFuncSetAttribute(summary_attn_fwd_fast_kernel<128>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr = true;
      }
      dim3 fgrid(Nq / n_sum, Hkv, B);
      summary_attn_fwd_fast_kernel<128><<<fgrid, kSumFwdThreads, fast_smem, reinterpret_cast<cudaStream_t>(stream)>>>(a, nk_max);
      KSA_CHECK_CUDA(cudaGetLastError());
      return 0;
    }
  }
  const size_t smem = (size_t)(HD + chunk + n_sum) * sizeof(float);
  KSA_REQUIRE(smem <= 48 * 1024, "summary_attn_fwd: chunk %d too large for the SIMT kernel", chunk);
  dim3 grid(Nq / n_sum, Hq, B);
  summary_attn_fwd_kernel<<<grid, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_summary_attn_bwd(const void* qs, const void* k, const void* v, const void* ks, const void* vs,
                                 const void* os, const void* d_os, const void* lse, void* dqs, void* dk, void* dv,
                                 void* dks, void* dvs, int B, int Hq, int Hkv, int HD, int Nq, int L, long long qs_rs,
                                 long long qs_bs, long long k_rs, long long k_bs, long long v_rs, long long v_bs,
                                 long long ks_rs, long long ks_bs, long long vs_rs, long long vs_bs, long long os_rs,
                                 long long os_bs, long long dqs_rs, long long dqs_bs, long long dk_rs, long long dk_bs,
                                 long long dv_rs, long long dv_bs, long long dks_rs, long long dks_bs, long long dvs_rs,
                                 long long dvs_bs, int chunk, int n_sum, int chunk0, int k_off, int s_off, float scale,
                                 const void* dks32, const void* dvs32, int Ns_k, void* stream) {
  KSA_ENTER(qs);
  KSA_REQUIRE(HD % 8 == 0 && Hq % Hkv == 0 && n_sum > 0 && Nq % n_sum == 0, "summary_attn_bwd: bad shape");
  if (B == 0 || Nq == 0) return 0;
  SumAttnArgs a{};
  a.qs = (const bf16*)qs; a.k = (const bf16*)k; a.v = (const bf16*)v; a.ks = (const bf16*)ks; a.vs = (const bf16*)vs;
  a.qs_rs = qs_rs; a.qs_bs = qs_bs; a.k_rs = k_rs; a.k_bs = k_bs; a.v_rs = v_rs; a.v_bs = v_bs;
  a.ks_rs = ks_rs; a.ks_bs = ks_bs; a.vs_rs = vs_rs; a.vs_bs = vs_bs;
  a.os = (bf16*)os; a.os_rs = os_rs; a.os_bs = os_bs; a.lse = (float*)lse;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.HD = HD; a.Nq = Nq; a.L = L; a.chunk = chunk; a.n_sum = n_sum;
  a.chunk0 = chunk0; a.k_off = k_off; a.s_off = s_off; a.scale = scale;
  a.d_os = (const bf16*)d_os; a.dqs = (bf16*)dqs; a.dqs_rs = dqs_rs; a.dqs_bs = dqs_bs;
  a.dk = (bf16*)dk; a.dv = (bf16*)dv; a.dks = (bf16*)dks; a.dvs = (bf16*)dvs;
  a.dk_rs = dk_rs; a.dk_bs = dk_bs; a.dv_rs = dv_rs; a.dv_bs = dv_bs;
  a.dks_rs = dks_rs; a.dks_bs = dks_bs; a.dvs_rs = dvs_rs; a.dvs_bs = dvs_bs;
  a.dks32 = (const float*)dks32; a.dvs32 = (const float*)dvs32; a.Ns_k = Ns_k;
  const int nq = (Hq / Hkv) * n_sum;
  {
    const int nk_max = chunk + n_sum;
    const size_t fast_smem = (size_t)nk_max * (HD + 8) * sizeof(bf16) + (size_t)nq * (2 * HD + 2 * nk_max + 2) * sizeof(float);
    if (HD == 128 && nq <= kSumBwdMaxQ && fast_smem <= 100 * 1024 && dqs_rs % 2 == 0) {
      static bool fattr = false;
      if (!fattr) {
        KSA_CHECK_CUDA(cudaFuncSetAttribute(summary_attn_bwd_fast_kernel<128>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        fattr = true;
      }
      dim3 fgrid(Nq / n_sum, Hkv, B);
      summary_attn_bwd_fast_kernel<128><<<fgrid, kSumBwdThreads, fast_smem, reinterpret_cast<cudaStream_t>(stream)>>>(a, nk_max);
      KSA_CHECK_CUDA(cudaGetLastError());
      return 0;
    }
  }
  const size_t smem = (size_t)nq * (2 * HD + 2 * (chunk + n_sum)) * sizeof(float);
  KSA_REQUIRE(smem <= 200 * 1024, "summary_attn_bwd: %zu bytes of shared memory needed (chunk %d, %d queries)", smem,
              chunk, nq);
  static bool attr = false;
  if (!attr) {
    KSA_CHECK_CUDA(cudaFuncSetAttribute(summary_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr = true;
  }
  dim3 grid(Nq / n_sum, Hkv, B);
  summary_attn_bwd_kernel<<<grid, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}
