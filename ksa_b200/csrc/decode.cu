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
};

template <int D>
__global__ void __launch_bounds__(kDecThreads) decode_attn_kernel(DecodeArgs a) {
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
}

// one CTA per (b, t, head): merge the splits
__global__ void __launch_bounds__(128) decode_combine_kernel(DecodeArgs a) {
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
KSA_API int ksa_decode_attn(const void* q, const void* k_cache, const void* v_cache, const void* start, const void* len,
                            void* part_o, void* part_ml, void* out, int B, int Tq, int Hq, int Hkv, int D, int cap,
                            int splits, int keys_per_split, float scale, void* stream) {
  KSA_ENTER(q);
  KSA_REQUIRE(D == 128 || D == 64, "decode_attn: head_dim %d unsupported (64 or 128)", D);
  KSA_REQUIRE(Hq % Hkv == 0 && (Hq / Hkv) * Tq <= kDecMaxQ, "decode_attn: (Hq/Hkv) * Tq = %d exceeds %d queries per CTA",
              (Hq / Hkv) * Tq, kDecMaxQ);
  KSA_REQUIRE(splits >= 1 && keys_per_split >= 1, "decode_attn: bad split configuration");
  if (B == 0) return 0;
  DecodeArgs a{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (const int*)start, (const int*)len,
               (float*)part_o, (float*)part_ml, (bf16*)out, B, Tq, Hq, Hkv, D, cap, splits, keys_per_split, scale};
  dim3 grid(splits, Hkv, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) decode_attn_kernel<128><<<grid, kDecThreads, 0, st>>>(a);
  else decode_attn_kernel<64><<<grid, kDecThreads, 0, st>>>(a);
  KSA_CHECK_CUDA(cudaGetLastError());
  decode_combine_kernel<<<B * Tq * Hq, 128, 0, st>>>(a);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_kv_cache_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const void* slots,
                                int B, int T, int H, int D, int cap, long long src_row_stride,
                                long long src_batch_stride, void* stream) {
  KSA_ENTER(k_new);
  KSA_REQUIRE(D % 8 == 0, "kv_cache_append: head_dim must be a multiple of 8");
  const long long n = (long long)B * T * H * (D / 8);
  if (n == 0) return 0;
  kv_cache_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const bf16*)k_new, (const bf16*)v_new, (bf16*)k_cache, (bf16*)v_cache, (const int*)slots, B, T, H, D, cap,
      src_row_stride, src_batch_stride);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_kv_cache_move(void* k_cache, void* v_cache, const void* src, const void* dst, const void* enable, int B,
                              int H, int D, int cap, int rows, void* stream) {
  KSA_ENTER(k_cache);
  const long long n = (long long)B * H * rows * (D / 8);
  if (n == 0) return 0;
  kv_cache_move_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (bf16*)k_cache, (bf16*)v_cache, (const int*)src, (const int*)dst, (const int*)enable, B, H, D, cap, rows);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}
