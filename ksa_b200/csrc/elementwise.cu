// Memory-bound fused kernels: (residual add +) RMSNorm, per-head QK-RMSNorm + RoPE,
// SwiGLU, embedding gather / scatter-add, softmax cross-entropy with in-place
// gradient, AdamW on fp32 master state.  Each replaces an unfused ATen chain of the
// reference (muse/layers/rms_norm.py:67-80, muse/layers/position_embeddings.py:245-293,
// muse/layers/feed_forward.py:70-83, muse/losses/ce.py:32-140, torch.optim.AdamW).
// All of them move 16 bytes per thread per access and keep their statistics in fp32.
#include "common.cuh"
#include "host.h"

#include "vec.cuh"

namespace ksa {


// ------------------------------------------------------------------------------ RMSNorm
// One CTA of 256 threads per row; D <= 256 * 8 * kMaxVec.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // D up to 8192

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ delta, const bf16* __restrict__ w,
                   bf16* __restrict__ res_out, bf16* __restrict__ y, float* __restrict__ rstd_out, int rows, int D,
                   float eps, int delta_rows) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const bool has_delta = delta != nullptr && row < delta_rows;
  const long long base = (long long)row * D;
  float v[kNormMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int c = (i * kNormThreads + threadIdx.x) * 8;
    if (c < D) {
      load8(x + base + c, v[i]);
      if (has_delta) {
        float d[8];
        load8(delta + base + c, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += d[j];
        // round the residual stream to bf16 first so that norm and stream agree
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
      }
      if (res_out) store8(res_out + base + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = block_sum<kNormThreads>(ss, red);
  const float rstd = rsqrtf(ss / (float)D + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int c = (i * kNormThreads + threadIdx.x) * 8;
    if (c < D) {
      float wv[8], o[8];
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      store8(y + base + c, o);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres); per-CTA partial dw rows in `dw_partial`.
// NVEC 16-byte vectors per thread cover D <= NVEC * 2048; R rows are in flight per iteration so that enough
// loads are outstanding to hide DRAM latency, and their R row reductions share one pair of barriers.
template <int NVEC, int R>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const float* __restrict__ rstd_in, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int D) {
  __shared__ float red[R][8];
  float wv[NVEC][8];
  float dw[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * kNormThreads + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw[i][j] = 0.f; wv[i][j] = 0.f; }
    if (c < D) load8(w + c, wv[i]);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    float xh[R][NVEC][8], g[R][NVEC][8];
    BF8 rr_raw[R][NVEC];      // the residual gradient, requested with x and dy so that it arrives under the reduction
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
      const int row = row0 + r;
      const float rstd = row < rows ? rstd_in[row] : 0.f;
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * kNormThreads + threadIdx.x) * 8;
        if (row < rows && c < D) {
          float xv[8], dyv[8];
          if (dres) rr_raw[r][i] = *reinterpret_cast<const BF8*>(dres + (long long)row * D + c);
          load8(x + (long long)row * D + c, xv);
          load8(dy + (long long)row * D + c, dyv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            xh[r][i][j] = xv[j] * rstd;
            g[r][i][j] = dyv[j] * wv[i][j];
            dot[r] += g[r][i][j] * xh[r][i][j];
            dw[i][j] += dyv[j] * xh[r][i][j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { xh[r][i][j] = 0.f; g[r][i][j] = 0.f; }
        }
      }
      dot[r] = warp_sum(dot[r]);
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) red[r][warp] = dot[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < kNormThreads / 32; ++k) t += red[r][k];
      const float mean = t / (float)D;
      const int row = row0 + r;
      if (row >= rows) continue;
      const float rstd = rstd_in[row];
#pragma unroll
      for (int i = 0; i < NVEC; ++i) {
        const int c = (i * kNormThreads + threadIdx.x) * 8;
        if (c < D) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rstd * (g[r][i][j] - xh[r][i][j] * mean);
          if (dres) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = unpack_bf16x2(rr_raw[r][i].u[j]);
              o[2 * j] += t.x;
              o[2 * j + 1] += t.y;
            }
          }
          store8(dx + (long long)row * D + c, o);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = (i * kNormThreads + threadIdx.x) * 8;
    if (c < D) {
      float* p = dw_partial + (long long)blockIdx.x * D + c;
      *reinterpret_cast<float4*>(p) = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

// dw[c] (+)= sum over partial rows.  Block = 32 columns x 8 row groups.
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nparts, int D, int accumulate) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < D)
    for (int p = ty; p < nparts; p += 8) s += partial[(long long)p * D + c];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][tx];
    dw[c] = accumulate ? dw[c] + t : t;
  }
}

// ------------------------------------------------------------------------------ QK-norm + RoPE
// One warp per (row, head); head_dim = 128 (4 elements per lane) or 64 (2 per lane).
// Lane l owns rotary pairs (p, p + D/2) for p in [l*PAIRS, (l+1)*PAIRS).
struct QkRopeArgs {
  const bf16* qkv;       // [rows, in_stride] : q heads | k heads | v heads
  bf16* out;             // [rows, out_stride]: q heads | k heads
  const bf16* q_w;       // [D] or null (no q-norm)
  const bf16* k_w;       // [D] or null
  const int* pos;        // [rows]
  float* rstd;           // [rows, Hq+Hkv] (written in fwd, read in bwd)
  long long in_stride, out_stride;
  int rows, Hq, Hkv, D;
  float log2_theta, eps;
  int interleaved;       // 1: adjacent-pair (Llama) rotary, 0: half-split (HF)
  int copy_v;            // 1: also copy the v heads (input column block 3) to the output
};

template <int D>
__global__ void __launch_bounds__(256) qknorm_rope_fwd_kernel(QkRopeArgs a) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  constexpr int PAIRS = D / 64;  // rotary pairs per lane
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int H = a.Hq + a.Hkv;
  const int Hall = H + (a.copy_v ? a.Hkv : 0);
  if (warp_global >= a.rows * Hall) return;
  const int row = warp_global / Hall, head = warp_global % Hall;
  const bf16* src = a.qkv + (long long)row * a.in_stride + (long long)head * D;
  bf16* dst = a.out + (long long)row * a.out_stride + (long long)head * D;
  if (head >= H) {  // v head: plain copy
#pragma unroll
    for (int p = 0; p < PAIRS; ++p)
      reinterpret_cast<uint32_t*>(dst)[lane * PAIRS + p] = reinterpret_cast<const uint32_t*>(src)[lane * PAIRS + p];
    return;
  }
  const bf16* w = head < a.Hq ? a.q_w : a.k_w;
  float x1[PAIRS], x2[PAIRS];
  int i1[PAIRS], i2[PAIRS];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int pi = lane * PAIRS + p;
    i1[p] = a.interleaved ? 2 * pi : pi;
    i2[p] = a.interleaved ? 2 * pi + 1 : pi + D / 2;
    x1[p] = __bfloat162float(src[i1[p]]);
    x2[p] = __bfloat162float(src[i2[p]]);
    ss += x1[p] * x1[p] + x2[p] * x2[p];
  }
  float rstd = 1.f;
  if (w) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)D + a.eps);
  }
  if (lane == 0) a.rstd[(long long)row * H + head] = rstd;
  const float pos = (float)a.pos[row];
#pragma unroll
  for (int p = 0; p < PAIRS; ++p) {
    const int pi = lane * PAIRS + p;
    float n1 = x1[p] * rstd, n2 = x2[p] * rstd;
    if (w) {
      n1 *= __bfloat162float(w[i1[p]]);
      n2 *= __bfloat162float(w[i2[p]]);
    }
    const float inv_freq = exp2f(-a.log2_theta * (2.f * (float)pi / (float)D));
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    dst[i1[p]] = __float2bfloat16(n1 * c - n2 * s);
    dst[i2[p]] = __float2bfloat16(n2 * c + n1 * s);
  }
}

// Backward: d_out [rows, out_stride] -> d_qkv (q and k parts) [rows, in_stride]; dw accumulated with atomics.
struct QkRopeBwdArgs {
  QkRopeArgs f;          // forward arguments (qkv = pre-norm input, rstd = saved)
  const bf16* d_out;     // gradient w.r.t. rotated q | k
  bf16* d_qkv;           // gradient w.r.t. pre-norm q | k (packed layout, v part untouched)
  float* dq_w;           // [D] fp32, accumulated
  float* dk_w;           // [D] fp32, accumulated
};

template <int D>
__global__ void __launch_bounds__(256) qknorm_rope_bwd_kernel(QkRopeBwdArgs b) {
  constexpr int PAIRS = D / 64;
  const QkRopeArgs& a = b.f;
  __shared__ float s_dw[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&s_dw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int H = a.Hq + a.Hkv;
  const int Hall = H + (a.copy_v ? a.Hkv : 0);
  const int total = a.rows * Hall;
  for (int wg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wg < total; wg += gridDim.x * (blockDim.x >> 5)) {
    const int row = wg / Hall, head = wg % Hall;
    const bf16* src = a.qkv + (long long)row * a.in_stride + (long long)head * D;
    const bf16* g = b.d_out + (long long)row * a.out_stride + (long long)head * D;
    bf16* dst = b.d_qkv + (long long)row * a.in_stride + (long long)head * D;
    if (head >= H) {  // v head: the gradient passes through
#pragma unroll
      for (int p = 0; p < PAIRS; ++p)
        reinterpret_cast<uint32_t*>(dst)[lane * PAIRS + p] = reinterpret_cast<const uint32_t*>(g)[lane * PAIRS + p];
      continue;
    }
    const bf16* w = head < a.Hq ? a.q_w : a.k_w;
    const float rstd = a.rstd[(long long)row * H + head];
    const float pos = (float)a.pos[row];
    float xh1[PAIRS], xh2[PAIRS], gn1[PAIRS], gn2[PAIRS];
    int i1[PAIRS], i2[PAIRS];
    float dot = 0.f;
#pragma unroll
    for (int p = 0; p < PAIRS; ++p) {
      const int pi = lane * PAIRS + p;
      i1[p] = a.interleaved ? 2 * pi : pi;
      i2[p] = a.interleaved ? 2 * pi + 1 : pi + D / 2;
      const float inv_freq = exp2f(-a.log2_theta * (2.f * (float)pi / (float)D));
      float s, c;
      sincosf(pos * inv_freq, &s, &c);
      const float g1 = __bfloat162float(g[i1[p]]), g2 = __bfloat162float(g[i2[p]]);
      // transpose of the rotation
      float dn1 = g1 * c + g2 * s;
      float dn2 = g2 * c - g1 * s;
      xh1[p] = __bfloat162float(src[i1[p]]) * rstd;
      xh2[p] = __bfloat162float(src[i2[p]]) * rstd;
      if (w) {
        atomicAdd(&s_dw[head < a.Hq ? 0 : 1][i1[p]], dn1 * xh1[p]);
        atomicAdd(&s_dw[head < a.Hq ? 0 : 1][i2[p]], dn2 * xh2[p]);
        dn1 *= __bfloat162float(w[i1[p]]);
        dn2 *= __bfloat162float(w[i2[p]]);
      }
      gn1[p] = dn1;
      gn2[p] = dn2;
      dot += dn1 * xh1[p] + dn2 * xh2[p];
    }
    if (w) {
      dot = warp_sum(dot) / (float)D;
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) {
        dst[i1[p]] = __float2bfloat16(rstd * (gn1[p] - xh1[p] * dot));
        dst[i2[p]] = __float2bfloat16(rstd * (gn2[p] - xh2[p] * dot));
      }
    } else {
#pragma unroll
      for (int p = 0; p < PAIRS; ++p) {
        dst[i1[p]] = __float2bfloat16(gn1[p]);
        dst[i2[p]] = __float2bfloat16(gn2[p]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    if (b.dq_w && s_dw[0][i] != 0.f) atomicAdd(&b.dq_w[i], s_dw[0][i]);
    if (b.dk_w && s_dw[1][i] != 0.f) atomicAdd(&b.dk_w[i], s_dw[1][i]);
  }
}

// ---- head_dim 128: one warp per row walks all heads of the row.  A lane owns two 32-bit words A and B of every head
// (half-split rotary: elements {2l, 2l+1} and {2l+64, 2l+65}; interleaved: {4l, 4l+1} and {4l+2, 4l+3}), i.e. the
// rotary pairs with frequency indices 2l and 2l+1, whose sine / cosine are computed once per row.  Loads of four heads
// are in flight together.
struct RopeLane {
  int offA, offB;          // 32-bit word offsets inside a head
  float c0, s0, c1, s1;    // cos / sin of the two pairs
  float wq[4], wk[4];      // norm weights of this lane's 4 elements (q and k), 1 if there is no weight
};

__device__ __forceinline__ RopeLane rope_lane_setup(const QkRopeArgs& a, int row, int lane) {
  RopeLane r;
  r.offA = a.interleaved ? 2 * lane : lane;
  r.offB = a.interleaved ? 2 * lane + 1 : lane + 32;
  const float pos = (float)a.pos[row];
  const float f0 = exp2f(-a.log2_theta * (2.f * (float)(2 * lane) / 128.f));
  const float f1 = exp2f(-a.log2_theta * (2.f * (float)(2 * lane + 1) / 128.f));
  sincosf(pos * f0, &r.s0, &r.c0);
  sincosf(pos * f1, &r.s1, &r.c1);
#pragma unroll
  for (int i = 0; i < 4; ++i) { r.wq[i] = 1.f; r.wk[i] = 1.f; }
  if (a.q_w) {
    const float2 x = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.q_w)[r.offA]);
    const float2 y = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.q_w)[r.offB]);
    r.wq[0] = x.x; r.wq[1] = x.y; r.wq[2] = y.x; r.wq[3] = y.y;
  }
  if (a.k_w) {
    const float2 x = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.k_w)[r.offA]);
    const float2 y = unpack_bf16x2(reinterpret_cast<const uint32_t*>(a.k_w)[r.offB]);
    r.wk[0] = x.x; r.wk[1] = x.y; r.wk[2] = y.x; r.wk[3] = y.y;
  }
  return r;
}

// v = {A.lo, A.hi, B.lo, B.hi}; pair p rotates (v[i1], v[i2]) by the angle of frequency index 2l + p
template <bool IL>
__device__ __forceinline__ void rope_pair_idx(int p, int& i1, int& i2) {
  if (IL) { i1 = 2 * p; i2 = 2 * p + 1; }
  else { i1 = p; i2 = p + 2; }
}

template <bool IL>
__global__ void __launch_bounds__(256) qknorm_rope_fwd128_kernel(QkRopeArgs a) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= a.rows) return;
  const int H = a.Hq + a.Hkv;
  const int Hall = H + (a.copy_v ? a.Hkv : 0);
  const RopeLane r = rope_lane_setup(a, row, lane);
  const uint32_t* src = reinterpret_cast<const uint32_t*>(a.qkv + (long long)row * a.in_stride);
  uint32_t* dst = reinterpret_cast<uint32_t*>(a.out + (long long)row * a.out_stride);
  for (int h0 = 0; h0 < Hall; h0 += 4) {
    uint32_t ua[4], ub[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int head = min(h0 + u, Hall - 1);
      ua[u] = src[head * 64 + r.offA];
      ub[u] = src[head * 64 + r.offB];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int head = h0 + u;
      if (head >= Hall) break;
      if (head >= H) {      // v head: plain copy
        dst[head * 64 + r.offA] = ua[u];
        dst[head * 64 + r.offB] = ub[u];
        continue;
      }
      const float2 fa = unpack_bf16x2(ua[u]), fb = unpack_bf16x2(ub[u]);
      float v[4] = {fa.x, fa.y, fb.x, fb.y};
      float rstd = 1.f;
      const bool has_w = head < a.Hq ? a.q_w != nullptr : a.k_w != nullptr;
      if (has_w) {
        const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
        rstd = rsqrtf(ss / 128.f + a.eps);
      }
      if (lane == 0) a.rstd[(long long)row * H + head] = rstd;
      const float* w = head < a.Hq ? r.wq : r.wk;
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * w[i];
      float o[4];
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        int i1, i2;
        rope_pair_idx<IL>(p, i1, i2);
        const float c = p ? r.c1 : r.c0, sn = p ? r.s1 : r.s0;
        o[i1] = v[i1] * c - v[i2] * sn;
        o[i2] = v[i2] * c + v[i1] * sn;
      }
      dst[head * 64 + r.offA] = pack_bf16x2(o[0], o[1]);
      dst[head * 64 + r.offB] = pack_bf16x2(o[2], o[3]);
    }
  }
}

// A decode step has a handful of rows: one warp per (row, head) instead of one warp per row, v heads copied as well,
// and the new K / V rows of the first `cache_rows` rows written straight into the KV cache [B, Hkv, cap, 128] at
// slots[row] (row = sequence; negative slot: not cached).
struct QkRopeCacheArgs {
  bf16* k_cache;
  bf16* v_cache;
  const int* slots;
  int cache_rows, cap;
};

template <bool IL>
__global__ void __launch_bounds__(256) qknorm_rope_decode128_kernel(QkRopeArgs a, QkRopeCacheArgs c) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int H = a.Hq + a.Hkv, Hall = H + a.Hkv;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= a.rows * Hall) return;
  const int row = w / Hall, head = w - row * Hall;
  const int offA = a.interleaved ? 2 * lane : lane, offB = a.interleaved ? 2 * lane + 1 : lane + 32;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(a.qkv + (long long)row * a.in_stride) + head * 64;
  uint32_t* dst = reinterpret_cast<uint32_t*>(a.out + (long long)row * a.out_stride) + head * 64;
  uint32_t oa = src[offA], ob = src[offB];
  if (head < H) {
    const RopeLane r = rope_lane_setup(a, row, lane);
    const float2 fa = unpack_bf16x2(oa), fb = unpack_bf16x2(ob);
    float v[4] = {fa.x, fa.y, fb.x, fb.y};
    float rstd = 1.f;
    const bool has_w = head < a.Hq ? a.q_w != nullptr : a.k_w != nullptr;
    if (has_w) {
      const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
      rstd = rsqrtf(ss / 128.f + a.eps);
    }
    if (lane == 0 && a.rstd) a.rstd[(long long)row * H + head] = rstd;
    const float* wn = head < a.Hq ? r.wq : r.wk;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = v[i] * rstd * wn[i];
    float o[4];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      int i1, i2;
      rope_pair_idx<IL>(p, i1, i2);
      const float cs = p ? r.c1 : r.c0, sn = p ? r.s1 : r.s0;
      o[i1] = v[i1] * cs - v[i2] * sn;
      o[i2] = v[i2] * cs + v[i1] * sn;
    }
    oa = pack_bf16x2(o[0], o[1]);
    ob = pack_bf16x2(o[2], o[3]);
  }
  dst[offA] = oa;
  dst[offB] = ob;
  if (head >= a.Hq && c.k_cache != nullptr && row < c.cache_rows) {
    const int slot = c.slots[row];
    if (slot >= 0) {
      const bool is_v = head >= H;
      const int kh = is_v ? head - H : head - a.Hq;
      uint32_t* cd = reinterpret_cast<uint32_t*>(is_v ? c.v_cache : c.k_cache) +
                     (((long long)row * a.Hkv + kh) * c.cap + slot) * 64;
      cd[offA] = oa;
      cd[offB] = ob;
    }
  }
}

template <bool IL>
__global__ void __launch_bounds__(256) qknorm_rope_bwd128_kernel(QkRopeBwdArgs b) {
  const QkRopeArgs& a = b.f;
  __shared__ float s_dw[2][128];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) (&s_dw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int H = a.Hq + a.Hkv;
  const int Hall = H + (a.copy_v ? a.Hkv : 0);
  float dwq[4] = {0.f, 0.f, 0.f, 0.f}, dwk[4] = {0.f, 0.f, 0.f, 0.f};   // this lane's 4 elements, summed over rows
  int offA = 0, offB = 0;
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < a.rows; row += gridDim.x * (blockDim.x >> 5)) {
    const RopeLane r = rope_lane_setup(a, row, lane);
    offA = r.offA; offB = r.offB;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.qkv + (long long)row * a.in_stride);
    const uint32_t* g = reinterpret_cast<const uint32_t*>(b.d_out + (long long)row * a.out_stride);
    uint32_t* dst = reinterpret_cast<uint32_t*>(b.d_qkv + (long long)row * a.in_stride);
    for (int h0 = 0; h0 < Hall; h0 += 4) {
      uint32_t xa[4], xb[4], ga[4], gb[4];
      float rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int head = min(h0 + u, Hall - 1);
        ga[u] = g[head * 64 + r.offA];
        gb[u] = g[head * 64 + r.offB];
        xa[u] = head < H ? src[head * 64 + r.offA] : 0u;
        xb[u] = head < H ? src[head * 64 + r.offB] : 0u;
        rs[u] = head < H ? a.rstd[(long long)row * H + head] : 1.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int head = h0 + u;
        if (head >= Hall) break;
        if (head >= H) {    // v head: the gradient passes through
          dst[head * 64 + r.offA] = ga[u];
          dst[head * 64 + r.offB] = gb[u];
          continue;
        }
        const bool is_q = head < a.Hq;
        const bool has_w = is_q ? a.q_w != nullptr : a.k_w != nullptr;
        const float* w = is_q ? r.wq : r.wk;
        const float2 g0 = unpack_bf16x2(ga[u]), g1 = unpack_bf16x2(gb[u]);
        const float2 x0 = unpack_bf16x2(xa[u]), x1 = unpack_bf16x2(xb[u]);
        const float gv[4] = {g0.x, g0.y, g1.x, g1.y};
        const float xh[4] = {x0.x * rs[u], x0.y * rs[u], x1.x * rs[u], x1.y * rs[u]};
        float dn[4];
#pragma unroll
        for (int p = 0; p < 2; ++p) {   // transpose of the rotation
          int i1, i2;
          rope_pair_idx<IL>(p, i1, i2);
          const float c = p ? r.c1 : r.c0, sn = p ? r.s1 : r.s0;
          dn[i1] = gv[i1] * c + gv[i2] * sn;
          dn[i2] = gv[i2] * c - gv[i1] * sn;
        }
        float o[4];
        if (has_w) {
          float dot = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (is_q) dwq[i] += dn[i] * xh[i]; else dwk[i] += dn[i] * xh[i];
            dn[i] *= w[i];
            dot += dn[i] * xh[i];
          }
          dot = warp_sum(dot) / 128.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = rs[u] * (dn[i] - xh[i] * dot);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = dn[i];
        }
        dst[head * 64 + r.offA] = pack_bf16x2(o[0], o[1]);
        dst[head * 64 + r.offB] = pack_bf16x2(o[2], o[3]);
      }
    }
  }
  // this lane's elements: words offA, offB -> elements 2*offA, 2*offA+1, 2*offB, 2*offB+1
  atomicAdd(&s_dw[0][2 * offA], dwq[0]); atomicAdd(&s_dw[0][2 * offA + 1], dwq[1]);
  atomicAdd(&s_dw[0][2 * offB], dwq[2]); atomicAdd(&s_dw[0][2 * offB + 1], dwq[3]);
  atomicAdd(&s_dw[1][2 * offA], dwk[0]); atomicAdd(&s_dw[1][2 * offA + 1], dwk[1]);
  atomicAdd(&s_dw[1][2 * offB], dwk[2]); atomicAdd(&s_dw[1][2 * offB + 1], dwk[3]);
  __syncthreads();
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    if (b.dq_w && s_dw[0][i] != 0.f) atomicAdd(&b.dq_w[i], s_dw[0][i]);
    if (b.dk_w && s_dw[1][i] != 0.f) atomicAdd(&b.dk_w[i], s_dw[1][i]);
  }
}

// ------------------------------------------------------------------------------ SwiGLU
// gate_up is [rows, 2F] = [gate | up]; out is [rows, F].
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long long rows, int F) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = F / 8;
  if (vec >= rows * per_row) return;
  const long long row = vec / per_row;
  const int c = (int)(vec % per_row) * 8;
  float g[8], u[8], o[8];
  load8(gu + row * 2 * F + c, g);
  load8(gu + row * 2 * F + F + c, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  store8(out + row * F + c, o);
}
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dout, bf16* __restrict__ dgu, long long rows,
                  int F) {
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = F / 8;
  if (vec >= rows * per_row) return;
  const long long row = vec / per_row;
  const int c = (int)(vec % per_row) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  load8(gu + row * 2 * F + c, g);
  load8(gu + row * 2 * F + F + c, u);
  load8(dout + row * F + c, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = 1.f / (1.f + __expf(-g[j]));
    const float silu = g[j] * sig;
    du[j] = d[j] * silu;
    dg[j] = d[j] * u[j] * sig * (1.f + g[j] * (1.f - sig));
  }
  store8(dgu + row * 2 * F + c, dg);
  store8(dgu + row * 2 * F + F + c, du);
}

// ------------------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ out,
                     long long rows, int D, long long vocab) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = D / 8;
  if (vec >= rows * per_row) return;
  const long long row = vec / per_row;
  const int c = (int)(vec % per_row) * 8;
  long long id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  *reinterpret_cast<BF8*>(out + row * D + c) = *reinterpret_cast<const BF8*>(table + id * D + c);
}
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dout, float* __restrict__ dtable,
                     long long rows, int D, long long vocab) {
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = D / 8;
  if (vec >= rows * per_row) return;
  const long long row = vec / per_row;
  const int c = (int)(vec % per_row) * 8;
  long long id = ids[row];
  if (id < 0 || id >= vocab) return;
  float g[8];
  load8(dout + row * D + c, g);
  float* dst = dtable + id * D + c;
#pragma unroll
  for (int j = 0; j < 8; ++j) atomicAdd(dst + j, g[j]);
}

// ------------------------------------------------------------------------------ cross entropy
// One CTA per row of bf16 logits [rows, V].  Writes per-row loss (0 for ignored rows) and turns the
// logits into d(loss)/d(logits) * (*grad_scale) in place.
constexpr int kCeThreads = 512;
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_loss,
                     const float* __restrict__ grad_scale, int V, long long ld, int ignore_index, int write_grad) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  bf16* lg = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int nvec = V / 8;
  if (ignored) {
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    if (write_grad) {
      BF8 z{{0, 0, 0, 0}};
      for (int i = threadIdx.x; i < nvec; i += kCeThreads) *reinterpret_cast<BF8*>(lg + i * 8) = z;
    }
    return;
  }
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float f[8];
    load8(lg + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
  }
  mx = block_max<kCeThreads>(mx, red);
  float sum = 0.f;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float f[8];
    load8(lg + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += __expf(f[j] - mx);
  }
  sum = block_sum<kCeThreads>(sum, red);
  const float lse = mx + __logf(sum);
  if (threadIdx.x == 0) row_loss[row] = lse - __bfloat162float(lg[label]);
  if (!write_grad) return;
  __syncthreads();
  const float gs = *grad_scale;
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float f[8];
    load8(lg + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - mx) * inv;
      if ((long long)i * 8 + j == label) p -= 1.f;
      f[j] = p * gs;
    }
    store8(lg + i * 8, f);
  }
}

// n_valid and 1/n_valid (times an extra scale) on the device: no host sync in the step.
__global__ void count_valid_kernel(const long long* __restrict__ labels, long long n, int ignore_index, float extra_scale,
                                   float* __restrict__ out /* [0]=count, [1]=extra/count */) {
  __shared__ float red[32];
  float c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += (labels[i] != ignore_index) ? 1.f : 0.f;
  c = block_sum<1024>(c, red);
  if (threadIdx.x == 0) {
    out[0] = c;
    out[1] = extra_scale / fmaxf(c, 1.f);
  }
}

// ------------------------------------------------------------------------------ AdamW
// hyper[0]=lr, [1]=1-beta1^t, [2]=1-beta2^t, [3]=gradient scale; read from device memory so that a
// captured CUDA graph stays valid while the schedule advances.
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
             bf16* __restrict__ out_bf16, long long n, const float* __restrict__ hyper, float beta1, float beta2,
             float eps, float weight_decay, float clip_value, float* __restrict__ sumsq) {
  __shared__ float red[32];
  const float lr = hyper[0], bc1 = hyper[1], bc2 = hyper[2], gscale = hyper[3];
  float sq = 0.f;
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float g[4] = {g4.x, g4.y, g4.z, g4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w},
          vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gscale;
      if (clip_value > 0.f) gj = fminf(fmaxf(gj, -clip_value), clip_value);
      sq += gj * gj;   // norm of the clipped gradients: the reference clips first (recipes/pretrain_kai_summary_unified.py:1045-1049)
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      const float denom = sqrtf(vv[j] / bc2) + eps;
      p[j] = p[j] * (1.f - lr * weight_decay) - lr * (mm[j] / bc1) / denom;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (out_bf16) {
      uint2 o = make_uint2(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]));
      reinterpret_cast<uint2*>(out_bf16)[i] = o;
    }
  }
  if (sumsq) {
    sq = block_sum<256>(sq, red);
    if (threadIdx.x == 0) atomicAdd(sumsq, sq);
  }
}

// fp32 -> bf16 cast (flat), used to refresh compute weights from master weights.
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long long n) {
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w));
  }
}

}  // namespace ksa

using namespace ksa;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// delta (optional) covers the first delta_rows rows only; res_out (optional) receives x (+ delta) for every row.
KSA_API int ksa_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* res_out, void* y, void* rstd,
                            int rows, int D, float eps, int delta_rows, void* stream) {
  KSA_ENTER(x);
  KSA_REQUIRE(D % 8 == 0 && D <= kNormThreads * 8 * kNormMaxVec, "rmsnorm: D=%d must be a multiple of 8 and <= %d", D,
              kNormThreads * 8 * kNormMaxVec);
  if (rows == 0) return 0;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), rmsnorm_fwd_kernel, dim3(rows), dim3(kNormThreads), 0,
                              ST(stream), (const bf16*)x, (const bf16*)delta, (const bf16*)w, (bf16*)res_out, (bf16*)y,
                              (float*)rstd, rows, D, eps, delta_rows));
  return 0;
}

// Number of partial rows the backward writes: the caller sizes `dw_partial` as [ksa_rmsnorm_bwd_parts(rows), D] fp32.
KSA_API int ksa_rmsnorm_bwd_parts(int rows) { return rows < 592 ? (rows > 0 ? rows : 1) : 592; }

template <int NVEC, int R>
static int launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres,
                              void* dx, void* dw_partial, int parts, int rows, int D, cudaStream_t st) {
  int blocks = (rows + R - 1) / R;
  if (blocks > parts) blocks = parts;
  // rows beyond `blocks` partial rows stay untouched; zero-fill is not needed because colsum reads `blocks` rows only
  rmsnorm_bwd_kernel<NVEC, R><<<blocks, kNormThreads, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w,
                                                               (const float*)rstd, (const bf16*)dres, (bf16*)dx,
                                                               (float*)dw_partial, rows, D);
  KSA_CHECK_CUDA(cudaGetLastError());
  return blocks;
}

KSA_API int ksa_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres, void* dx,
                            void* dw_partial, void* dw, int accumulate_dw, int rows, int D, void* stream) {
  KSA_ENTER(dy);
  KSA_REQUIRE(D % 8 == 0 && D <= kNormThreads * 8 * kNormMaxVec, "rmsnorm: D=%d unsupported", D);
  if (rows == 0) return 0;
  const int parts = ksa_rmsnorm_bwd_parts(rows);
  int used;
  if (D <= 2048) used = launch_rmsnorm_bwd<1, 4>(dy, x, w, rstd, dres, dx, dw_partial, parts, rows, D, ST(stream));
  else if (D <= 4096) used = launch_rmsnorm_bwd<2, 2>(dy, x, w, rstd, dres, dx, dw_partial, parts, rows, D, ST(stream));
  else used = launch_rmsnorm_bwd<4, 1>(dy, x, w, rstd, dres, dx, dw_partial, parts, rows, D, ST(stream));
  if (used < 0) return used;
  if (dw) {
    colsum_partials_kernel<<<(D + 31) / 32, 256, 0, ST(stream)>>>((const float*)dw_partial, (float*)dw, used, D,
                                                                  accumulate_dw);
    KSA_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
}

KSA_API int ksa_qknorm_rope_fwd(const void* qkv, void* out, const void* q_w, const void* k_w, const void* pos,
                                void* rstd, long long in_stride, long long out_stride, int rows, int Hq, int Hkv, int D,
                                float theta, float eps, int interleaved, int copy_v, void* stream) {
  KSA_ENTER(qkv);
  KSA_REQUIRE(D == 128 || D == 64, "qknorm_rope: head_dim %d unsupported (64 or 128)", D);
  if (rows == 0) return 0;
  QkRopeArgs a{(const bf16*)qkv, (bf16*)out, (const bf16*)q_w, (const bf16*)k_w, (const int*)pos, (float*)rstd,
               in_stride, out_stride, rows, Hq, Hkv, D, log2f(theta), eps, interleaved, copy_v};
  const long long warps = (long long)rows * (Hq + Hkv + (copy_v ? Hkv : 0));
  const int blocks = (int)((warps + 7) / 8);
  const bool dep = dependent_launch_enabled();
  if (D == 128 && interleaved)
    KSA_CHECK_CUDA(launch_kernel(dep, qknorm_rope_fwd128_kernel<true>, dim3((rows + 7) / 8), dim3(256), 0, ST(stream), a));
  else if (D == 128)
    KSA_CHECK_CUDA(launch_kernel(dep, qknorm_rope_fwd128_kernel<false>, dim3((rows + 7) / 8), dim3(256), 0, ST(stream), a));
  else
    KSA_CHECK_CUDA(launch_kernel(dep, qknorm_rope_fwd_kernel<64>, dim3(blocks), dim3(256), 0, ST(stream), a));
  return 0;
}

// QK-norm + RoPE for the few rows of a decode step (head_dim 128): q | k | v rows -> out (same layout, v copied), and
// K / V of rows [0, cache_rows) also into the KV cache [B, Hkv, cap, 128] at slots[row] (k_cache null: no cache).
KSA_API int ksa_qknorm_rope_decode(const void* qkv, void* out, const void* q_w, const void* k_w, const void* pos,
                                   long long in_stride, long long out_stride, int rows, int Hq, int Hkv, int D,
                                   float theta, float eps, int interleaved, void* k_cache, void* v_cache,
                                   const void* slots, int cache_rows, int cap, void* stream) {
  KSA_ENTER(qkv);
  KSA_REQUIRE(D == 128, "qknorm_rope_decode: head_dim %d unsupported (128)", D);
  KSA_REQUIRE(k_cache == nullptr || (v_cache != nullptr && slots != nullptr && cache_rows <= rows && cap > 0),
              "qknorm_rope_decode: cache arguments are incomplete");
  if (rows == 0) return 0;
  QkRopeArgs a{(const bf16*)qkv, (bf16*)out, (const bf16*)q_w, (const bf16*)k_w, (const int*)pos, nullptr,
               in_stride, out_stride, rows, Hq, Hkv, D, log2f(theta), eps, interleaved, 1};
  QkRopeCacheArgs c{(bf16*)k_cache, (bf16*)v_cache, (const int*)slots, cache_rows, cap};
  const int warps = rows * (Hq + 2 * Hkv);
  const bool dep = dependent_launch_enabled();
  if (interleaved)
    KSA_CHECK_CUDA(launch_kernel(dep, qknorm_rope_decode128_kernel<true>, dim3((warps + 7) / 8), dim3(256), 0, ST(stream), a, c));
  else
    KSA_CHECK_CUDA(launch_kernel(dep, qknorm_rope_decode128_kernel<false>, dim3((warps + 7) / 8), dim3(256), 0, ST(stream), a, c));
  return 0;
}

KSA_API int ksa_qknorm_rope_bwd(const void* qkv, const void* d_out, void* d_qkv, const void* q_w, const void* k_w,
                                const void* pos, const void* rstd, void* dq_w, void* dk_w, long long in_stride,
                                long long out_stride, int rows, int Hq, int Hkv, int D, float theta, float eps,
                                int interleaved, int copy_v, void* stream) {
  KSA_ENTER(qkv);
  KSA_REQUIRE(D == 128 || D == 64, "qknorm_rope: head_dim %d unsupported (64 or 128)", D);
  if (rows == 0) return 0;
  QkRopeBwdArgs b{{(const bf16*)qkv, nullptr, (const bf16*)q_w, (const bf16*)k_w, (const int*)pos, (float*)rstd,
                   in_stride, out_stride, rows, Hq, Hkv, D, log2f(theta), eps, interleaved, copy_v},
                  (const bf16*)d_out, (bf16*)d_qkv, (float*)dq_w, (float*)dk_w};
  const long long warps = (long long)rows * (Hq + Hkv + (copy_v ? Hkv : 0));
  long long blocks = (warps + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (D == 128) {
    int rb = (rows + 7) / 8;
    if (rb > 148 * 8) rb = 148 * 8;
    if (interleaved) qknorm_rope_bwd128_kernel<true><<<rb, 256, 0, ST(stream)>>>(b);
    else qknorm_rope_bwd128_kernel<false><<<rb, 256, 0, ST(stream)>>>(b);
  } else {
    qknorm_rope_bwd_kernel<64><<<(int)blocks, 256, 0, ST(stream)>>>(b);
  }
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_swiglu_fwd(const void* gu, void* out, long long rows, int F, void* stream) {
  KSA_ENTER(gu);
  KSA_REQUIRE(F % 8 == 0, "swiglu: F=%d must be a multiple of 8", F);
  const long long n = rows * (F / 8);
  if (n == 0) return 0;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), swiglu_fwd_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256),
                              0, ST(stream), (const bf16*)gu, (bf16*)out, rows, F));
  return 0;
}
KSA_API int ksa_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int F, void* stream) {
  KSA_ENTER(gu);
  KSA_REQUIRE(F % 8 == 0, "swiglu: F=%d must be a multiple of 8", F);
  const long long n = rows * (F / 8);
  if (n == 0) return 0;
  swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(stream)>>>((const bf16*)gu, (const bf16*)dout, (bf16*)dgu,
                                                                        rows, F);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_embedding_fwd(const void* ids, const void* table, void* out, long long rows, int D, long long vocab,
                              void* stream) {
  KSA_ENTER(ids);
  KSA_REQUIRE(D % 8 == 0, "embedding: D=%d must be a multiple of 8", D);
  const long long n = rows * (D / 8);
  if (n == 0) return 0;
  KSA_CHECK_CUDA(launch_kernel(dependent_launch_enabled(), embedding_fwd_kernel, dim3((unsigned)((n + 255) / 256)),
                              dim3(256), 0, ST(stream), (const long long*)ids, (const bf16*)table, (bf16*)out, rows, D,
                              vocab));
  return 0;
}
KSA_API int ksa_embedding_bwd(const void* ids, const void* dout, void* dtable_f32, long long rows, int D,
                              long long vocab, void* stream) {
  KSA_ENTER(ids);
  KSA_REQUIRE(D % 8 == 0, "embedding: D=%d must be a multiple of 8", D);
  const long long n = rows * (D / 8);
  if (n == 0) return 0;
  embedding_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(stream)>>>((const long long*)ids, (const bf16*)dout,
                                                                           (float*)dtable_f32, rows, D, vocab);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_count_valid(const void* labels, long long n, int ignore_index, float extra_scale, void* out2,
                            void* stream) {
  KSA_ENTER(labels);
  count_valid_kernel<<<1, 1024, 0, ST(stream)>>>((const long long*)labels, n, ignore_index, extra_scale, (float*)out2);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_cross_entropy(void* logits, const void* labels, void* row_loss, const void* grad_scale, long long rows,
                              int V, long long ld, int ignore_index, int write_grad, void* stream) {
  KSA_ENTER(logits);
  KSA_REQUIRE(V % 8 == 0 && ld % 8 == 0, "cross_entropy: V=%d and ld=%lld must be multiples of 8", V, ld);
  if (rows == 0) return 0;
  cross_entropy_kernel<<<(unsigned)rows, kCeThreads, 0, ST(stream)>>>((bf16*)logits, (const long long*)labels,
                                                                     (float*)row_loss, (const float*)grad_scale, V, ld,
                                                                     ignore_index, write_grad);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_adamw(void* master, const void* grad, void* m, void* v, void* out_bf16, long long n, const void* hyper,
                      float beta1, float beta2, float eps, float weight_decay, float clip_value, void* sumsq,
                      void* stream) {
  KSA_ENTER(master);
  KSA_REQUIRE(n % 4 == 0, "adamw: n=%lld must be a multiple of 4 (pad the flat buffer)", n);
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>((float*)master, (const float*)grad, (float*)m, (float*)v,
                                                        (bf16*)out_bf16, n, (const float*)hyper, beta1, beta2, eps,
                                                        weight_decay, clip_value, (float*)sumsq);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

KSA_API int ksa_cast_f32_bf16(const void* src, void* dst, long long n, void* stream) {
  KSA_ENTER(src);
  KSA_REQUIRE(n % 4 == 0, "cast: n=%lld must be a multiple of 4", n);
  if (n == 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cast_f32_bf16_kernel<<<(unsigned)blocks, 256, 0, ST(stream)>>>((const float*)src, (bf16*)dst, n);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}
