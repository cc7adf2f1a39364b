// Device routines for communication over peer memory, shared by the standalone kernels (comm.cu) and by the
// communication CTAs / communication warps of the GEMM kernels (gemm.cu, gemm2.cu).  Two transports:
//   * plain P2P loads/stores of 16 bytes per thread through pointers into other GPUs' memory (weak loads ordered after
//     a system-scope acquire of the producer's flag; no read-only/non-coherent path, since the same addresses are
//     rewritten every step);
//   * untiled bulk copies driven by one thread (peer memory -> shared-memory ring -> own memory), for a spare warp of
//     a CTA whose other warps do tensor-core work.
// Waits on peer-written flags and on the copy ring's barriers are bounded.
#pragma once
#include "common.cuh"

namespace ksa {

constexpr int kMaxPeers = 8;
constexpr int kCommThreads = 512;

struct GatherJob {
  const uint8_t* peers[kMaxPeers];  // every rank's copy of the flat buffer; peers[rank] is the local (destination) copy
  int world, rank;
  long long shard_bytes;
  const uint32_t* ready_flags;  // optional, own memory: shard r may be read once ready_flags[r] >= target
  const uint32_t* epoch_ptr;    // target = (epoch_ptr ? *epoch_ptr : 0) + epoch_add; a device-resident epoch keeps
  uint32_t epoch_add;           // a captured CUDA graph valid from step to step
  int max_segs;                 // bulk gather only: most segments a shard is reported in (1..kBulkSegs)
  uint32_t* done;               // optional, own memory: bulk gather only, kMaxPeers x kBulkSegs counters (zero at
                                // launch): done[r * kBulkSegs + g] += chunks of segment g of shard r that have landed
};

struct ReduceAdamwJob {
  const float* grads[kMaxPeers];  // every rank's full fp32 gradient buffer of the unit
  int world, rank;
  long long shard_lo, n;          // this rank owns elements [shard_lo, shard_lo + n)
  float* master; float* m; float* v;  // this rank's shard state
  bf16* out_bf16;                 // own full compute buffer (written at shard_lo + i), may be null
  const float* hyper;             // [lr, 1-beta1^t, 1-beta2^t, grad_scale]
  float beta1, beta2, eps, weight_decay, clip_value;
  float* sumsq;                   // optional accumulator of sum(g^2) over the shard
  const uint32_t* ready_flags;    // optional, own memory: all `world` flags must reach the target first
  const uint32_t* epoch_ptr;      // target = (epoch_ptr ? *epoch_ptr : 0) + epoch_add
  uint32_t epoch_add;
};

struct SignalTargets {
  uint32_t* ptr[kMaxPeers];
  int n;
};

__device__ __forceinline__ uint32_t epoch_target(const uint32_t* epoch_ptr, uint32_t add) {
  return (epoch_ptr ? *reinterpret_cast<const volatile uint32_t*>(epoch_ptr) : 0u) + add;
}

__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// CTA `cta` of `nctas` copies its slice of every remote shard.  Returns false if a flag wait timed out.
__device__ __forceinline__ bool run_gather_job(const GatherJob& j, int cta, int nctas, int* status) {
  __shared__ int s_ok;
  const long long vecs = j.shard_bytes / 16;
  uint8_t* dst_base = const_cast<uint8_t*>(j.peers[j.rank]);
  const uint32_t target = epoch_target(j.epoch_ptr, j.epoch_add);
  for (int step = 1; step < j.world; ++step) {
    const int r = (j.rank + step) % j.world;  // start with the next rank so that ranks do not all hit one peer at once
    if (!KSA_DEV_CHECK(r >= 0 && r < kMaxPeers && j.peers[r] != nullptr && (j.shard_bytes & 15) == 0, status)) return false;
    if (j.ready_flags) {
      if (threadIdx.x == 0) s_ok = flag_wait_ge(j.ready_flags + r, target, status, kTimeoutPeerFlag, true) ? 1 : 0;
      __syncthreads();
      const int ok = s_ok;
      __syncthreads();
      if (!ok) return false;
    }
    const uint8_t* src = j.peers[r] + (long long)r * j.shard_bytes;
    uint8_t* dst = dst_base + (long long)r * j.shard_bytes;
    const long long stride = (long long)nctas * blockDim.x;
    long long i = (long long)cta * blockDim.x + threadIdx.x;
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * stride < vecs; i += 4 * stride) {
      const uint4 a = ld_peer_16(src + i * 16), b = ld_peer_16(src + (i + stride) * 16);
      const uint4 c = ld_peer_16(src + (i + 2 * stride) * 16), d = ld_peer_16(src + (i + 3 * stride) * 16);
      *reinterpret_cast<uint4*>(dst + i * 16) = a;
      *reinterpret_cast<uint4*>(dst + (i + stride) * 16) = b;
      *reinterpret_cast<uint4*>(dst + (i + 2 * stride) * 16) = c;
      *reinterpret_cast<uint4*>(dst + (i + 3 * stride) * 16) = d;
    }
    for (; i < vecs; i += stride) *reinterpret_cast<uint4*>(dst + i * 16) = ld_peer_16(src + i * 16);
  }
  return true;
}

// ----------------------------------------------------------------------------------------------
// The same gather driven by the copy engine of the SM instead of by load/store instructions, for use by ONE spare
// thread of a CTA whose other warps do tensor-core work: untiled bulk copies peer memory -> small shared-memory ring ->
// own memory.  A single SM copies about 40 GB/s this way (measured: 8 CTAs doing nothing else moved 320 GB/s, 12 moved
// 440 GB/s, whatever the ring's shape), so the transfer is spread over every CTA of the launch, a few GB/s each,
// instead of taking whole SMs away from the math.  Both addresses of every copy are 16-byte aligned and every size is
// a multiple of 16 bytes (shard_bytes and the chunk size are).
constexpr int kBulkChunk = 8192;
constexpr int kBulkStages = 4;
constexpr int kBulkRingBytes = kBulkStages * kBulkChunk + 64;   // + the ring's mbarriers and its abort flag

// A shard is moved and reported in up to kBulkSegs segments of (almost) equal numbers of chunks, so that a consumer of
// the first rows of a shard does not wait for its last ones.  Leaving a segment costs the copying thread a full wait
// for its stores, so a shard is only split while every CTA still moves kBulkMinPerSeg chunks or more per segment.
constexpr int kBulkSegs = 4;
constexpr int kBulkMinPerSeg = 12;

__host__ __device__ constexpr long long bulk_chunks(long long shard_bytes) {
  return (shard_bytes + kBulkChunk - 1) / kBulkChunk;
}
// segments a shard of n_chunks is split into when nctas CTAs move it (at most max_segs <= kBulkSegs)
__host__ __device__ constexpr int bulk_segs(long long n_chunks, int nctas, int max_segs) {
  const long long g = n_chunks / ((long long)nctas * kBulkMinPerSeg);
  return g < 1 ? 1 : (g > max_segs ? max_segs : (int)g);
}
// first chunk of segment g of `segs` (g = segs gives the number of chunks)
__host__ __device__ constexpr long long bulk_seg_begin(long long n_chunks, int segs, int g) {
  return (n_chunks * g + segs - 1) / segs;
}
// segment that chunk c belongs to: the largest g with bulk_seg_begin(g) <= c
__host__ __device__ constexpr int bulk_seg_of(long long n_chunks, int segs, long long c) {
  int g = (int)(c * segs / n_chunks);
  while (g + 1 < segs && bulk_seg_begin(n_chunks, segs, g + 1) <= c) ++g;
  while (g > 0 && bulk_seg_begin(n_chunks, segs, g) > c) --g;
  return g;
}

__device__ __forceinline__ void bulk_load_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_wait_read_all_but_one() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// writes of the copy engine (async proxy) ordered before later generic-proxy accesses and the other way round
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Called by ONE thread.  CTA `cta` of `nctas` moves chunks cta, cta + nctas, ... of every remote shard through `ring`
// (16-byte aligned shared memory of kBulkRingBytes that nobody else touches) and, whenever it leaves a segment of a
// shard, adds the number of chunks of that segment it has written to done[r * kBulkSegs + segment]: the segment is
// complete when the counter has reached bulk_seg_begin(n, segs, g + 1) - bulk_seg_begin(n, segs, g), with
// segs = bulk_segs(n, nctas, max_segs).
// Chunks are numbered in the order this CTA moves them, across shards: chunk n uses stage n % kBulkStages and the
// (n / kBulkStages)-th phase of that stage's barrier.  Returns false if a wait gave up; nothing is left in flight
// either way.
__device__ __forceinline__ bool run_gather_job_bulk(const GatherJob& j, int cta, int nctas, uint8_t* ring, int* status) {
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kBulkStages * kBulkChunk);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kBulkStages);
  for (int s = 0; s < kBulkStages; ++s) mbar_init(&bars[s], 1);
  *abort_flag = 0;
  fence_mbar_init();
  const WaitGuard guard{abort_flag, status};
  uint8_t* dst_base = const_cast<uint8_t*>(j.peers[j.rank]);
  const uint32_t target = epoch_target(j.epoch_ptr, j.epoch_add);
  const long long n_chunks = bulk_chunks(j.shard_bytes);
  const int segs = bulk_segs(n_chunks, nctas, j.max_segs);
  long long issued = 0;    // loads issued
  long long stored = 0;    // stores issued
  long long freed = 0;     // stores known to have finished reading their stage
  bool ok = true;
  for (int step = 1; step < j.world && ok; ++step) {
    const int r = (j.rank + step) % j.world;
    if (!KSA_DEV_CHECK(r >= 0 && r < kMaxPeers && j.peers[r] != nullptr && (j.shard_bytes & 15) == 0, status)) { ok = false; break; }
    if (j.ready_flags && !flag_wait_ge(j.ready_flags + r, target, status, kTimeoutPeerFlag, true)) { ok = false; break; }
    const uint8_t* src = j.peers[r] + (long long)r * j.shard_bytes;
    uint8_t* dst = dst_base + (long long)r * j.shard_bytes;
    long long next_load = cta, next_store = cta;
    uint32_t moved = 0;                                   // chunks of segment `seg` stored by this CTA
    int seg = next_store < n_chunks ? bulk_seg_of(n_chunks, segs, next_store) : 0;
    while (next_store < n_chunks) {
      while (next_load < n_chunks && issued - freed < kBulkStages) {
        const int s = (int)(issued % kBulkStages);
        const long long off = next_load * kBulkChunk;
        const uint32_t bytes = (uint32_t)min((long long)kBulkChunk, j.shard_bytes - off);
        mbar_expect_tx(&bars[s], bytes);
        bulk_load_g2s(ring + s * kBulkChunk, src + off, bytes, &bars[s]);
        ++issued;
        next_load += nctas;
      }
      const int s = (int)(stored % kBulkStages);
      if (!mbar_wait(&bars[s], (uint32_t)((stored / kBulkStages) & 1), guard, kTimeoutTmaFull)) { ok = false; break; }
      const long long off = next_store * kBulkChunk;
      const uint32_t bytes = (uint32_t)min((long long)kBulkChunk, j.shard_bytes - off);
      fence_proxy_async();
      bulk_store_s2g(dst + off, ring + s * kBulkChunk, bytes);
      tma_store_commit();
      ++stored;
      ++moved;
      next_store += nctas;
      const bool leaves = next_store >= n_chunks || next_store >= bulk_seg_begin(n_chunks, segs, seg + 1);
      if (!leaves) {
        bulk_wait_read_all_but_one();   // every store but the newest has read its stage: those stages may be refilled
        freed = stored - 1;
      } else {
        tma_store_wait0();              // this CTA's part of the segment is written: report it
        freed = stored;
        if (j.done) {
          fence_proxy_async_all();
          __threadfence();
          red_release_gpu_add(j.done + r * kBulkSegs + seg, moved);
        }
        moved = 0;
        if (next_store < n_chunks) seg = bulk_seg_of(n_chunks, segs, next_store);
      }
    }
    if (!ok) break;
  }
  if (!ok) {
    // give loads that are still in flight a bounded time to land (their destination is this CTA's shared memory)
    for (long long n = stored; n < issued; ++n) {
      const int s = (int)(n % kBulkStages);
      const uint32_t parity = (uint32_t)((n / kBulkStages) & 1);
      for (int spin = 0; spin < (1 << 22) && !mbar_try_wait(&bars[s], parity); ++spin) {}
    }
    tma_store_wait0();
  }
  return ok;
}

// CTA `cta` of `nctas` reduces + updates its slice of the owned shard.
__device__ __forceinline__ bool run_reduce_adamw_job(const ReduceAdamwJob& j, int cta, int nctas, int* status) {
  __shared__ int s_ok;
  __shared__ float s_red[32];
  if (j.ready_flags) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < j.world &&
        !flag_wait_ge(j.ready_flags + threadIdx.x, epoch_target(j.epoch_ptr, j.epoch_add), status, kTimeoutPeerFlag, true))
      s_ok = 0;
    __syncthreads();
    if (!s_ok) return false;
  }
  const float lr = j.hyper[0], bc1 = j.hyper[1], bc2 = j.hyper[2], gscale = j.hyper[3];
  const long long nvec = j.n / 4;
  float sq = 0.f;
  constexpr int U = 2;  // vectors per thread per iteration: all peer loads of both are issued before any is used
  const long long stride = (long long)nctas * blockDim.x;
  for (long long i0 = (long long)cta * blockDim.x + threadIdx.x; i0 < nvec; i0 += U * stride) {
    float4 g[U], p4[U], m4[U], v4[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
        const long long e = j.shard_lo + i * 4;
        g[u] = ld_peer_f4(j.grads[j.rank] + e);
        p4[u] = reinterpret_cast<float4*>(j.master)[i];
        m4[u] = reinterpret_cast<float4*>(j.m)[i];
        v4[u] = reinterpret_cast<float4*>(j.v)[i];
      }
    }
#pragma unroll
    for (int s = 1; s < kMaxPeers; ++s) {
      if (s < j.world) {
        const int r = (j.rank + s) % j.world;
        float4 t[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < nvec) t[u] = ld_peer_f4(j.grads[r] + j.shard_lo + i * 4);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * stride < nvec) { g[u].x += t[u].x; g[u].y += t[u].y; g[u].z += t[u].z; g[u].w += t[u].w; }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      const long long e = j.shard_lo + i * 4;
      float gg[4] = {g[u].x, g[u].y, g[u].z, g[u].w}, p[4] = {p4[u].x, p4[u].y, p4[u].z, p4[u].w},
            mm[4] = {m4[u].x, m4[u].y, m4[u].z, m4[u].w}, vv[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float gk = gg[k] * gscale;
        if (j.clip_value > 0.f) gk = fminf(fmaxf(gk, -j.clip_value), j.clip_value);
        sq += gk * gk;   // norm of the clipped gradients, as in adamw_kernel
        mm[k] = j.beta1 * mm[k] + (1.f - j.beta1) * gk;
        vv[k] = j.beta2 * vv[k] + (1.f - j.beta2) * gk * gk;
        const float denom = sqrtf(vv[k] / bc2) + j.eps;
        p[k] = p[k] * (1.f - lr * j.weight_decay) - lr * (mm[k] / bc1) / denom;
      }
      reinterpret_cast<float4*>(j.master)[i] = make_float4(p[0], p[1], p[2], p[3]);
      reinterpret_cast<float4*>(j.m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(j.v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (j.out_bf16)
        *reinterpret_cast<uint2*>(j.out_bf16 + e) = make_uint2(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]));
    }
  }
  if (j.sumsq) {
    sq = warp_sum(sq);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) atomicAdd(j.sumsq, t);
    }
  }
  return true;
}

}  // namespace ksa
