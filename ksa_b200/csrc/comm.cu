// Communication kernels over NVLink / NVSwitch peer memory (P2P loads and stores issued from inside the
// kernels; no TMA multicast, no library collective):
//
//   ksa_peer_gather         pull all-gather: every rank copies the other ranks' shards of a flat bf16 buffer out of
//                           their memory into its own copy (FSDP parameter all-gather; TP all-gather).
//   ksa_peer_reduce_adamw   reduce-scatter fused with the optimizer: the owner of a shard reads that shard of every
//                           rank's fp32 gradient buffer over NVLink, sums and scales it, clips by value, applies
//                           AdamW to its fp32 master weights and moments, writes the refreshed bf16 weights into its
//                           shard of the compute buffer and accumulates sum(g^2) for the gradient-norm metric.
//                           Replaces NCCL reduce-scatter -> foreach AdamW -> cast of the reference
//                           (muse/training/distributed.py:232-287, recipes/pretrain_kai_summary_unified.py:1045-1053).
//   ksa_signal_set / wait   release-store a step counter into every peer's signal pad / bounded acquire-wait on it.
//
// The same device routines run as "communication CTAs" inside the GEMM kernel (gemm.cu), which is how the
// parameter all-gather of the next FSDP unit and the reduce-scatter + AdamW of the previous one overlap with the
// tensor-core tiles of the current GEMM in one launch.
//
// Every wait on a peer flag is bounded (about a second) and reports through the status word.
#include "comm.cuh"
#include "host.h"

#include <string.h>

namespace ksa {

__global__ void __launch_bounds__(kCommThreads) peer_gather_kernel(GatherJob job, int* status) {
  run_gather_job(job, blockIdx.x, gridDim.x, status);
}

// at most 64 registers per thread: two of these CTAs, or one next to a GEMM CTA, fit on an SM
__global__ void __launch_bounds__(kCommThreads, 2) peer_reduce_adamw_kernel(ReduceAdamwJob job, int* status) {
  run_reduce_adamw_job(job, blockIdx.x, gridDim.x, status);
}

__global__ void signal_set_kernel(SignalTargets t, const uint32_t* epoch_ptr, uint32_t add) {
  if (threadIdx.x < t.n && t.ptr[threadIdx.x] != nullptr) {
    __threadfence_system();
    st_release_sys(t.ptr[threadIdx.x], epoch_target(epoch_ptr, add));
  }
}

__global__ void signal_wait_kernel(const uint32_t* flags, int n, const uint32_t* epoch_ptr, uint32_t add, int* status) {
  if (threadIdx.x < n) flag_wait_ge(flags + threadIdx.x, epoch_target(epoch_ptr, add), status, kTimeoutPeerFlag, true);
}

// dst (local) = src (peer or local) for nbytes (multiple of 16), after an optional bounded wait on a local flag.
__global__ void __launch_bounds__(kCommThreads)
peer_copy_kernel(uint8_t* dst, const uint8_t* src, long long nbytes, const uint32_t* flag, const uint32_t* epoch_ptr,
                 uint32_t add, int* status) {
  __shared__ int s_ok;
  if (flag) {
    if (threadIdx.x == 0) s_ok = flag_wait_ge(flag, epoch_target(epoch_ptr, add), status, kTimeoutPeerFlag, true) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const long long vecs = nbytes / 16, stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
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

// dst (local bf16) += src (peer bf16) over n elements (multiple of 8), fp32 adds, after an optional flag wait.
__global__ void __launch_bounds__(kCommThreads)
peer_add_bf16_kernel(bf16* dst, const bf16* src, long long n, const uint32_t* flag, const uint32_t* epoch_ptr,
                     uint32_t add, int* status) {
  __shared__ int s_ok;
  if (flag) {
    if (threadIdx.x == 0) s_ok = flag_wait_ge(flag, epoch_target(epoch_ptr, add), status, kTimeoutPeerFlag, true) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const long long vecs = n / 8, stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride) {
    const uint4 a = ld_peer_16(src + i * 8);
    uint4 d = *reinterpret_cast<uint4*>(dst + i * 8);
    const uint32_t au[4] = {a.x, a.y, a.z, a.w};
    uint32_t du[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = unpack_bf16x2(au[k]), y = unpack_bf16x2(du[k]);
      du[k] = pack_bf16x2(x.x + y.x, x.y + y.y);
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(du[0], du[1], du[2], du[3]);
  }
}

// 2-D copy: `rows` rows of `row_bytes` (multiple of 16) from src (any rank's memory, pitch src_pitch) to dst (own
// memory, pitch dst_pitch), after an optional bounded wait on a local flag.  The building block of the all-to-all
// that turns sequence shards into head shards and back.
__global__ void __launch_bounds__(kCommThreads)
peer_copy2d_kernel(uint8_t* dst, long long dst_pitch, const uint8_t* src, long long src_pitch, long long rows,
                   int row_vecs, const uint32_t* flag, const uint32_t* epoch_ptr, uint32_t add, int* status) {
  __shared__ int s_ok;
  if (flag) {
    if (threadIdx.x == 0) s_ok = flag_wait_ge(flag, epoch_target(epoch_ptr, add), status, kTimeoutPeerFlag, true) ? 1 : 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const long long total = rows * row_vecs, stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < total; i += 2 * stride) {
    const long long r0 = i / row_vecs, c0 = i - r0 * row_vecs;
    const long long j = i + stride, r1 = j / row_vecs, c1 = j - r1 * row_vecs;
    const uint4 a = ld_peer_16(src + r0 * src_pitch + c0 * 16), b = ld_peer_16(src + r1 * src_pitch + c1 * 16);
    *reinterpret_cast<uint4*>(dst + r0 * dst_pitch + c0 * 16) = a;
    *reinterpret_cast<uint4*>(dst + r1 * dst_pitch + c1 * 16) = b;
  }
  for (; i < total; i += stride) {
    const long long r0 = i / row_vecs, c0 = i - r0 * row_vecs;
    *reinterpret_cast<uint4*>(dst + r0 * dst_pitch + c0 * 16) = ld_peer_16(src + r0 * src_pitch + c0 * 16);
  }
}

}  // namespace ksa

using namespace ksa;

// ------------------------------------------------------------------------------------------ memory + IPC
KSA_API int ksa_symm_alloc(void** out, long long bytes) {
  KSA_REQUIRE(bytes > 0, "symm_alloc: bytes must be positive");
  void* p = nullptr;
  KSA_CHECK_CUDA(cudaMalloc(&p, (size_t)bytes));
  KSA_CHECK_CUDA(cudaMemset(p, 0, (size_t)bytes));
  *out = p;
  return 0;
}
KSA_API int ksa_symm_free(void* p) {
  if (p) KSA_CHECK_CUDA(cudaFree(p));
  return 0;
}
// handle_out: 64 bytes
KSA_API int ksa_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  KSA_CHECK_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
KSA_API int ksa_ipc_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  KSA_CHECK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}
KSA_API int ksa_ipc_close(void* p) {
  if (p) KSA_CHECK_CUDA(cudaIpcCloseMemHandle(p));
  return 0;
}

// ------------------------------------------------------------------------------------------ kernels
// peers: world pointers to the ranks' copies of the flat buffer (peers[rank] = own copy).  Shard r of every copy is
// elements [r*shard_elems, (r+1)*shard_elems); the call copies every shard r != rank from peers[r] into peers[rank].
// ready_flags (optional): world flags in OWN memory; shard r is copied once ready_flags[r] >= *epoch_ptr + epoch_add (epoch_ptr: device uint32, may be null = 0).
KSA_API int ksa_peer_gather(const void* const* peers, int world, int rank, long long shard_elems, int elem_bytes,
                            const void* ready_flags, const void* epoch_ptr, unsigned epoch_add, int ctas, void* stream) {
  KSA_ENTER(peers[rank]);
  KSA_REQUIRE(world >= 1 && world <= kMaxPeers, "peer_gather: world %d out of range (max %d)", world, kMaxPeers);
  KSA_REQUIRE((shard_elems * elem_bytes) % 16 == 0, "peer_gather: shard bytes must be a multiple of 16");
  if (world == 1) return 0;
  GatherJob job{};
  for (int r = 0; r < world; ++r) job.peers[r] = static_cast<const uint8_t*>(peers[r]);
  job.world = world; job.rank = rank; job.shard_bytes = shard_elems * elem_bytes;
  job.ready_flags = static_cast<const uint32_t*>(ready_flags);
  job.epoch_ptr = static_cast<const uint32_t*>(epoch_ptr); job.epoch_add = epoch_add;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  if (ctas <= 0) ctas = 16;
  peer_gather_kernel<<<ctas, kCommThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(job, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// grads: world pointers to the ranks' fp32 gradient buffers (full unit); this rank owns [shard_lo, shard_lo + n).
// master / m / v: this rank's fp32 shard (n elements); out_bf16: OWN full compute buffer (the shard region is written).
// hyper: device [lr, 1-b1^t, 1-b2^t, grad_scale].  ready_flags (optional): world flags in own memory; the reduction
// starts once all of them are >= *epoch_ptr + epoch_add (every rank has finished writing this unit's gradients).
KSA_API int ksa_peer_reduce_adamw(const void* const* grads, int world, int rank, long long shard_lo, long long n,
                                  void* master, void* m, void* v, void* out_bf16, const void* hyper, float beta1,
                                  float beta2, float eps, float weight_decay, float clip_value, void* sumsq,
                                  const void* ready_flags, const void* epoch_ptr, unsigned epoch_add, int ctas,
                                  void* stream) {
  KSA_ENTER(master);
  KSA_REQUIRE(world >= 1 && world <= kMaxPeers, "peer_reduce_adamw: world %d out of range (max %d)", world, kMaxPeers);
  KSA_REQUIRE(n % 4 == 0 && shard_lo % 4 == 0, "peer_reduce_adamw: shard offset/size must be multiples of 4");
  if (n == 0) return 0;
  ReduceAdamwJob job{};
  for (int r = 0; r < world; ++r) job.grads[r] = static_cast<const float*>(grads[r]);
  job.world = world; job.rank = rank; job.shard_lo = shard_lo; job.n = n;
  job.master = (float*)master; job.m = (float*)m; job.v = (float*)v; job.out_bf16 = (bf16*)out_bf16;
  job.hyper = (const float*)hyper; job.beta1 = beta1; job.beta2 = beta2; job.eps = eps;
  job.weight_decay = weight_decay; job.clip_value = clip_value; job.sumsq = (float*)sumsq;
  job.ready_flags = static_cast<const uint32_t*>(ready_flags);
  job.epoch_ptr = static_cast<const uint32_t*>(epoch_ptr); job.epoch_add = epoch_add;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  if (ctas <= 0) ctas = 32;
  peer_reduce_adamw_kernel<<<ctas, kCommThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(job, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Context parallelism: fold what the later ranks added into this rank's fp32 return block into its bf16 gradients,
// and clear the block for its next use.  dst [B, rows, width] bf16 (row / batch strides in elements), ret the same
// shape in fp32.  flags (optional): n_flags flags in own memory that the contributing ranks raise to `target` when
// their backward kernels are done; the wait is bounded.
__global__ void __launch_bounds__(256) cp_fold_return_kernel(bf16* dst, float* ret, int B, int rows, int width,
                                                             long long dst_rs, long long dst_bs, long long ret_rs,
                                                             long long ret_bs, const uint32_t* flags, int n_flags,
                                                             uint32_t target, int* status) {
  __shared__ int s_ok;
  if (flags != nullptr && n_flags > 0) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < n_flags && !flag_wait_ge(flags + threadIdx.x, target, status, kTimeoutPeerFlag, true)) s_ok = 0;
    __syncthreads();
    if (!s_ok) return;
  }
  const long long vec_per_row = width / 4;
  const long long total = (long long)B * rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long c = i % vec_per_row, rw = (i / vec_per_row) % rows, b = i / (vec_per_row * rows);
    float4* src = reinterpret_cast<float4*>(ret + b * ret_bs + rw * ret_rs + c * 4);
    uint2* d = reinterpret_cast<uint2*>(dst + b * dst_bs + rw * dst_rs + c * 4);
    const float4 a = *src;
    const uint2 old = *d;
    const float2 lo = unpack_bf16x2(old.x), hi = unpack_bf16x2(old.y);
    *d = make_uint2(pack_bf16x2(lo.x + a.x, lo.y + a.y), pack_bf16x2(hi.x + a.z, hi.y + a.w));
    *src = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

KSA_API int ksa_cp_fold_return(void* dst, void* ret, int B, int rows, int width, long long dst_rs, long long dst_bs,
                               long long ret_rs, long long ret_bs, const void* flags, int n_flags, unsigned target,
                               void* stream) {
  KSA_ENTER(dst);
  KSA_REQUIRE(width % 4 == 0 && dst_rs % 4 == 0 && ret_rs % 4 == 0, "cp_fold_return: width and strides must be multiples of 4");
  KSA_REQUIRE(n_flags >= 0 && n_flags <= 256, "cp_fold_return: %d flags", n_flags);
  if (B == 0 || rows == 0) return 0;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  const long long total = (long long)B * rows * (width / 4);
  const int blocks = (int)((total + 255) / 256 < 592 ? (total + 255) / 256 : 592);
  cp_fold_return_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (bf16*)dst, (float*)ret, B, rows, width, dst_rs, dst_bs, ret_rs, ret_bs, (const uint32_t*)flags, n_flags, target, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Store *epoch_ptr + epoch_add (release, system scope) to n flag addresses (own and peer memory), after all prior work of the stream.
KSA_API int ksa_signal_set(const void* const* flag_ptrs, int n, const void* epoch_ptr, unsigned epoch_add, void* stream) {
  KSA_REQUIRE(n >= 1 && n <= kMaxPeers, "signal_set: n %d out of range", n);
  SignalTargets t{};
  t.n = n;
  for (int i = 0; i < n; ++i) t.ptr[i] = static_cast<uint32_t*>(const_cast<void*>(flag_ptrs[i]));
  signal_set_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(t, static_cast<const uint32_t*>(epoch_ptr), epoch_add);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Bounded wait until n consecutive flags in own memory are >= *epoch_ptr + epoch_add (a timeout is reported via the status word).
KSA_API int ksa_signal_wait(const void* flags, int n, const void* epoch_ptr, unsigned epoch_add, void* stream) {
  KSA_ENTER(flags);
  KSA_REQUIRE(n >= 1 && n <= 32, "signal_wait: n %d out of range", n);
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  signal_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>((const uint32_t*)flags, n,
                                                                            static_cast<const uint32_t*>(epoch_ptr), epoch_add, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// dst (own memory) = src (any rank's memory) for nbytes (multiple of 16).  flag (optional, own memory): wait, bounded,
// until *flag >= *epoch_ptr + epoch_add before reading src.
KSA_API int ksa_peer_copy(void* dst, const void* src, long long nbytes, const void* flag, const void* epoch_ptr,
                          unsigned epoch_add, int ctas, void* stream) {
  KSA_ENTER(dst);
  KSA_REQUIRE(nbytes % 16 == 0, "peer_copy: nbytes must be a multiple of 16");
  if (nbytes == 0) return 0;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  if (ctas <= 0) ctas = 32;
  peer_copy_kernel<<<ctas, kCommThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (uint8_t*)dst, (const uint8_t*)src, nbytes, (const uint32_t*)flag, (const uint32_t*)epoch_ptr, epoch_add, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// dst (own bf16) += src (any rank's bf16) over n elements (multiple of 8), with the same optional flag wait.
KSA_API int ksa_peer_add_bf16(void* dst, const void* src, long long n, const void* flag, const void* epoch_ptr,
                              unsigned epoch_add, int ctas, void* stream) {
  KSA_ENTER(dst);
  KSA_REQUIRE(n % 8 == 0, "peer_add_bf16: n must be a multiple of 8");
  if (n == 0) return 0;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  if (ctas <= 0) ctas = 32;
  peer_add_bf16_kernel<<<ctas, kCommThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (bf16*)dst, (const bf16*)src, n, (const uint32_t*)flag, (const uint32_t*)epoch_ptr, epoch_add, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// dst (own memory, pitch dst_pitch) = src (any rank's memory, pitch src_pitch): rows x row_bytes, every address and
// pitch a multiple of 16 bytes, with the same optional flag wait as ksa_peer_copy.
KSA_API int ksa_peer_copy2d(void* dst, long long dst_pitch, const void* src, long long src_pitch, long long rows,
                            long long row_bytes, const void* flag, const void* epoch_ptr, unsigned epoch_add, int ctas,
                            void* stream) {
  KSA_ENTER(dst);
  KSA_REQUIRE(row_bytes % 16 == 0 && dst_pitch % 16 == 0 && src_pitch % 16 == 0,
              "peer_copy2d: row bytes and pitches must be multiples of 16");
  KSA_REQUIRE(row_bytes <= dst_pitch && row_bytes <= src_pitch, "peer_copy2d: a row is longer than its pitch");
  if (rows == 0 || row_bytes == 0) return 0;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  if (ctas <= 0) ctas = 32;
  peer_copy2d_kernel<<<ctas, kCommThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (uint8_t*)dst, dst_pitch, (const uint8_t*)src, src_pitch, rows, (int)(row_bytes / 16), (const uint32_t*)flag,
      (const uint32_t*)epoch_ptr, epoch_add, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}
