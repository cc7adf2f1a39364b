// Tensor-parallel inference: all-reduce of a row-parallel GEMM's partial outputs fused with the residual add and the
// RMSNorm that follow it.  Every rank's partial [rows, D] bf16 block sits at the same offset of a symmetric buffer; the
// kernel announces its own block to the peers, waits (bounded) for theirs, and then reads each row from all ranks with
// plain P2P loads, sums in rank order in fp32 (so every rank computes bit-identical results), adds the residual row,
// rounds the new residual stream to bf16 and normalises it.  One pass, no intermediate all-reduced tensor.
#include "comm.cuh"
#include "host.h"
#include "vec.cuh"

namespace ksa {

struct TpReduceArgs {
  const bf16* partial[kMaxPeers];  // partial[r]: rank r's block (peer pointer), same shape everywhere
  uint32_t* announce[kMaxPeers];   // address of flag[rank] in every rank's flag array
  const uint32_t* local_flags;     // flag[0..world) in own memory
  int world, rank;
  const bf16* x;                   // residual stream [rows_x, D]; rows >= delta_rows keep x unchanged
  const bf16* w;                   // norm scale [D] (null: no normalised output)
  bf16* res_out;                   // new residual stream [rows_x, D]
  bf16* y;                         // normalised output [rows_x, D]
  int rows_x, delta_rows, D;
  float eps;
  const uint32_t* epoch;           // device counter of finished all-reduces; this call's flag value is *epoch + 1
  uint32_t* done;                  // CTAs of this launch that have finished (the last one advances *epoch)
  int row_lo, row_hi;              // rows reduced by this rank (all of them, or its shard in the two-phase form)
  uint32_t* notify[kMaxPeers];     // two-phase form: flag2[rank] on every rank, raised when the shard is written
};

constexpr int kTpThreads = 256;
constexpr int kTpMaxVec = 4;  // D <= 8192

__device__ __forceinline__ void tp_reduce_rows(const TpReduceArgs& a, float* red) {
  for (int row = a.row_lo + blockIdx.x; row < a.row_hi; row += gridDim.x) {
    const long long base = (long long)row * a.D;
    const bool has_delta = row < a.delta_rows;
    float v[kTpMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kTpMaxVec; ++i) {
      const int c = (i * kTpThreads + threadIdx.x) * 8;
      if (c < a.D) {
        load8(a.x + base + c, v[i]);
        if (has_delta) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int r = 0; r < a.world; ++r) {
            const uint4 p = ld_peer_16(a.partial[r] + base + c);
            const uint32_t pu[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = unpack_bf16x2(pu[k]);
              acc[2 * k] += f.x;
              acc[2 * k + 1] += f.y;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j] + acc[j]));
        }
        store8(a.res_out + base + c, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    if (a.w != nullptr) {
      ss = block_sum<kTpThreads>(ss, red);
      const float rstd = rsqrtf(ss / (float)a.D + a.eps);
#pragma unroll
      for (int i = 0; i < kTpMaxVec; ++i) {
        const int c = (i * kTpThreads + threadIdx.x) * 8;
        if (c < a.D) {
          float wv[8], o[8];
          load8(a.w + c, wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
          store8(a.y + base + c, o);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kTpThreads) tp_allreduce_add_rmsnorm_kernel(TpReduceArgs a, int* status) {
  grid_dependency_launch();   // a dependent-launched successor may start (the skinny GEMM: its weight loads)
  grid_dependency_wait();     // launched dependently itself: the previous kernel's results are complete from here on
  __shared__ float red[32];
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // The exchange number lives on the device so that a captured CUDA graph stays valid from replay to replay: every
  // CTA reads it before it can finish, and only the last CTA to finish advances it.
  const uint32_t target = *reinterpret_cast<const volatile uint32_t*>(a.epoch) + 1u;
  // the partial block was written by the previous kernel of this stream: publish it, then wait for every peer's
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.announce[threadIdx.x], target);
  }
  if (threadIdx.x < a.world) {
    if (!flag_wait_ge(a.local_flags + threadIdx.x, target, status, kTimeoutPeerFlag, true)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) tp_reduce_rows(a, red);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {   // a timed-out launch still advances: the ranks stay in step
      *a.done = 0u;
      __threadfence();
      *const_cast<uint32_t*>(a.epoch) = target;
      // every CTA's rows were fenced before its increment of `done`: the shard is complete, tell the peers
      __threadfence_system();
      for (int r = 0; r < a.world; ++r)
        if (a.notify[r] != nullptr) st_release_sys(a.notify[r], target);
    }
  }
}

}  // namespace ksa

using namespace ksa;

static int tp_launch(const void* x, const void* const* partial_ptrs, const void* const* announce_ptrs,
                     const void* local_flags, int world, int rank, const void* w, void* res_out, void* y, int rows_x,
                     int delta_rows, int D, float eps, void* epoch, void* done, int row_lo, int row_hi,
                     const void* const* notify_ptrs, void* stream) {
  KSA_REQUIRE(world >= 1 && world <= kMaxPeers, "tp all-reduce: world %d out of range", world);
  KSA_REQUIRE(D % 8 == 0 && D <= kTpThreads * 8 * kTpMaxVec, "tp all-reduce: D=%d unsupported", D);
  KSA_REQUIRE(delta_rows <= rows_x, "tp all-reduce: delta rows exceed residual rows");
  KSA_REQUIRE(row_lo >= 0 && row_hi <= rows_x, "tp all-reduce: row range out of bounds");
  if (rows_x == 0) return 0;
  int* status = status_word();
  KSA_REQUIRE(status != nullptr, "could not allocate the status word");
  TpReduceArgs a{};
  for (int r = 0; r < world; ++r) {
    a.partial[r] = static_cast<const bf16*>(partial_ptrs[r]);
    a.announce[r] = static_cast<uint32_t*>(const_cast<void*>(announce_ptrs[r]));
    a.notify[r] = notify_ptrs ? static_cast<uint32_t*>(const_cast<void*>(notify_ptrs[r])) : nullptr;
  }
  a.local_flags = static_cast<const uint32_t*>(local_flags);
  a.world = world; a.rank = rank;
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.res_out = (bf16*)res_out; a.y = (bf16*)y;
  a.rows_x = rows_x; a.delta_rows = delta_rows; a.D = D; a.eps = eps;
  a.epoch = static_cast<const uint32_t*>(epoch); a.done = static_cast<uint32_t*>(done);
  a.row_lo = row_lo; a.row_hi = row_hi;
  KSA_REQUIRE(a.epoch != nullptr && a.done != nullptr, "tp all-reduce: epoch and done counters are required");
  // every CTA must be resident while it waits for the peers: at most 4 CTAs of 256 threads per SM are launched
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int rows = row_hi - row_lo;
  int grid = rows < sms * 4 ? (rows > 0 ? rows : 1) : sms * 4;
  tp_allreduce_add_rmsnorm_kernel<<<grid, kTpThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a, status);
  KSA_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// partial_ptrs[r]: rank r's partial block; announce_ptrs[r]: &flags[rank] on rank r; local_flags: own flags[0..world).
// epoch: device uint32, the number of all-reduces finished so far (identical on every rank; advanced by the kernel);
// done: device uint32 scratch counter, zero between launches.
KSA_API int ksa_tp_allreduce_add_rmsnorm(const void* x, const void* const* partial_ptrs, const void* const* announce_ptrs,
                                         const void* local_flags, int world, int rank, const void* w, void* res_out,
                                         void* y, int rows_x, int delta_rows, int D, float eps, void* epoch, void* done,
                                         void* stream) {
  KSA_ENTER(x);
  return tp_launch(x, partial_ptrs, announce_ptrs, local_flags, world, rank, w, res_out, y, rows_x, delta_rows, D, eps,
                   epoch, done, 0, rows_x, nullptr, stream);
}

// Two-phase form for many rows (prefill): this rank reduces only rows [row_lo, row_hi) - reduce-scatter + residual add
// + RMSNorm - into res_out / y, which are the same symmetric buffers on every rank, then raises notify_ptrs[r] (its
// flag in every rank's second flag array).  The peers' shards are fetched afterwards with ksa_peer_gather waiting on
// those flags.  Each rank reads rows*D partial elements instead of world*rows*D.
KSA_API int ksa_tp_reduce_scatter_add_rmsnorm(const void* x, const void* const* partial_ptrs,
                                              const void* const* announce_ptrs, const void* local_flags, int world,
                                              int rank, const void* w, void* res_out, void* y, int rows_x, int delta_rows,
                                              int D, float eps, void* epoch, void* done, int row_lo, int row_hi,
                                              const void* const* notify_ptrs, void* stream) {
  KSA_ENTER(x);
  KSA_REQUIRE(notify_ptrs != nullptr, "tp reduce-scatter: notify flags are required");
  return tp_launch(x, partial_ptrs, announce_ptrs, local_flags, world, rank, w, res_out, y, rows_x, delta_rows, D, eps,
                   epoch, done, row_lo, row_hi, notify_ptrs, stream);
}
