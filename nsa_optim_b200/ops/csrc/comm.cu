// Peer-memory collectives over NVLink / NVSwitch for the sharded runtime.
//
// Every rank owns one "arena" allocation that all ranks of the node map (CUDA IPC); a kernel
// receives an array of W base pointers (its own included) and reads or writes peers directly.
// Synchronisation uses monotonically increasing epoch words in the arena: a producer stores
// `epoch` into slot [its rank] of every peer's flag row with system-scope release; a consumer
// spins with acquire loads until the slot reaches the epoch.  Epochs never decrease, so there
// are no reset races.  Every spin is bounded by a cycle budget; on expiry the kernel records
// STATUS_TIMEOUT_PEER_FLAG (with the peer index) and returns without touching the data.
//
// Kernels
//   signal   : publish an epoch to all peers (ordered after prior work on the stream).
//   wait     : wait for a row of flags (used by tests and by host-ordered paths).
//   allgather: pull every peer's parameter shard into the local gathered buffer.
//   reduce_scatter: sum the W ranks' fp32 gradient buffers over this rank's slice in fixed
//              rank order (deterministic), scale, accumulate into the fp32 gradient shard and
//              optionally emit per-CTA partial sums of squares for the gradient norm.
//   reduce_scatter_adamw8bit: the same reduction feeding the blockwise 8-bit AdamW update of
//              the owned parameter shard in one pass (no gradient shard round trip).
// Peer memory is only ever accessed with plain loads and stores issued by these kernels.
#include "codebook.cuh"
#include "host.cuh"
#include <cuda_bf16.h>
#include <cstring>

namespace {
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *flag >= epoch or the cycle budget runs out.
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned epoch, long long max_cycles) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < max_cycles) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    __nanosleep(64);
  }
  return false;
}

// One thread per peer: flag_rows[p] is peer p's flag row; slot = this rank.
__global__ void signal_kernel(unsigned* const* flag_rows, int W, int slot, unsigned epoch) {
  const int p = threadIdx.x;
  if (p < W) {
    __threadfence_system();
    st_release_sys(flag_rows[p] + slot, epoch);
  }
}

__global__ void wait_kernel(const unsigned* flags, int n, unsigned epoch, long long max_cycles, KernelStatus* status) {
  const int i = threadIdx.x;
  if (i < n && !wait_flag(flags + i, epoch, max_cycles)) status_report(status, STATUS_TIMEOUT_PEER_FLAG, i, (int)epoch);
}

// CTA-wide wait for peers [0, W) except `skip`; returns false (uniformly) on timeout.
__device__ __forceinline__ bool cta_wait_peers(const unsigned* flags, int W, int skip, unsigned epoch,
                                               long long max_cycles, KernelStatus* status, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (flags != nullptr && threadIdx.x < W && threadIdx.x != skip) {
    if (!wait_flag(flags + threadIdx.x, epoch, max_cycles)) {
      status_report(status, STATUS_TIMEOUT_PEER_FLAG, threadIdx.x, (int)epoch);
      *sh_ok = 0;
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}

// grid (ctas_per_peer, W): blockIdx.y = k, peer p = (rank + k) % W so that ranks start on different peers.
__global__ void __launch_bounds__(256) allgather_kernel(const uint4* const* shards, uint4* out, long shard_vec, int W,
                                                        int rank, const unsigned* flags, unsigned epoch,
                                                        long long max_cycles, KernelStatus* status) {
  __shared__ int sh_ok;
  const int p = (rank + blockIdx.y) % W;
  if (threadIdx.x == 0) {
    sh_ok = 1;
    if (p != rank && flags != nullptr && !wait_flag(flags + p, epoch, max_cycles)) {
      status_report(status, STATUS_TIMEOUT_PEER_FLAG, p, (int)epoch);
      sh_ok = 0;
    }
  }
  __syncthreads();
  if (!sh_ok) return;
  const uint4* src = shards[p];
  uint4* dst = out + static_cast<long>(p) * shard_vec;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  constexpr int U = 8;                                  // independent 16-byte peer loads in flight per thread
  for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < shard_vec; i0 += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      if (i < shard_vec) v[u] = src[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      if (i < shard_vec) dst[i] = v[u];
    }
  }
}

// grads[p]: rank p's full fp32 gradient buffer (W * S floats).  This rank reduces slice `rank`.
__global__ void __launch_bounds__(256) reduce_scatter_kernel(const float* const* grads, float* grad_shard, long S4, int W,
                                                             int rank, float scale, int accumulate, float* sumsq_partial,
                                                             const unsigned* flags, unsigned epoch, long long max_cycles,
                                                             KernelStatus* status) {
  __shared__ int sh_ok;
  __shared__ float red[8];
  if (!cta_wait_peers(flags, W, rank, epoch, max_cycles, status, &sh_ok)) return;
  float ss = 0.f;
  const long base = static_cast<long>(rank) * S4;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  constexpr int U = 8;                                  // independent 16-byte loads in flight per thread and peer
  for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < S4; i0 += stride * U) {
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < W; ++p) {                      // fixed order: bitwise reproducible
      const float4* g = reinterpret_cast<const float4*>(grads[p]) + base;
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + u * stride;
        v[u] = i < S4 ? g[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      if (i >= S4) break;
      float4 a = acc[u];
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      float4* o = reinterpret_cast<float4*>(grad_shard) + i;
      if (accumulate) { const float4 q = *o; a.x += q.x; a.y += q.y; a.z += q.z; a.w += q.w; }
      *o = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  if (sumsq_partial) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < 8; ++k) t += red[k];
      sumsq_partial[blockIdx.x] = t;
    }
  }
}

struct AdamArgs { float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt; };

// One CTA per 256-element block of the owned shard.  wd_mask[b] != 0 -> weight decay applies.
template <typename PT>
__global__ void __launch_bounds__(256) rs_adamw8bit_kernel(const float* const* grads, PT* p_shard, uint8_t* mq, float* mabs,
                                                           uint8_t* vq, float* vabs, const float* cb_signed,
                                                           const float* cb_unsigned, const uint8_t* wd_mask, long nblocks,
                                                           long S, int W, int rank, float scale, AdamArgs a,
                                                           const unsigned* flags, unsigned epoch, long long max_cycles,
                                                           KernelStatus* status) {
  __shared__ int sh_ok;
  __shared__ float cs[256], cu[256], red_m[8], red_v[8];
  __shared__ uint8_t ts[cbk::kTable], tu[cbk::kTable];
  cs[threadIdx.x] = cb_signed[threadIdx.x];
  cu[threadIdx.x] = cb_unsigned[threadIdx.x];
  __syncthreads();
  cbk::build_table(cs, ts);
  cbk::build_table(cu, tu);
  if (!cta_wait_peers(flags, W, rank, epoch, max_cycles, status, &sh_ok)) return;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  for (long b = blockIdx.x; b < nblocks; b += gridDim.x) {
    const long i = b * 256 + threadIdx.x;
    float gr = 0.f;
    for (int p = 0; p < W; ++p) gr += grads[p][static_cast<long>(rank) * S + i];
    gr *= scale;
    const float mm = a.beta1 * (cs[mq[i]] * mabs[b]) + (1.f - a.beta1) * gr;
    const float vv = a.beta2 * (cu[vq[i]] * vabs[b]) + (1.f - a.beta2) * gr * gr;
    float wt = static_cast<float>(p_shard[i]);
    if (wd_mask == nullptr || wd_mask[b]) wt *= (1.f - a.lr * a.wd);
    wt -= (a.lr / a.bc1) * mm / (sqrtf(vv) / a.bc2_sqrt + a.eps);
    p_shard[i] = static_cast<PT>(wt);
    float am = fabsf(mm), av = vv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o)); av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, o)); }
    __syncthreads();
    if (l == 0) { red_m[w] = am; red_v[w] = av; }
    __syncthreads();
    am = red_m[0]; av = red_v[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) { am = fmaxf(am, red_m[k]); av = fmaxf(av, red_v[k]); }
    mq[i] = static_cast<uint8_t>(cbk::nearest_code(cs, ts, mm / fmaxf(am, 1e-30f)));
    vq[i] = static_cast<uint8_t>(cbk::nearest_code(cu, tu, vv / fmaxf(av, 1e-30f)));
    if (threadIdx.x == 0) { mabs[b] = am; vabs[b] = av; }
  }
}

inline int grid_cap(long want, int per_sm) {
  long cap = static_cast<long>(nsa::sm_count()) * per_sm;
  return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
}
}  // namespace

// Make `peer_device`'s memory addressable from kernels on the current device.
extern "C" int nsa_enable_peer_access(int peer_device) {
  int cur = 0;
  cudaGetDevice(&cur);
  if (cur == peer_device) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, cur, peer_device);
  if (e != cudaSuccess) return nsa::fail_cuda(e, "cudaDeviceCanAccessPeer");
  if (!can) return nsa::fail(NSA_ERR_CUDA, "peer access between these devices is not supported");
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "cudaDeviceEnablePeerAccess");
}

// flag_rows: device array of W pointers (each peer's flag row for this channel).
extern "C" int nsa_comm_signal(unsigned* const* flag_rows, int W, int slot, unsigned epoch, cudaStream_t st) {
  if (W > 32) return nsa::fail(NSA_ERR_SHAPE, "comm: at most 32 ranks per node");
  signal_kernel<<<1, 32, 0, st>>>(flag_rows, W, slot, epoch);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_comm_wait(const unsigned* flags, int n, unsigned epoch, long long max_cycles, cudaStream_t st) {
  if (n > 32) return nsa::fail(NSA_ERR_SHAPE, "comm: at most 32 flags per wait");
  wait_kernel<<<1, 32, 0, st>>>(flags, n, epoch, max_cycles, nsa::status_ptr());
  nsa::count_launch();
  return 0;
}
// shards: device array of W pointers to the ranks' shards (shard_bytes each, multiple of 16).
extern "C" int nsa_comm_allgather(const void* const* shards, void* out, long shard_bytes, int W, int rank,
                                  const unsigned* flags, unsigned epoch, long long max_cycles, int ctas_per_peer,
                                  cudaStream_t st) {
  if (shard_bytes % 16) return nsa::fail(NSA_ERR_ALIGNMENT, "allgather: shard size must be a multiple of 16 bytes");
  if (ctas_per_peer <= 0) ctas_per_peer = 16;
  allgather_kernel<<<dim3(ctas_per_peer, W), 256, 0, st>>>((const uint4* const*)shards, (uint4*)out, shard_bytes / 16, W,
                                                           rank, flags, epoch, max_cycles, nsa::status_ptr());
  nsa::count_launch();
  return 0;
}
// A reduce-scatter runs beside the backward pass of the next block: a small grid (well under one
// CTA per SM) with several loads in flight per thread keeps the link busy without taking the
// compute kernels' SMs.
extern "C" int nsa_comm_reduce_scatter_parts(void) { return 96; }
// grads: device array of W pointers to full fp32 gradient buffers (W*S floats); S multiple of 4.
extern "C" int nsa_comm_reduce_scatter(const float* const* grads, float* grad_shard, long S, int W, int rank, float scale,
                                       int accumulate, float* sumsq_partial, const unsigned* flags, unsigned epoch,
                                       long long max_cycles, cudaStream_t st) {
  if (S % 4) return nsa::fail(NSA_ERR_ALIGNMENT, "reduce_scatter: shard length must be a multiple of 4");
  const int grid = nsa_comm_reduce_scatter_parts();
  reduce_scatter_kernel<<<grid, 256, 0, st>>>(grads, grad_shard, S / 4, W, rank, scale, accumulate, sumsq_partial, flags,
                                              epoch, max_cycles, nsa::status_ptr());
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_comm_rs_adamw8bit(const float* const* grads, void* p_shard, int p_fp32, uint8_t* mq, float* mabs,
                                     uint8_t* vq, float* vabs, const float* cb_signed, const float* cb_unsigned,
                                     const uint8_t* wd_mask, long S, int W, int rank, float scale, int step, float lr,
                                     float b1, float b2, float eps, float wd, const unsigned* flags, unsigned epoch,
                                     long long max_cycles, cudaStream_t st) {
  if (S % 256) return nsa::fail(NSA_ERR_ALIGNMENT, "rs_adamw8bit: shard length must be a multiple of 256");
  AdamArgs a;
  a.lr = lr; a.beta1 = b1; a.beta2 = b2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(b1, (float)step);
  a.bc2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  const long nb = S / 256;
  const int grid = grid_cap(nb, 8);
  if (p_fp32)
    rs_adamw8bit_kernel<float><<<grid, 256, 0, st>>>(grads, (float*)p_shard, mq, mabs, vq, vabs, cb_signed, cb_unsigned,
                                                     wd_mask, nb, S, W, rank, scale, a, flags, epoch, max_cycles, nsa::status_ptr());
  else
    rs_adamw8bit_kernel<bf16><<<grid, 256, 0, st>>>(grads, (bf16*)p_shard, mq, mabs, vq, vabs, cb_signed, cb_unsigned,
                                                    wd_mask, nb, S, W, rank, scale, a, flags, epoch, max_cycles, nsa::status_ptr());
  nsa::count_launch();
  return 0;
}

// ---- arena allocation and CUDA IPC.  The arena is a plain cudaMalloc allocation so that its
// handle describes exactly this buffer.  A peer must open the handle with ITS OWN device
// current: the mapping (and the lazily enabled peer access) then belongs to the context whose
// kernels will dereference the pointer.
extern "C" int nsa_ipc_alloc(long nbytes, void** out_ptr, unsigned char* handle64) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(nbytes));
  if (e != cudaSuccess) return nsa::fail_cuda(e, "nsa_ipc_alloc: cudaMalloc");
  e = cudaMemset(p, 0, static_cast<size_t>(nbytes));
  if (e != cudaSuccess) return nsa::fail_cuda(e, "nsa_ipc_alloc: cudaMemset");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return nsa::fail_cuda(e, "nsa_ipc_alloc: cudaIpcGetMemHandle"); }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *out_ptr = p;
  return 0;
}
extern "C" int nsa_ipc_open(const unsigned char* handle64, void** out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ipc_open: cudaIpcOpenMemHandle");
}
extern "C" int nsa_ipc_close(void* p) {
  cudaError_t e = cudaIpcCloseMemHandle(p);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ipc_close");
}
extern "C" int nsa_ipc_free(void* p) {
  cudaError_t e = cudaFree(p);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ipc_free");
}
