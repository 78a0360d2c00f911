// bf16 GEMM for sm_100a: C[M,N] = op(A) * op(B) with fp32 accumulation in tensor memory.
//
//   * persistent: one CTA per SM walks a grouped (L2-friendly) tile order;
//   * warp-specialised: warp 0 = TMA producer, warp 1 = tcgen05.mma issuer (one elected
//     thread) and TMEM owner, warps 2..5 = epilogue (one TMEM lane quarter each);
//   * 128 x 256 output tile, K step 64, 4-stage shared-memory ring (48 KB per stage);
//   * two 256-column TMEM accumulators so the epilogue of tile i overlaps the MMAs of i+1;
//   * both operands may be K-major or MN-major (selected in the instruction descriptor and
//     the shared-memory descriptors), which covers y = x W^T, dx = dy W and dW = dy^T x
//     without any transposed copy;
//   * output bf16 or fp32, optional accumulate into C (C += A*B) for gradient accumulation.
//
// Operand conventions (all row-major in global memory, leading dimension in elements):
//   a_mn = 0: A is [M, K] (K contiguous)      a_mn = 1: A is [K, M] (M contiguous)
//   b_mn = 0: B is [N, K] (K contiguous)      b_mn = 1: B is [K, N] (N contiguous)
// Requirements: base pointers 16-byte aligned, leading dimensions multiples of 8 elements.
#include <cstdlib>
#include <cstring>
#include "host.cuh"
#include "tc5.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;      // one 64-wide MN chunk of an MN-major tile: 8 KB
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t TMEM_COLS = 512;

// All-gather fused into the GEMM: the B operand (a weight inside a sharded unit's gathered
// buffer `full`) is still being assembled while the GEMM runs.  The first `copy_ctas` CTAs of
// the grid pull every rank's shard (peer memory, plain 16-byte loads) into `full` in chunks and
// publish chunk_flags[id] = epoch; the TMA producer of each GEMM CTA waits for the chunks that
// cover a B tile before loading it.  Ranks start pulling from different peers, and the
// N-block order is rotated to follow the same order, so no peer is read by everyone at once.
struct AgFuse {
  int enabled;
  int W, rank;
  const uint4* const* shards;   // W pointers (device array), one shard per rank
  uint4* full;                  // local gathered buffer: W * shard_vec 16-byte units
  long shard_vec, chunk_vec;    // in 16-byte units
  int chunks_per_shard;
  unsigned* chunk_flags;        // local, W * chunks_per_shard words
  const unsigned* peer_flags;   // local flag row: shard p is final when peer_flags[p] >= epoch
  unsigned epoch;
  long b_vec_offset;            // offset of B inside `full`, 16-byte units
  long long max_cycles;
  int copy_ctas;
  int n_rot;                    // rotation of the N-block order
  int w_lo, w_hi, w_start;      // chunk ids (shard-major numbering) that hold B, and the one the sweep needs first
};

struct GemmParams {
  AgFuse ag;
  int M, N, K;
  int ldc, ldb;
  int a_mn, b_mn;
  int out_fp32;
  int accumulate;
  int split_k;                  // pair kernel: parts the reduction is cut into (1 = none); parts meet in
                                // an fp32 C through TMA reduce-add stores
  void* C;
  KernelStatus* status;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool spin_until(const unsigned* flag, unsigned epoch, long long max_cycles, bool sys) {
  const long long t0 = clock64();
  for (;;) {
    const unsigned v = sys ? ld_acquire_sys_u32(flag) : ld_acquire_gpu(flag);
    if (v >= epoch) return true;
    if (clock64() - t0 > max_cycles) return false;
    __nanosleep(32);
  }
}
__device__ __forceinline__ int ag_chunk_id(const AgFuse& ag, long g) {
  const long pidx = g / ag.shard_vec;
  const long i = g - pidx * ag.shard_vec;
  return static_cast<int>(pidx * ag.chunks_per_shard + i / ag.chunk_vec);
}

// Copy role of the fused all-gather (all threads of the CTA).
__device__ void ag_copy_role(const AgFuse& ag, int cta, KernelStatus* status) {
  __shared__ int sh_ok;
  const int jobs = ag.W * ag.chunks_per_shard;
  int ready_peer = -1;
  for (int q = cta; q < jobs; q += ag.copy_ctas) {
    const int k = q / ag.chunks_per_shard, c = q - k * ag.chunks_per_shard;
    const int pr = (ag.rank + k) % ag.W;
    if (pr != ag.rank && pr != ready_peer) {
      if (threadIdx.x == 0) {
        sh_ok = 1;
        if (ag.peer_flags != nullptr && !spin_until(ag.peer_flags + pr, ag.epoch, ag.max_cycles, true)) {
          status_report(status, STATUS_TIMEOUT_PEER_FLAG, pr, (int)ag.epoch);
          sh_ok = 0;
        }
      }
      __syncthreads();
      if (!sh_ok) return;
      ready_peer = pr;
    }
    const long lo = static_cast<long>(c) * ag.chunk_vec;
    const long hi = lo + ag.chunk_vec < ag.shard_vec ? lo + ag.chunk_vec : ag.shard_vec;
    const uint4* src = ag.shards[pr];
    uint4* dst = ag.full + static_cast<long>(pr) * ag.shard_vec;
    // eight independent 16-byte loads in flight per thread: a peer load takes microseconds, and one
    // load at a time per thread would leave the link almost idle
    constexpr int U = 8;
    for (long i0 = lo + threadIdx.x; i0 < hi; i0 += static_cast<long>(blockDim.x) * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + static_cast<long>(u) * blockDim.x;
        if (i < hi) v[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + static_cast<long>(u) * blockDim.x;
        if (i < hi) dst[i] = v[u];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ag.chunk_flags + pr * ag.chunks_per_shard + c), "r"(ag.epoch) : "memory");
    }
  }
}

// One thread stores 32 consecutive accumulator columns of its row straight to global memory
// (fp32 or bf16 output, optional accumulation into C, any alignment).
__device__ __forceinline__ void store_direct(const uint32_t (&r)[32], int row, int col, const GemmParams& p) {
  const bool full = (col + 32 <= p.N);
  if (p.out_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
    if (full && (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        float4* q = reinterpret_cast<float4*>(dst) + j;
        if (p.accumulate) { float4 o = *q; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
        *q = v;
      }
    } else {
      for (int j = 0; j < 32 && col + j < p.N; ++j) {
        float v = __uint_as_float(r[j]);
        dst[j] = p.accumulate ? dst[j] + v : v;
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
    if (full && (p.ldc & 7) == 0 && !p.accumulate && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = tc5::pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        v.y = tc5::pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        v.z = tc5::pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        v.w = tc5::pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        reinterpret_cast<uint4*>(dst)[j] = v;
      }
    } else {
      for (int j = 0; j < 32 && col + j < p.N; ++j) {
        float v = __uint_as_float(r[j]);
        if (p.accumulate) v += __bfloat162float(dst[j]);
        dst[j] = __float2bfloat16(v);
      }
    }
  }
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int local = t - g * per_group;
  mb = first_m + local % gm;
  nb = local / gm;
}

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]  TMA -> MMA
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]  MMA -> TMA
  uint64_t* tfull_bar = bars + 2 * STAGES;       // [2]       MMA -> epilogue
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]       epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (p.ag.enabled && static_cast<int>(blockIdx.x) < p.ag.copy_ctas) {
    ag_copy_role(p.ag, blockIdx.x, p.status);
    return;
  }
  const int cta = p.ag.enabled ? blockIdx.x - p.ag.copy_ctas : blockIdx.x;
  const int n_ctas = p.ag.enabled ? gridDim.x - p.ag.copy_ctas : gridDim.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  // With the fused all-gather the TMA producer may wait up to ag.max_cycles for a peer's shard, so
  // everything downstream of it (MMA issuer, epilogue) must be at least that patient: otherwise
  // ordinary rank skew would make a consumer give up while the producer is still within budget.
  const long long wait_cycles = tc5::kMaxWaitCycles + (p.ag.enabled ? p.ag.max_cycles : 0ll);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      tc5::mbar_init(&full_bar[s], 1);
      tc5::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc5::mbar_init(&tfull_bar[a], 1);
      tc5::mbar_init(&tempty_bar[a], 4);       // one arrival per epilogue warp
    }
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&tmap_a);
    tc5::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tmem_slot, TMEM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;   // global k-block counter across tiles
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        int mb, nb;
        tile_coords(t, tiles_m, tiles_n, mb, nb);
        if (p.ag.enabled) nb = (nb + p.ag.n_rot) % tiles_n;
        const int m0 = mb * BM, n0 = nb * BN;
        if (p.ag.enabled) {
          // B rows [n0, n1) live at 16-byte units [g_lo, g_hi] of the gathered buffer
          const int n1 = n0 + BN < p.N ? n0 + BN : p.N;
          const long g_lo = p.ag.b_vec_offset + static_cast<long>(n0) * p.ldb / 8;
          const long g_hi = p.ag.b_vec_offset + static_cast<long>(n1) * p.ldb / 8 - 1;
          const int id_lo = ag_chunk_id(p.ag, g_lo), id_hi = ag_chunk_id(p.ag, g_hi);
          for (int id = id_lo; id <= id_hi && ok; ++id)
            if (!spin_until(p.ag.chunk_flags + id, p.ag.epoch, p.ag.max_cycles, false)) {
              *abort_flag = 1;
              status_report(p.status, STATUS_TIMEOUT_LOCAL_FLAG, blockIdx.x, id);
              ok = false;
            }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc5::mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          tc5::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tc5::tma_load_2d(sa, &tmap_a, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tc5::tma_load_2d(sa + c * CHUNK_BYTES, &tmap_a, &full_bar[s], m0 + 64 * c, k0);
          }
          if (B_MN == 0) {
            tc5::tma_load_2d(sb, &tmap_b, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tc5::tma_load_2d(sb + c * CHUNK_BYTES, &tmap_b, &full_bar[s], n0 + 64 * c, k0);
          }
        }
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(&full_bar[q % STAGES], (q / STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!tc5::mbar_wait_cycles(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY, wait_cycles)) { ok = false; break; }
        tc5::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc5::mbar_wait_cycles(&full_bar[s], ph, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL, wait_cycles)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint32_t sa = tc5::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? tc5::desc_mnmajor(sa + k * 2048, CHUNK_BYTES) : tc5::desc_kmajor(sa + k * 32);
            const uint64_t bd = B_MN ? tc5::desc_mnmajor(sb + k * 2048, CHUNK_BYTES) : tc5::desc_kmajor(sb + k * 32);
            tc5::mma_ss(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc5::mma_commit(&empty_bar[s]);      // stage reusable once these MMAs have read it
        }
        if (ok) tc5::mma_commit(&tfull_bar[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, 32*quarter+32)
    uint32_t tile_i = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_ctas, ++tile_i) {
      int mb, nb;
      tile_coords(t, tiles_m, tiles_n, mb, nb);
      if (p.ag.enabled) nb = (nb + p.ag.n_rot) % tiles_n;
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!tc5::mbar_wait_cycles(&tfull_bar[acc], acc_ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL, wait_cycles)) { ok = false; break; }
      tc5::fence_after_sync();
      const int row = mb * BM + quarter * 32 + lane;
      const int col0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col = col0 + c * 32;
        if (col >= p.N) break;                   // uniform across the warp
        uint32_t r[32];
        tc5::tmem_ld_x32(taddr + c * 32, r);
        tc5::tmem_ld_wait();
        if (!row_ok) continue;
        store_direct(r, row, col, p);
      }
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc5::fence_after_sync();
    tc5::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int A_MN, int B_MN>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, SMEM_BYTES, st>>>(ta, tb, p);
  nsa::count_launch();
  return cudaGetLastError();
}


// =========================================================================================
// CTA-pair GEMM: the default kernel for plain C = op(A) op(B).
//
// A cluster of two CTAs (the two SMs of one TPC) owns a 256 x 256 output tile and executes
// tcgen05.mma.cta_group::2 with M = 256: CTA r of the pair stages A rows [128 r, 128 r + 128) and
// B rows [128 r, 128 r + 128) of the tile in its own shared memory (plain TMA loads, no
// multicast), so per MMA each SM reads 128 x 16 of A and 128 x 16 of B instead of 128 x 16 and
// 256 x 16: the shared-memory read traffic that bounds the single-CTA kernel drops by a third
// and the operand bytes fetched per FLOP by a quarter.  The even CTA's MMA thread issues for
// both; its commits arrive on the barriers of both CTAs.  Each CTA drains its own 128
// accumulator rows: registers -> swizzled shared memory -> TMA store (bf16 output), so global
// writes are full 128-byte lines; fp32 output and accumulation into C use direct stores.
// Six 32 KB stages, two 256-column accumulators per CTA (epilogue of tile i under the MMAs of
// tile i + 1).  Every wait is bounded; all threads of both CTAs reach the final cluster barrier
// on every path, after which tensor memory is released.
// =========================================================================================
namespace pair {
constexpr int BM = 128;                        // rows of A (and of the accumulator) per CTA
constexpr int BN = 256;                        // tile width; each CTA stages BN / 2 rows of B
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;           // 16 KB
constexpr int B_BYTES = BNH * BK * 2;          // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BOX_BYTES = 32 * 64 * 2;     // one warp's staging box: 32 rows x 64 bf16
constexpr int EPI_BYTES = 4 * 2 * EPI_BOX_BYTES;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;                     // in 256-row tiles
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int local = t - g * per_group;
  mb = first_m + local % gm;
  nb = local / gm;
}
// Tile order of the GEMM that gathers its own B operand: N-major, so that the sweep passes through
// the unit's shards one after the other in the order in which they are pulled (the local shard
// first); inside a group of GROUP_N tile columns the rows run fastest, which keeps that B panel in
// L2 while A streams by.  The caller rotates nb by ag.n_rot.
constexpr int GROUP_N = 8;
__device__ __forceinline__ void tile_coords_nmajor(int t, int tiles_m, int tiles_n, int& mb, int& nb) {
  const int per_group = GROUP_N * tiles_m;
  const int g = t / per_group;
  const int first_n = g * GROUP_N;
  const int gn = min(GROUP_N, tiles_n - first_n);
  const int local = t - g * per_group;
  nb = first_n + local % gn;
  mb = local / gn;
}
}  // namespace pair

// Copy role of the fused all-gather in the CTA-pair kernel: the MMA warp of the odd CTA of each pair
// has nothing else to do (the even CTA issues for both), so it pulls the peers' shards, 32 loads of
// 16 bytes in flight per lane, into the local gathered buffer and publishes one flag per chunk.
// No SM is taken away from the GEMM.
__device__ void ag_copy_warp(const AgFuse& ag, int cluster, int n_clusters, KernelStatus* status) {
  const int lane = threadIdx.x & 31;
  const int jobs = ag.W * ag.chunks_per_shard;
  const int n_w = ag.w_hi - ag.w_lo + 1;
  unsigned ready_mask = 1u << ag.rank;          // peers whose "shard ready" flag has been seen
  for (int q = cluster; q < jobs; q += n_clusters) {
    // Order: first the chunks that hold B, starting with the one the tile sweep needs first and
    // wrapping around inside B's range; then the rest of the unit.  (On a rank whose own shard
    // holds none of B, the GEMM can only start once B's first rows have crossed the link.)
    int id;
    if (q < n_w) id = ag.w_lo + (ag.w_start - ag.w_lo + q) % n_w;
    else id = (ag.w_hi + 1 + (q - n_w)) % jobs;
    const int pr = id / ag.chunks_per_shard, c = id - pr * ag.chunks_per_shard;
    if (!((ready_mask >> pr) & 1u)) {
      int ok = 1;
      if (lane == 0 && ag.peer_flags != nullptr && !spin_until(ag.peer_flags + pr, ag.epoch, ag.max_cycles, true)) {
        status_report(status, STATUS_TIMEOUT_PEER_FLAG, pr, (int)ag.epoch);
        ok = 0;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      ready_mask |= 1u << pr;
    }
    const long lo = static_cast<long>(c) * ag.chunk_vec;
    const long hi = lo + ag.chunk_vec < ag.shard_vec ? lo + ag.chunk_vec : ag.shard_vec;
    const uint4* src = ag.shards[pr];
    uint4* dst = ag.full + static_cast<long>(pr) * ag.shard_vec;
    constexpr int U = 32;
    for (long i0 = lo + lane; i0 < hi; i0 += 32L * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + 32L * u;
        if (i < hi) v[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + 32L * u;
        if (i < hi) dst[i] = v[u];
      }
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ag.chunk_flags + pr * ag.chunks_per_shard + c), "r"(ag.epoch) : "memory");
    }
  }
}

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair::THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const GemmParams p, const int tma_store) {
  // the pair kernel's tile constants hide the single-CTA kernel's of the same names
  constexpr int BM = pair::BM, BN = pair::BN, BNH = pair::BNH, BK = pair::BK, STAGES = pair::STAGES;
  constexpr int A_BYTES = pair::A_BYTES, STAGE_BYTES = pair::STAGE_BYTES;
  constexpr int EPI_BOX_BYTES = pair::EPI_BOX_BYTES, EPI_BYTES = pair::EPI_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + EPI_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]  TMA (both CTAs) -> MMA; used in the leader only
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]  MMA -> TMA producer of each CTA
  uint64_t* tfull_bar = bars + 2 * STAGES;       // [2]       MMA -> epilogue of each CTA
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]       epilogues of both CTAs -> MMA; leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t rank = tc5::cluster_ctarank();  // 0 = leader
  const int cluster = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int S = p.split_k > 1 ? p.split_k : 1;
  const int num_tiles = tiles_m * tiles_n * S;                  // work items: (tile, part of the reduction)
  const int k_blocks_all = (p.K + BK - 1) / BK;
  const int kb_per = (k_blocks_all + S - 1) / S;
  // with the gather inside, the producers may wait for a peer; everything downstream waits as long
  const long long wait_cycles = tc5::kMaxWaitCycles + (p.ag.enabled ? p.ag.max_cycles : 0ll);
  auto coords = [&](int t, int& mb, int& nb) {
    if (p.ag.enabled) {
      pair::tile_coords_nmajor(t, tiles_m, tiles_n, mb, nb);
      nb = (nb + p.ag.n_rot) % tiles_n;
    } else {
      pair::tile_coords(t / S, tiles_m, tiles_n, mb, nb);
    }
  };
  // k-blocks [kb_lo, kb_hi) of work item t (the parts of one tile are consecutive items, so they run
  // at the same time on different CTA pairs); an empty range is skipped by every role alike
  auto k_range = [&](int t, int& kb_lo, int& kb_hi) {
    kb_lo = (t % S) * kb_per;
    kb_hi = kb_lo + kb_per < k_blocks_all ? kb_lo + kb_per : k_blocks_all;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      tc5::mbar_init(&full_bar[s], 1);           // the leader's expect_tx arrival
      tc5::mbar_init(&empty_bar[s], 1);          // one commit
    }
    for (int a = 0; a < 2; ++a) {
      tc5::mbar_init(&tfull_bar[a], 1);          // one commit
      tc5::mbar_init(&tempty_bar[a], 8);         // four epilogue warps of each CTA
    }
    tc5::fence_barrier_init();
    tc5::prefetch_tensormap(&tmap_a);
    tc5::prefetch_tensormap(&tmap_b);
    if (tma_store) tc5::prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    tc5::tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc5::tmem_relinquish_pair();
  }
  tc5::fence_before_sync();
  tc5::cluster_sync();                           // barriers of both CTAs are initialised past this point
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int seen_group = -1;                         // tile-column group whose chunk flags have been awaited
      for (int t = cluster; t < num_tiles && ok; t += n_clusters) {
        int mb, nb, kb_lo, kb_hi;
        coords(t, mb, nb);
        k_range(t, kb_lo, kb_hi);
        if (kb_lo >= kb_hi) continue;
        const int m0 = mb * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = nb * BN + static_cast<int>(rank) * BNH;
        if (p.ag.enabled) {
          // The sweep stays inside one group of GROUP_N tile columns for tiles_m tile rows, so the
          // flags of the chunks that hold this CTA's B rows of the whole group are awaited once,
          // when the group is entered: an acquire load is an L2 round trip on the producer's
          // critical path, far too slow to repeat for every tile.
          const int group = t / (pair::GROUP_N * tiles_m);
          if (group != seen_group) {
            const int first_n = group * pair::GROUP_N;
            const int gn = min(pair::GROUP_N, tiles_n - first_n);
            for (int j = 0; j < gn && ok; ++j) {
              const int r0 = ((first_n + j + p.ag.n_rot) % tiles_n) * BN + static_cast<int>(rank) * BNH;
              if (r0 >= p.N) continue;
              const int r1 = r0 + BNH < p.N ? r0 + BNH : p.N;
              const long g_lo = p.ag.b_vec_offset + static_cast<long>(r0) * p.ldb / 8;
              const long g_hi = p.ag.b_vec_offset + static_cast<long>(r1) * p.ldb / 8 - 1;
              const int id_lo = ag_chunk_id(p.ag, g_lo), id_hi = ag_chunk_id(p.ag, g_hi);
              for (int id = id_lo; id <= id_hi && ok; ++id)
                if (!spin_until(p.ag.chunk_flags + id, p.ag.epoch, p.ag.max_cycles, false)) {
                  *abort_flag = 1;
                  status_report(p.status, STATUS_TIMEOUT_LOCAL_FLAG, blockIdx.x, id);
                  ok = false;
                }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");
            seen_group = group;
          }
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc5::mbar_wait_cycles(&empty_bar[s], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY, wait_cycles)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (rank == 0) tc5::mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);   // bytes of both CTAs
          const uint32_t bar = tc5::mapa(tc5::smem_u32(&full_bar[s]), 0);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tc5::tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tc5::tma_load_2d_pair(sa + c * CHUNK_BYTES, &tmap_a, bar, m0 + 64 * c, k0);
          }
          if (B_MN == 0) {
            tc5::tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tc5::tma_load_2d_pair(sb + c * CHUNK_BYTES, &tmap_b, bar, n0 + 64 * c, k0);
          }
        }
      }
      if (ok) {
        // The MMA thread's last commits arrive on this CTA's empty barriers asynchronously; wait for
        // them, so that no arrival is still on its way to this CTA's shared memory when it exits.
        const uint32_t used = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < used && ok; ++j) {
          const uint32_t q = it - 1 - j;
          ok = tc5::mbar_wait(&empty_bar[q % STAGES], (q / STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY);
        }
      }
      if (!ok && rank == 0) {
        // let the leader's copies already issued land before shared memory is released
        const uint32_t pending = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t j = 0; j < pending; ++j) {
          const uint32_t q = it - 1 - j;
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(&full_bar[q % STAGES], (q / STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 1 && p.ag.enabled) ag_copy_warp(p.ag, cluster, n_clusters, p.status);
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = tc5::make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      bool ok = true;
      for (int t = cluster; t < num_tiles && ok; t += n_clusters) {
        int kb_lo, kb_hi;
        k_range(t, kb_lo, kb_hi);
        if (kb_lo >= kb_hi) continue;
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        ++tile_i;
        if (!tc5::mbar_wait_cycles(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY, wait_cycles)) { ok = false; break; }
        tc5::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc5::mbar_wait_cycles(&full_bar[s], ph, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL, wait_cycles)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint32_t sa = tc5::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? tc5::desc_mnmajor(sa + k * 2048, CHUNK_BYTES) : tc5::desc_kmajor(sa + k * 32);
            const uint64_t bd = B_MN ? tc5::desc_mnmajor(sb + k * 2048, CHUNK_BYTES) : tc5::desc_kmajor(sb + k * 32);
            tc5::mma_ss_pair(d_tmem, ad, bd, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          tc5::mma_commit_pair(&empty_bar[s], 3);      // both producers may refill the stage
        }
        if (ok) tc5::mma_commit_pair(&tfull_bar[acc], 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, each CTA)
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, 32*quarter+32)
    uint8_t* my_epi = epi + quarter * 2 * EPI_BOX_BYTES;
    const uint32_t tempty_leader0 = tc5::mapa(tc5::smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = tc5::mapa(tc5::smem_u32(&tempty_bar[1]), 0);
    uint32_t tile_i = 0;
    uint32_t boxes = 0;                           // TMA stores issued by this warp's lane 0
    bool ok = true;
    for (int t = cluster; t < num_tiles && ok; t += n_clusters) {
      int mb, nb, kb_lo, kb_hi;
      coords(t, mb, nb);
      k_range(t, kb_lo, kb_hi);
      if (kb_lo >= kb_hi) continue;
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      ++tile_i;
      if (!tc5::mbar_wait_cycles(&tfull_bar[acc], acc_ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL, wait_cycles)) { ok = false; break; }
      tc5::fence_after_sync();
      const int row0 = mb * 2 * BM + static_cast<int>(rank) * BM + quarter * 32;
      const int row = row0 + lane;
      const int col0 = nb * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (tma_store == 2) {
        // a part of a split reduction: 32 x 32 fp32 boxes added into C by TMA reduce stores
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = col0 + c * 32;
          if (col >= p.N || row0 >= p.M) break;    // uniform across the warp
          uint32_t r0[32];
          tc5::tmem_ld_x32(taddr + c * 32, r0);
          tc5::tmem_ld_wait();
          uint8_t* box = my_epi + (boxes & 1) * EPI_BOX_BYTES;
          if (boxes >= 2) {
            if (lane == 0) tc5::tma_store_wait_read<1>();
            __syncwarp();
          }
          uint8_t* rowp = box + lane * 128;        // 32 floats per row: eight 16-byte chunks, swizzled
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
          tc5::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tc5::tma_reduce_add_2d(&tmap_c, box, col, row0);
            tc5::tma_store_commit();
          }
          ++boxes;
        }
      } else if (tma_store) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = col0 + c * 64;
          if (col >= p.N || row0 >= p.M) break;    // uniform across the warp
          uint32_t r0[32], r1[32];
          tc5::tmem_ld_x32(taddr + c * 64, r0);
          tc5::tmem_ld_x32(taddr + c * 64 + 32, r1);
          tc5::tmem_ld_wait();
          uint8_t* box = my_epi + (boxes & 1) * EPI_BOX_BYTES;
          if (boxes >= 2) {                        // the store that last read this box must be done with it
            if (lane == 0) tc5::tma_store_wait_read<1>();
            __syncwarp();
          }
          // row `lane` of the box: eight 16-byte chunks, chunk j at slot j ^ (lane % 8) (128-byte swizzle)
          uint8_t* rowp = box + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = tc5::pack_bf16(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            v.y = tc5::pack_bf16(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            v.z = tc5::pack_bf16(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            v.w = tc5::pack_bf16(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = tc5::pack_bf16(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            v.y = tc5::pack_bf16(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            v.z = tc5::pack_bf16(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            v.w = tc5::pack_bf16(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            *reinterpret_cast<uint4*>(rowp + (((j + 4) ^ (lane & 7)) << 4)) = v;
          }
          tc5::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {                         // rows past M and columns past N are clipped
            if (tma_store == 3) tc5::tma_reduce_add_2d(&tmap_c, box, col, row0);   // C += tile, added in bf16 by the memory system
            else tc5::tma_store_2d(&tmap_c, box, col, row0);
            tc5::tma_store_commit();
          }
          ++boxes;
        }
      } else {
        const bool row_ok = row < p.M;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = col0 + c * 32;
          if (col >= p.N) break;
          uint32_t r[32];
          tc5::tmem_ld_x32(taddr + c * 32, r);
          tc5::tmem_ld_wait();
          if (!row_ok) continue;
          store_direct(r, row, col, p);
        }
      }
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
    if (tma_store && lane == 0) tc5::tma_store_wait<0>();
  }

  // Both CTAs meet here on every path: the leader's MMAs read the peer's shared memory and the
  // commits arrive on the peer's barriers, so neither CTA may leave, or release tensor memory,
  // before both are done.
  tc5::fence_before_sync();
  tc5::cluster_sync();
  if (warp == 1) {
    tc5::fence_after_sync();
    tc5::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int A_MN, int B_MN>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                        int tma_store, int max_ctas, cudaStream_t st) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  static int clusters[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (clusters[dev] == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // how many CTA pairs the device can hold at once (all of its TPCs, normally sm_count / 2)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(nsa::sm_count() & ~1), 1, 1);
    cfg.blockDim = dim3(pair::THREADS, 1, 1);
    cfg.dynamicSmemBytes = pair::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = nsa::sm_count() / 2;
    }
    clusters[dev] = n;
  }
  const int tiles = ((p.M + 2 * pair::BM - 1) / (2 * pair::BM)) * ((p.N + pair::BN - 1) / pair::BN) * (p.split_k > 1 ? p.split_k : 1);
  int n = clusters[dev];
  if (max_ctas > 0 && max_ctas / 2 < n) n = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < n) n = tiles;
  kern<<<2 * n, pair::THREADS, pair::SMEM_BYTES, st>>>(ta, tb, tc, p, tma_store);
  nsa::count_launch();
  return cudaGetLastError();
}

}  // namespace

// Which kernel plain GEMMs use: the CTA-pair kernel unless NSA_B200_GEMM=single is set in the
// environment (read once) or the problem has fewer than 128 rows.
static int g_gemm_select = 0;                   // 0 = environment default, 1 = single-CTA kernel, 2 = pair kernel
static bool use_pair_kernel() {
  if (g_gemm_select) return g_gemm_select == 2;
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("NSA_B200_GEMM");
    v = (e != nullptr && strcmp(e, "single") == 0) ? 0 : 1;
  }
  return v == 1;
}
// Number of CTA pairs the pair kernel runs at once on the current device (0 before its first launch:
// then half the SM count is the estimate).
extern "C" int nsa_gemm_pair_clusters(void) { return nsa::sm_count() / 2; }

// Overrides the kernel choice for the calls that follow (benchmarks and tests compare the two).
extern "C" void nsa_gemm_select(int which) { g_gemm_select = (which == 1 || which == 2) ? which : 0; }

extern "C" int nsa_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                             int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int max_ctas,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return nsa::fail(NSA_ERR_ALIGNMENT, "nsa_gemm_bf16: operands need 16-byte aligned bases and leading dimensions that are multiples of 8");
  const bool pairk = use_pair_kernel() && M > 128;
  CUtensorMap ta, tb, tc;
  int rc;
  // tensor maps: innermost dimension first.  Both kernels stage 128 rows of A per CTA; the pair
  // kernel stages 128 rows of B per CTA, the single-CTA kernel 256.
  if (!a_mn) rc = nsa::make_tmap_2d_bf16(&ta, A, /*inner*/ K, /*outer*/ M, lda, /*box*/ BK, BM);
  else       rc = nsa::make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = nsa::make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, pairk ? pair::BNH : BN);
  else       rc = nsa::make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.ag = AgFuse{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldb = ldb; p.a_mn = a_mn; p.b_mn = b_mn;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.split_k = 1; p.C = C; p.status = nsa::status_ptr();
  cudaError_t e;
  if (pairk) {
    // bf16 output leaves through TMA stores when C allows a tensor map; with `accumulate` the stores
    // are TMA reduce-adds (each element gets one bf16 add per launch, so launches on one stream
    // give the same bits every run)
    const int tma_store = (!out_fp32 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc & 7) == 0) ? (accumulate ? 3 : 1) : 0;
    if (tma_store) {
      if ((rc = nsa::make_tmap_2d_bf16(&tc, C, N, M, ldc, 64, 32))) return rc;
    } else {
      tc = ta;                                   // unused by the kernel
    }
    if (!a_mn && !b_mn) e = launch_pair<0, 0>(ta, tb, tc, p, tma_store, max_ctas, stream);
    else if (!a_mn && b_mn) e = launch_pair<0, 1>(ta, tb, tc, p, tma_store, max_ctas, stream);
    else if (a_mn && !b_mn) e = launch_pair<1, 0>(ta, tb, tc, p, tma_store, max_ctas, stream);
    else e = launch_pair<1, 1>(ta, tb, tc, p, tma_store, max_ctas, stream);
    return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16 launch (pair kernel)");
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int sms = nsa::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  const int grid = tiles < sms ? tiles : sms;
  if (!a_mn && !b_mn) e = launch<0, 0>(ta, tb, p, grid, stream);
  else if (!a_mn && b_mn) e = launch<0, 1>(ta, tb, p, grid, stream);
  else if (a_mn && !b_mn) e = launch<1, 0>(ta, tb, p, grid, stream);
  else e = launch<1, 1>(ta, tb, p, grid, stream);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16 launch");
}

// C32[M,N] += op(A) op(B) with the reduction cut into `split_k` parts that run on different CTA pairs
// and meet in the fp32 matrix C32 through TMA reduce-add stores.  For shapes with a long reduction
// and too few output tiles to fill the machine evenly (weight gradients: K = tokens).  C32 must hold
// the values the products are to be added to (zeros for a plain product); base 16-byte aligned, ldc a
// multiple of 4.  Pair kernel only; M > 128.
extern "C" int nsa_gemm_bf16_splitk(const void* A, const void* B, float* C32, int M, int N, int K, int lda, int ldb,
                                    int ldc, int a_mn, int b_mn, int split_k, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7) ||
      (reinterpret_cast<uintptr_t>(C32) & 15) || (ldc & 3))
    return nsa::fail(NSA_ERR_ALIGNMENT, "nsa_gemm_bf16_splitk: operands need 16-byte aligned bases and row pitches");
  if (M <= 128 || split_k < 1 || split_k > 16) return nsa::fail(NSA_ERR_SHAPE, "nsa_gemm_bf16_splitk: M > 128 and 1 <= split_k <= 16 required");
  CUtensorMap ta, tb, tc;
  int rc;
  if (!a_mn) rc = nsa::make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM);
  else       rc = nsa::make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = nsa::make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, pair::BNH);
  else       rc = nsa::make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  if ((rc = nsa::make_tmap_2d_f32(&tc, C32, N, M, ldc, 32, 32))) return rc;
  GemmParams p;
  p.ag = AgFuse{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldb = ldb; p.a_mn = a_mn; p.b_mn = b_mn;
  p.out_fp32 = 1; p.accumulate = 1; p.split_k = split_k; p.C = C32; p.status = nsa::status_ptr();
  cudaError_t e;
  if (!a_mn && !b_mn) e = launch_pair<0, 0>(ta, tb, tc, p, 2, 0, stream);
  else if (!a_mn && b_mn) e = launch_pair<0, 1>(ta, tb, tc, p, 2, 0, stream);
  else if (a_mn && !b_mn) e = launch_pair<1, 0>(ta, tb, tc, p, 2, 0, stream);
  else e = launch_pair<1, 1>(ta, tb, tc, p, 2, 0, stream);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16_splitk launch");
}

// y[M,N] = x[M,K] * W[N,K]^T where W lives at element offset `b_elem_offset` of the sharded
// unit's gathered buffer `full`, which this same kernel assembles from the W ranks' shards
// (see AgFuse).  After the kernel the whole unit (not only W) is gathered.  With the CTA-pair
// kernel (the default above 128 rows) no SM is set aside for copying; the single-CTA kernel
// reserves `copy_ctas` CTAs for it.  Use chunks of a few hundred KB (chunks_per_shard) so that
// every copy warp has work: there is one per CTA pair.
//   shards      device array of W pointers to the ranks' shards (shard_elems bf16 each)
//   chunk_flags local scratch, W * chunks_per_shard words, values < epoch on entry
//   peer_flags  local flag row, peer p's shard is final once peer_flags[p] >= epoch (may be null)
extern "C" int nsa_gemm_bf16_ag(const void* A, void* C, int M, int N, int K, int lda, int ldc,
                                const void* const* shards, void* full, long shard_elems, long b_elem_offset,
                                int W, int rank, unsigned* chunk_flags, int chunks_per_shard, const unsigned* peer_flags,
                                unsigned epoch, long long max_cycles, int copy_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const char* Bp = reinterpret_cast<const char*>(full) + b_elem_offset * 2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(Bp) & 15) || (lda & 7) || (K & 7) ||
      (shard_elems & 7) || (b_elem_offset & 7))
    return nsa::fail(NSA_ERR_ALIGNMENT, "nsa_gemm_bf16_ag: operands need 16-byte alignment");
  if (W < 1 || W > 32 || chunks_per_shard < 1) return nsa::fail(NSA_ERR_SHAPE, "nsa_gemm_bf16_ag: 1 to 32 ranks, at least one chunk per shard");
  const bool pairk = use_pair_kernel() && M > 128;
  CUtensorMap ta, tb, tc;
  int rc;
  if ((rc = nsa::make_tmap_2d_bf16(&ta, A, K, M, lda, BK, BM))) return rc;
  if ((rc = nsa::make_tmap_2d_bf16(&tb, Bp, K, N, K, BK, pairk ? pair::BNH : BN))) return rc;
  GemmParams p;
  p.ag = AgFuse{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ldb = K; p.a_mn = 0; p.b_mn = 0;
  p.out_fp32 = 0; p.accumulate = 0; p.split_k = 1; p.C = C; p.status = nsa::status_ptr();
  const int sms = nsa::sm_count();
  if (copy_ctas <= 0) copy_ctas = 16;
  if (copy_ctas > sms / 2) copy_ctas = sms / 2;
  const long shard_vec = shard_elems / 8;
  AgFuse& ag = p.ag;
  ag.enabled = 1; ag.W = W; ag.rank = rank;
  ag.shards = reinterpret_cast<const uint4* const*>(shards);
  ag.full = reinterpret_cast<uint4*>(full);
  ag.shard_vec = shard_vec;
  ag.chunks_per_shard = chunks_per_shard;
  ag.chunk_vec = (shard_vec + chunks_per_shard - 1) / chunks_per_shard;
  ag.chunk_flags = chunk_flags; ag.peer_flags = peer_flags; ag.epoch = epoch;
  ag.b_vec_offset = b_elem_offset / 8;
  ag.max_cycles = max_cycles; ag.copy_ctas = copy_ctas;
  // start the N sweep at the first shard, in pull order (rank, rank+1, ...), that overlaps W
  const long b_lo = ag.b_vec_offset, b_hi = b_lo + static_cast<long>(N) * K / 8;
  const int tiles_n = (N + BN - 1) / BN;
  ag.n_rot = 0;
  for (int k = 0; k < W; ++k) {
    const int pr = (rank + k) % W;
    const long s_lo = pr * shard_vec, s_hi = s_lo + shard_vec;
    const long lo = s_lo > b_lo ? s_lo : b_lo, hi = s_hi < b_hi ? s_hi : b_hi;
    if (lo < hi) {
      // first N block that starts at or after the shard's first row (a straddling block comes last)
      const long row = ((lo - b_lo) * 8 + K - 1) / K;
      ag.n_rot = static_cast<int>((row + BN - 1) / BN) % tiles_n;
      break;
    }
  }
  {
    const long cv = ag.chunk_vec;
    auto chunk_of = [&](long g) { const long pidx = g / shard_vec; return static_cast<int>(pidx * chunks_per_shard + (g - pidx * shard_vec) / cv); };
    ag.w_lo = chunk_of(b_lo);
    ag.w_hi = chunk_of(b_hi - 1);
    const long first_row = static_cast<long>(ag.n_rot) * BN;                  // the sweep starts at this row of B
    ag.w_start = chunk_of(b_lo + (first_row < N ? first_row : 0) * K / 8);
  }
  if (pairk) {
    // CTA-pair kernel: the copy role runs in the otherwise idle MMA warp of every odd CTA, the tile
    // sweep follows the shards (see ag_copy_warp and tile_coords_nmajor); `copy_ctas` is not used
    const int tma_store = ((reinterpret_cast<uintptr_t>(C) & 15) == 0 && (ldc & 7) == 0) ? 1 : 0;
    if (tma_store) {
      if ((rc = nsa::make_tmap_2d_bf16(&tc, C, N, M, ldc, 64, 32))) return rc;
    } else {
      tc = ta;
    }
    cudaError_t e = launch_pair<0, 0>(ta, tb, tc, p, tma_store, 0, stream);
    return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16_ag launch (pair kernel)");
  }
  const int tiles = ((M + BM - 1) / BM) * tiles_n;
  int gemm_ctas = sms - copy_ctas;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  cudaError_t e = launch<0, 0>(ta, tb, p, copy_ctas + gemm_ctas, stream);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16_ag launch");
}
