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

struct GemmParams {
  int M, N, K;
  int ldc;
  int a_mn, b_mn;
  int out_fp32;
  int accumulate;
  void* C;
  KernelStatus* status;
};

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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;

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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, tiles_m, tiles_n, mb, nb);
        const int m0 = mb * BM, n0 = nb * BN;
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!tc5::mbar_wait(&tempty_bar[acc], acc_ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc5::fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!tc5::mbar_wait(&full_bar[s], ph, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
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
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
      int mb, nb;
      tile_coords(t, tiles_m, tiles_n, mb, nb);
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!tc5::mbar_wait(&tfull_bar[acc], acc_ph, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
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
        const bool full = (col + 32 <= p.N);
        if (p.out_fp32) {
          float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col;
          if (full && (p.ldc & 3) == 0) {
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
          if (full && (p.ldc & 7) == 0 && !p.accumulate) {
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

}  // namespace

extern "C" int nsa_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                             int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int max_ctas,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return nsa::fail(NSA_ERR_ALIGNMENT, "nsa_gemm_bf16: operands need 16-byte aligned bases and leading dimensions that are multiples of 8");
  CUtensorMap ta, tb;
  int rc;
  // tensor maps: innermost dimension first
  if (!a_mn) rc = nsa::make_tmap_2d_bf16(&ta, A, /*inner*/ K, /*outer*/ M, lda, /*box*/ BK, BM);
  else       rc = nsa::make_tmap_2d_bf16(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = nsa::make_tmap_2d_bf16(&tb, B, K, N, ldb, BK, BN);
  else       rc = nsa::make_tmap_2d_bf16(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.a_mn = a_mn; p.b_mn = b_mn;
  p.out_fp32 = out_fp32; p.accumulate = accumulate; p.C = C; p.status = nsa::status_ptr();
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int sms = nsa::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  const int grid = tiles < sms ? tiles : sms;
  cudaError_t e;
  if (!a_mn && !b_mn) e = launch<0, 0>(ta, tb, p, grid, stream);
  else if (!a_mn && b_mn) e = launch<0, 1>(ta, tb, p, grid, stream);
  else if (a_mn && !b_mn) e = launch<1, 0>(ta, tb, p, grid, stream);
  else e = launch<1, 1>(ta, tb, p, grid, stream);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gemm_bf16 launch");
}
