// Gated DeltaNet: the sequential (inter-chunk) part of the chunkwise gated delta rule,
// forward and backward, on tcgen05 tensor cores with the K x V state resident in tensor
// memory.  Chunk length 64, key width 128, value width a multiple of 64.
//
// Per head, with S the K x V state entering chunk c (fp32), and per-chunk inputs prepared by
// the parallel pre-pass (w, q_dec, k_tail: 64 x K; u: 64 x V; gamma = exp(total log-decay)):
//     v_new   = u - w S                 o_inter = q_dec S
//     S_next  = gamma S + k_tail^T v_new
// One CTA owns one (head, 64-wide V tile) and walks the chunks in order.  Each step is two
// MMA groups: D1[128 x 64] = [w ; q_dec] * S  and  S += k_tail^T * v_new, with S kept in TMEM
// as fp32 and mirrored to shared memory as the bf16 B operand of the next step.  Operand
// tiles for chunk c+1 arrive by TMA while chunk c computes.
//
// Backward walks the chunks in reverse with dS (K x 64 tile) in TMEM:
//     dv_tot  = dv_new + k_tail dS              du      = dv_tot
//     dk_tail = v_new dS^T   (partial over V tiles)
//     dw      = -dv_tot S^T  (partial)          dq_dec  = do S^T  (partial)
//     dgamma  = <S, dS>      (partial)
//     dS_prev = gamma dS + q_dec^T do - w^T dv_tot
// Partials are written per V tile and summed by the caller (deterministic).
#include "host.cuh"
#include "tc5.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int KD = 128;   // key width
constexpr int VT = 64;    // V tile per CTA
constexpr int CH = 64;    // chunk length
constexpr int BOX = 8192; // bytes of one [64 rows][64 bf16] swizzled box

__device__ __forceinline__ void write_row_swz(uint8_t* tile, int row, const uint32_t (&packed)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    *reinterpret_cast<uint4*>(tile + row * 128 + ((j ^ (row & 7)) << 4)) = v;
  }
}
__device__ __forceinline__ void read_row_swz(const uint8_t* tile, int row, float (&out)[64]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v = *reinterpret_cast<const uint4*>(tile + row * 128 + ((j ^ (row & 7)) << 4));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      out[8 * j + 2 * k] = f.x;
      out[8 * j + 2 * k + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void load_row_global(const bf16* src, uint32_t (&packed)[32]) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v = s4[j];
    packed[4 * j] = v.x; packed[4 * j + 1] = v.y; packed[4 * j + 2] = v.z; packed[4 * j + 3] = v.w;
  }
}
__device__ __forceinline__ void store_row_global(bf16* dst, const uint32_t (&packed)[32]) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int j = 0; j < 8; ++j) d4[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
}
__device__ __forceinline__ void unpack_row(const uint32_t (&packed)[32], float (&out)[64]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&packed[j]));
    out[2 * j] = f.x;
    out[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void tmem_ld_row64(uint32_t taddr, float (&out)[64]) {
  uint32_t a[32], b[32];
  tc5::tmem_ld_x32(taddr, a);
  tc5::tmem_ld_x32(taddr + 32, b);
  tc5::tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) { out[j] = __uint_as_float(a[j]); out[32 + j] = __uint_as_float(b[j]); }
}
__device__ __forceinline__ void tmem_st_row64(uint32_t taddr, const float (&in)[64]) {
  uint32_t a[32], b[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) { a[j] = __float_as_uint(in[j]); b[j] = __float_as_uint(in[32 + j]); }
  tc5::tmem_st_x32(taddr, a);
  tc5::tmem_st_x32(taddr + 32, b);
  tc5::tmem_st_wait();
}
__device__ __forceinline__ void pack_row(const float (&in)[64], uint32_t (&packed)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) packed[j] = tc5::pack_bf16(in[2 * j], in[2 * j + 1]);
}

struct FwdParams {
  const bf16* u;        // [BH, NC, 64, V]
  const float* gamma;   // [BH, NC]
  bf16* v_new;          // [BH, NC, 64, V]
  bf16* o_inter;        // [BH, NC, 64, V]  (rounded once here: it is added to a bf16 product next)
  bf16* S_all;          // [BH, NC, KD, V]  state entering each chunk
  int NC, V;
  KernelStatus* status;
};

constexpr int FWD_STAGE = 2 * 2 * BOX /*[w;qd] two k-blocks*/ + 2 * BOX /*k_tail*/;   // 48 KB
constexpr int FWD_SMEM = 2 * FWD_STAGE + 2 * BOX /*Sb*/ + BOX /*Vb*/ + BOX /*Ob*/ + 1024 + 128;

__global__ void __launch_bounds__(128, 1)
gdn_seq_fwd_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_qd,
                   const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_vn,
                   const __grid_constant__ CUtensorMap tm_oi, const __grid_constant__ CUtensorMap tm_sa,
                   const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* Sb = smem + 2 * FWD_STAGE;           // [KD rows][64] bf16, B operand of MMA1
  uint8_t* Vb = Sb + 2 * BOX;                   // [64 rows][64] bf16, B operand of MMA2
  uint8_t* Ob = Vb + BOX;                       // [64 rows][64] bf16: o_inter on its way out
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ob + BOX);
  uint64_t* full = bars;        // [2]
  uint64_t* m1 = bars + 2;
  uint64_t* m2 = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int r = threadIdx.x;               // TMEM lane / tile row owned by this thread
  const int warp = r >> 5;
  const int vt = blockIdx.x, bh = blockIdx.y;
  const int NC = p.NC, V = p.V;

  if (r == 0) {
    *abort_flag = 0;
    tc5::mbar_init(&full[0], 1);
    tc5::mbar_init(&full[1], 1);
    tc5::mbar_init(m1, 1);
    tc5::mbar_init(m2, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 128); tc5::tmem_relinquish(); }
  // S = 0: bf16 mirror in shared memory
  {
    uint32_t z[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) z[j] = 0u;
    write_row_swz(Sb, r, z);
  }
  tc5::fence_proxy_async();
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tD1 = tmem + lane_off;          // columns [0, 64)
  const uint32_t tS = tmem + lane_off + 64;      // columns [64, 128)
  {
    float z[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) z[j] = 0.f;
    tmem_st_row64(tS, z);
  }
  tc5::fence_before_sync();
  __syncthreads();
  // Outputs leave as TMA stores from the swizzled tiles they are in anyway (a thread owns a row, so
  // direct stores would be 32 separate 16-byte writes per instruction; they were a third of the
  // chunk loop).  One thread issues and waits; at most one store group stays pending across a point
  // where a tile is overwritten.  Chunk 0 enters with the zero state that Sb holds now.
  if (r == 0) {
    tc5::tma_store_2d(&tm_sa, Sb, vt * VT, bh * NC * KD);
    tc5::tma_store_commit();
  }

  auto issue_loads = [&](int c) {
    const int s = c & 1;
    uint8_t* st = smem + s * FWD_STAGE;
    const int row0 = (bh * NC + c) * CH;
    tc5::mbar_expect_tx(&full[s], FWD_STAGE);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tc5::tma_load_2d(st + kb * 2 * BOX, &tm_w, &full[s], kb * 64, row0);
      tc5::tma_load_2d(st + kb * 2 * BOX + BOX, &tm_qd, &full[s], kb * 64, row0);
      tc5::tma_load_2d(st + 4 * BOX + kb * BOX, &tm_kt, &full[s], kb * 64, row0);
    }
  };
  if (r == 0) issue_loads(0);

  constexpr uint32_t idesc1 = tc5::make_idesc_bf16(128, VT, 0, 1);   // A K-major, B MN-major
  constexpr uint32_t idesc2 = tc5::make_idesc_bf16(128, VT, 1, 1);   // A MN-major (k_tail^T), B MN-major
  bool ok = true;
  // The chunk loop is one dependent chain, so every global load in it would add its full latency to
  // every chunk: the u row and the decay of the next chunk are fetched one chunk ahead instead.
  uint32_t upk_next[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) upk_next[j] = 0u;
  if (r < CH) load_row_global(p.u + (static_cast<long>(bh * NC) * CH + r) * V + vt * VT, upk_next);
  float g_next = NC > 1 ? p.gamma[bh * NC + 1] : 0.f;
  for (int c = 0; c < NC && ok; ++c) {
    const int s = c & 1;
    uint8_t* st = smem + s * FWD_STAGE;
    const long row0 = static_cast<long>(bh * NC + c) * CH;
    uint32_t upk[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) upk[j] = upk_next[j];
    const float g = g_next;                        // decay applied to the state that enters chunk c + 1
    if (warp == 0) {
      // The issuing warp stays converged and one elected lane issues: descriptors then live in
      // uniform registers and an MMA costs the issuing thread a few cycles instead of 70 to 100,
      // which matters in a loop that is one dependent chain.
      const bool lead = tc5::elect_one();
      if (__all_sync(0xffffffffu, tc5::mbar_wait(&full[s], (c >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL))) {
        tc5::fence_after_sync();
        const uint64_t a1 = tc5::desc_kmajor(tc5::smem_u32(st)), sb = tc5::desc_mnmajor(tc5::smem_u32(Sb), BOX);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < KD / 16; ++kk)
            tc5::mma_ss(tmem, a1 + static_cast<uint64_t>(((kk >> 2) * 2 * BOX + (kk & 3) * 32) >> 4),
                        sb + static_cast<uint64_t>((kk * 2048) >> 4), idesc1, kk > 0 ? 1u : 0u);
          tc5::mma_commit(m1);
          if (c + 1 < NC) issue_loads(c + 1);
        }
      }
      __syncwarp();
    }
    // next chunk's u row (rows 0..63 only) and the decay after it, in flight while this chunk computes
    if (c + 1 < NC && r < CH) load_row_global(p.u + (row0 + CH + r) * V + vt * VT, upk_next);
    if (c + 2 < NC) g_next = p.gamma[bh * NC + c + 2];
    if (r == 0) tc5::tma_store_wait_read<1>();     // the previous chunk's v_new / o_inter tiles have been read
    if (!tc5::mbar_wait(m1, c & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; }
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    {
      float d1[64];
      tmem_ld_row64(tD1, d1);
      if (r < CH) {
        float uf[64];
        unpack_row(upk, uf);
#pragma unroll
        for (int j = 0; j < 64; ++j) d1[j] = uf[j] - d1[j];
        uint32_t pk[32];
        pack_row(d1, pk);
        write_row_swz(Vb, r, pk);
      } else {
        uint32_t pk[32];
        pack_row(d1, pk);
        write_row_swz(Ob, r - CH, pk);
      }
    }
    tc5::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    if (r == 0) {
      tc5::tma_store_2d(&tm_vn, Vb, vt * VT, static_cast<int>(row0));
      tc5::tma_store_2d(&tm_oi, Ob, vt * VT, static_cast<int>(row0));
      tc5::tma_store_commit();
    }
    if (warp == 0) {
      const bool lead = tc5::elect_one();
      tc5::fence_after_sync();
      const uint64_t kt = tc5::desc_mnmajor(tc5::smem_u32(st + 4 * BOX), BOX), vb = tc5::desc_mnmajor(tc5::smem_u32(Vb), BOX);
      if (lead) {
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)
          tc5::mma_ss(tmem + 64, kt + static_cast<uint64_t>((kk * 2048) >> 4), vb + static_cast<uint64_t>((kk * 2048) >> 4), idesc2, 1u);
        tc5::mma_commit(m2);
      }
      __syncwarp();
    }
    if (r == 0) tc5::tma_store_wait_read<1>();     // the previous state tile has been read
    if (!tc5::mbar_wait(m2, c & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; }
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    if (c + 1 < NC) {
      float sv[64];
      tmem_ld_row64(tS, sv);                       // S entering chunk c+1, row r
      uint32_t pk[32];
      pack_row(sv, pk);
      write_row_swz(Sb, r, pk);
#pragma unroll
      for (int j = 0; j < 64; ++j) sv[j] *= g;
      tmem_st_row64(tS, sv);
      tc5::fence_proxy_async();
    }
    tc5::fence_before_sync();
    __syncthreads();
    if (r == 0 && c + 1 < NC) {
      tc5::tma_store_2d(&tm_sa, Sb, vt * VT, (bh * NC + c + 1) * KD);
      tc5::tma_store_commit();
    }
  }
  if (r == 0) tc5::tma_store_wait_read<0>();
  if (!ok && r == 0) {
    // a load for the next chunk may still be in flight: give it a bounded chance to land
    const long long t0 = clock64();
    for (int s = 0; s < 2; ++s)
      for (uint32_t i = 0; i < (1u << 16); ++i) {
        if (tc5::mbar_try_wait(&full[s], 0) || tc5::mbar_try_wait(&full[s], 1)) break;
        if (clock64() - t0 > tc5::kMaxWaitCycles) break;
      }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 128); }
}

struct BwdParams {
  const bf16* v_new;     // [BH, NC, 64, V]
  const bf16* dv_new;    // [BH, NC, 64, V]  gradient arriving at v_new from the intra-chunk output term
  const bf16* d_o;       // [BH, NC, 64, V]  gradient of o_inter
  const float* gamma;    // [BH, NC]
  bf16* du;              // [BH, NC, 64, V]
  bf16* dw_part;         // [VTILES, BH, NC, 64, KD]
  bf16* dqd_part;        // [VTILES, BH, NC, 64, KD]
  bf16* dkt_part;        // [VTILES, BH, NC, 64, KD]
  float* dgamma_part;    // [VTILES, BH, NC]
  int NC, V, BH;
  KernelStatus* status;
};

// stage: k-block kb of [k_tail ; w] (2 x 16 KB), q_dec (2 x 8 KB), S_prev [KD][64] (16 KB)
constexpr int BWD_STAGE = 2 * 2 * BOX + 2 * BOX + 2 * BOX;                 // 64 KB
constexpr int BWD_SMEM = 2 * BWD_STAGE + 2 * BOX /*[dv_tot;do]*/ + 2 * BOX /*[v_new;do]*/ + 2 * BOX /*dSb*/ +
                         2 * BOX /*dk_tail out*/ + 4 * BOX /*dw, dq_dec out*/ + 1024 + 128;

__global__ void __launch_bounds__(128, 1)
gdn_seq_bwd_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_qd,
                   const __grid_constant__ CUtensorMap tm_kt, const __grid_constant__ CUtensorMap tm_S,
                   const __grid_constant__ CUtensorMap tm_du, const __grid_constant__ CUtensorMap tm_dkt,
                   const __grid_constant__ CUtensorMap tm_dw, const __grid_constant__ CUtensorMap tm_dqd,
                   const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* AD = smem + 2 * BWD_STAGE;     // [dv_tot (64 rows) ; do (64 rows)] x 64 cols
  uint8_t* AV = AD + 2 * BOX;             // [v_new ; do]
  uint8_t* dSb = AV + 2 * BOX;            // [KD rows][64] bf16 mirror of dS
  // Outputs leave as TMA stores from swizzled tiles (see the forward kernel): du straight from AD,
  // the dk_tail partial from Kst, the -dw and dq_dec partials from Wst.
  uint8_t* Kst = dSb + 2 * BOX;           // [2 k-blocks][64 rows][64]
  uint8_t* Wst = Kst + 2 * BOX;           // [2 k-blocks][128 rows][64]: rows 0..63 -dw, rows 64..127 dq_dec
  uint64_t* bars = reinterpret_cast<uint64_t*>(Wst + 4 * BOX);
  uint64_t* full = bars;
  uint64_t* m1 = bars + 2;
  uint64_t* m2 = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tmem_slot + 2);     // [4]

  const int r = threadIdx.x;
  const int warp = r >> 5;
  const int vt = blockIdx.x, bh = blockIdx.y;
  const int NC = p.NC, V = p.V;

  if (r == 0) {
    *abort_flag = 0;
    tc5::mbar_init(&full[0], 1);
    tc5::mbar_init(&full[1], 1);
    tc5::mbar_init(m1, 1);
    tc5::mbar_init(m2, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  {
    uint32_t z[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) z[j] = 0u;
    write_row_swz(dSb, r, z);
  }
  tc5::fence_proxy_async();
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  // TMEM columns: Da [0,64)  Dc [64,192)  Db [192,320)  dS [320,384)
  const uint32_t cDa = 0, cDc = 64, cDb = 192, cDs = 320;
  {
    float z[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) z[j] = 0.f;
    tmem_st_row64(tmem + lane_off + cDs, z);
  }
  tc5::fence_before_sync();
  __syncthreads();

  auto issue_loads = [&](int c, int it) {
    const int s = it & 1;
    uint8_t* st = smem + s * BWD_STAGE;
    const int row0 = (bh * NC + c) * CH;
    tc5::mbar_expect_tx(&full[s], BWD_STAGE);
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
      tc5::tma_load_2d(st + kb * 2 * BOX, &tm_kt, &full[s], kb * 64, row0);
      tc5::tma_load_2d(st + kb * 2 * BOX + BOX, &tm_w, &full[s], kb * 64, row0);
      tc5::tma_load_2d(st + 4 * BOX + kb * BOX, &tm_qd, &full[s], kb * 64, row0);
    }
    tc5::tma_load_2d(st + 6 * BOX, &tm_S, &full[s], vt * VT, (bh * NC + c) * KD);
  };
  if (r == 0) issue_loads(NC - 1, 0);

  constexpr uint32_t id_a = tc5::make_idesc_bf16(128, VT, 0, 1);        // [kt;w] (K-major) x dS (MN-major)
  constexpr uint32_t id_c = tc5::make_idesc_bf16(128, KD, 0, 0);        // [v_new;do] x dS^T  and  [dv_tot;do] x S^T
  constexpr uint32_t id_d = tc5::make_idesc_bf16(128, VT, 1, 1);        // q_dec^T x do
  constexpr uint32_t id_dn = tc5::make_idesc_bf16(128, VT, 1, 1, 1);    // (-w)^T x dv_tot
  const long part_rows = static_cast<long>(p.BH) * NC * CH;      // rows of one V tile's partials
  bool ok = true;
  // The chunk loop is one dependent chain: the rows that come straight from global memory (v_new and
  // dv_new for rows 0..63, do for rows 64..127) and the decay are fetched one chunk ahead, so their
  // latency is not paid once per chunk.
  uint32_t row_next[32], dv_next[32];
  auto fetch_rows = [&](int cc) {
    const long rr = static_cast<long>(bh * NC + cc) * CH;
    if (r < CH) {
      load_row_global(p.v_new + (rr + r) * V + vt * VT, row_next);
      load_row_global(p.dv_new + (rr + r) * V + vt * VT, dv_next);
    } else {
      load_row_global(p.d_o + (rr + r - CH) * V + vt * VT, row_next);
    }
  };
#pragma unroll
  for (int j = 0; j < 32; ++j) dv_next[j] = 0u;
  fetch_rows(NC - 1);
  float g_next = p.gamma[bh * NC + NC - 1];
  for (int it = 0; it < NC && ok; ++it) {
    const int c = NC - 1 - it;
    const int s = it & 1;
    uint8_t* st = smem + s * BWD_STAGE;
    const long row0 = static_cast<long>(bh * NC + c) * CH;
    // stage this chunk's rows (already in registers) and start the next chunk's loads
    uint32_t dvin[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) dvin[j] = dv_next[j];
    write_row_swz(AV, r, row_next);
    if (r >= CH) write_row_swz(AD, r, row_next);
    const float g = g_next;
    if (c > 0) {
      fetch_rows(c - 1);
      g_next = p.gamma[bh * NC + c - 1];
    }
    tc5::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 0) {
      // converged issuing warp, one elected lane issues (see the forward kernel)
      const bool lead = tc5::elect_one();
      if (__all_sync(0xffffffffu, tc5::mbar_wait(&full[s], (it >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL))) {
        tc5::fence_after_sync();
        const uint64_t a = tc5::desc_kmajor(tc5::smem_u32(st)), dsbm = tc5::desc_mnmajor(tc5::smem_u32(dSb), BOX);
        const uint64_t dsbk = tc5::desc_kmajor(tc5::smem_u32(dSb)), av = tc5::desc_kmajor(tc5::smem_u32(AV));
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < KD / 16; ++kk)      // Da = [k_tail ; w] * dS
            tc5::mma_ss(tmem + cDa, a + static_cast<uint64_t>(((kk >> 2) * 2 * BOX + (kk & 3) * 32) >> 4),
                        dsbm + static_cast<uint64_t>((kk * 2048) >> 4), id_a, kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < VT / 16; ++kk)      // Dc = [v_new ; do] * dS^T
            tc5::mma_ss(tmem + cDc, av + static_cast<uint64_t>((kk * 32) >> 4), dsbk + static_cast<uint64_t>((kk * 32) >> 4), id_c, kk > 0 ? 1u : 0u);
          tc5::mma_commit(m1);
          if (it + 1 < NC) issue_loads(c - 1, it + 1);
        }
      }
      __syncwarp();
    }
    if (r == 0) tc5::tma_store_wait_read<1>();     // the previous chunk's du / dk_tail tiles have been read
    if (!tc5::mbar_wait(m1, it & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; }
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    float part_dg = 0.f;
    {
      // dS (entering from chunk c+1): dgamma partial with S_prev, then scale by gamma in place
      float ds[64], sp[64];
      tmem_ld_row64(tmem + lane_off + cDs, ds);
      read_row_swz(st + 6 * BOX, r, sp);
#pragma unroll
      for (int j = 0; j < 64; ++j) { part_dg += ds[j] * sp[j]; ds[j] *= g; }
      tmem_st_row64(tmem + lane_off + cDs, ds);
    }
    if (r < CH) {
      float da[64], dvf[64];
      tmem_ld_row64(tmem + lane_off + cDa, da);
      unpack_row(dvin, dvf);
#pragma unroll
      for (int j = 0; j < 64; ++j) da[j] += dvf[j];
      uint32_t pk[32];
      pack_row(da, pk);
      write_row_swz(AD, r, pk);
      // dk_tail partial: row r of Dc, KD columns
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float dc[64];
        tmem_ld_row64(tmem + lane_off + cDc + h * 64, dc);
        uint32_t pk2[32];
        pack_row(dc, pk2);
        write_row_swz(Kst + h * BOX, r, pk2);
      }
    }
    // block reduction of the dgamma partial
    for (int o = 16; o > 0; o >>= 1) part_dg += __shfl_xor_sync(0xffffffffu, part_dg, o);
    if ((r & 31) == 0) red[warp] = part_dg;
    tc5::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    if (r == 0) {
      p.dgamma_part[(static_cast<long>(vt) * p.BH + bh) * NC + c] = red[0] + red[1] + red[2] + red[3];
      tc5::tma_store_2d(&tm_du, AD, vt * VT, static_cast<int>(row0));
      tc5::tma_store_2d(&tm_dkt, Kst, 0, static_cast<int>(vt * part_rows + row0));
      tc5::tma_store_2d(&tm_dkt, Kst + BOX, 64, static_cast<int>(vt * part_rows + row0));
      tc5::tma_store_commit();
    }
    if (warp == 0) {
      const bool lead = tc5::elect_one();
      tc5::fence_after_sync();
      const uint64_t adk = tc5::desc_kmajor(tc5::smem_u32(AD)), spk = tc5::desc_kmajor(tc5::smem_u32(st + 6 * BOX));
      const uint64_t qdm = tc5::desc_mnmajor(tc5::smem_u32(st + 4 * BOX), BOX), dom = tc5::desc_mnmajor(tc5::smem_u32(AD + BOX), BOX);
      const uint64_t wm = tc5::desc_mnmajor(tc5::smem_u32(st + BOX), 2 * BOX), adm = tc5::desc_mnmajor(tc5::smem_u32(AD), BOX);
      if (lead) {
#pragma unroll
        for (int kk = 0; kk < VT / 16; ++kk)        // Db = [dv_tot ; do] * S_prev^T
          tc5::mma_ss(tmem + cDb, adk + static_cast<uint64_t>((kk * 32) >> 4), spk + static_cast<uint64_t>((kk * 32) >> 4), id_c, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)        // dS += q_dec^T * do      (do = rows 64..127 of AD)
          tc5::mma_ss(tmem + cDs, qdm + static_cast<uint64_t>((kk * 2048) >> 4), dom + static_cast<uint64_t>((kk * 2048) >> 4), id_d, 1u);
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)        // dS -= w^T * dv_tot      (w = second half of each k-block)
          tc5::mma_ss(tmem + cDs, wm + static_cast<uint64_t>((kk * 2048) >> 4), adm + static_cast<uint64_t>((kk * 2048) >> 4), id_dn, 1u);
        tc5::mma_commit(m2);
      }
      __syncwarp();
    }
    if (r == 0) tc5::tma_store_wait_read<1>();     // the previous chunk's dw / dq_dec tiles have been read
    if (!tc5::mbar_wait(m2, it & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; }
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    {
      // rows 0..63: -dw partial; rows 64..127: dq_dec partial
      const float sign = r < CH ? -1.f : 1.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float db[64];
        tmem_ld_row64(tmem + lane_off + cDb + h * 64, db);
#pragma unroll
        for (int j = 0; j < 64; ++j) db[j] *= sign;
        uint32_t pk[32];
        pack_row(db, pk);
        write_row_swz(Wst + h * 2 * BOX, r, pk);
      }
      float ds[64];
      tmem_ld_row64(tmem + lane_off + cDs, ds);
      uint32_t pk[32];
      pack_row(ds, pk);
      write_row_swz(dSb, r, pk);
    }
    tc5::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    if (r == 0) {
      const int prow = static_cast<int>(vt * part_rows + row0);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tc5::tma_store_2d(&tm_dw, Wst + h * 2 * BOX, h * 64, prow);
        tc5::tma_store_2d(&tm_dqd, Wst + h * 2 * BOX + BOX, h * 64, prow);
      }
      tc5::tma_store_commit();
    }
  }
  if (r == 0) tc5::tma_store_wait_read<0>();
  if (!ok && r == 0) {
    const long long t0 = clock64();
    for (int s = 0; s < 2; ++s)
      for (uint32_t i = 0; i < (1u << 16); ++i) {
        if (tc5::mbar_try_wait(&full[s], 0) || tc5::mbar_try_wait(&full[s], 1)) break;
        if (clock64() - t0 > tc5::kMaxWaitCycles) break;
      }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

int make_rows_map(CUtensorMap* m, const void* base, long rows, int cols, int box_rows) {
  return nsa::make_tmap_2d_bf16(m, base, cols, rows, cols, 64, box_rows);
}
}  // namespace

// w, qd, kt: [BH*NC*64, 128] bf16; u: [BH*NC*64, V] bf16; gamma: [BH*NC] fp32.
// Outputs: v_new [BH*NC*64, V] bf16, o_inter [BH*NC*64, V] bf16, S_all [BH*NC*128, V] bf16.
extern "C" int nsa_gdn_seq_fwd(const void* w, const void* qd, const void* kt, const void* u, const float* gamma,
                               void* v_new, void* o_inter, void* S_all, int BH, int NC, int K, int V,
                               cudaStream_t st) {
  if (K != KD || V % VT) return nsa::fail(NSA_ERR_SHAPE, "gdn: key width must be 128 and value width a multiple of 64");
  CUtensorMap tw, tq, tk;
  const long rows = static_cast<long>(BH) * NC * CH;
  int rc;
  if ((rc = make_rows_map(&tw, w, rows, KD, 64))) return rc;
  if ((rc = make_rows_map(&tq, qd, rows, KD, 64))) return rc;
  if ((rc = make_rows_map(&tk, kt, rows, KD, 64))) return rc;
  CUtensorMap tvn, toi, tsa;
  if ((rc = make_rows_map(&tvn, v_new, rows, V, CH))) return rc;
  if ((rc = make_rows_map(&toi, o_inter, rows, V, CH))) return rc;
  if ((rc = make_rows_map(&tsa, S_all, static_cast<long>(BH) * NC * KD, V, KD))) return rc;
  FwdParams p{(const bf16*)u, gamma, (bf16*)v_new, (bf16*)o_inter, (bf16*)S_all, NC, V, nsa::status_ptr()};
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_seq_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e != cudaSuccess) return nsa::fail_cuda(e, "gdn fwd smem attribute");
    configured = true;
  }
  gdn_seq_fwd_kernel<<<dim3(V / VT, BH), 128, FWD_SMEM, st>>>(tw, tq, tk, tvn, toi, tsa, p);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gdn_seq_fwd launch");
}

// Partials: dw_part/dqd_part/dkt_part [V/64, BH*NC*64, 128] bf16, dgamma_part [V/64, BH*NC] fp32.
extern "C" int nsa_gdn_seq_bwd(const void* w, const void* qd, const void* kt, const void* S_all, const void* v_new,
                               const void* dv_new, const void* d_o, const float* gamma, void* du, void* dw_part,
                               void* dqd_part, void* dkt_part, float* dgamma_part, int BH, int NC, int K, int V,
                               cudaStream_t st) {
  if (K != KD || V % VT) return nsa::fail(NSA_ERR_SHAPE, "gdn: key width must be 128 and value width a multiple of 64");
  CUtensorMap tw, tq, tk, ts;
  const long rows = static_cast<long>(BH) * NC * CH;
  int rc;
  if ((rc = make_rows_map(&tw, w, rows, KD, 64))) return rc;
  if ((rc = make_rows_map(&tq, qd, rows, KD, 64))) return rc;
  if ((rc = make_rows_map(&tk, kt, rows, KD, 64))) return rc;
  if ((rc = make_rows_map(&ts, S_all, static_cast<long>(BH) * NC * KD, V, KD))) return rc;
  CUtensorMap tdu, tdkt, tdw, tdqd;
  const long prows = rows * (V / VT);
  if ((rc = make_rows_map(&tdu, du, rows, V, CH))) return rc;
  if ((rc = make_rows_map(&tdkt, dkt_part, prows, KD, CH))) return rc;
  if ((rc = make_rows_map(&tdw, dw_part, prows, KD, CH))) return rc;
  if ((rc = make_rows_map(&tdqd, dqd_part, prows, KD, CH))) return rc;
  BwdParams p{(const bf16*)v_new, (const bf16*)dv_new, (const bf16*)d_o, gamma, (bf16*)du, (bf16*)dw_part,
              (bf16*)dqd_part, (bf16*)dkt_part, dgamma_part, NC, V, BH, nsa::status_ptr()};
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_seq_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e != cudaSuccess) return nsa::fail_cuda(e, "gdn bwd smem attribute");
    configured = true;
  }
  gdn_seq_bwd_kernel<<<dim3(V / VT, BH), 128, BWD_SMEM, st>>>(tw, tq, tk, ts, tdu, tdkt, tdw, tdqd, p);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_gdn_seq_bwd launch");
}
