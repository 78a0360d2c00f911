// Mamba-2 SSD (state-space duality) on tcgen05 tensor cores.  Chunk length 128, state width
// N = 128, head width P = 64, one group of B/C shared by all heads.
//
// For one (batch, head) with a_t = dt_t * A (<= 0), cum = inclusive cumsum of a inside the
// chunk, tot = cum at the chunk end, and H the N x P state entering the chunk:
//     P_ij    = (C_i . B_j) exp(cum_i - cum_j) dt_j   (j <= i)          "decayed scores"
//     y_i     = sum_j P_ij x_j + exp(cum_i) C_i H + D x_i
//     H_next  = exp(tot) H + sum_j exp(tot - cum_j) dt_j B_j (outer) x_j
// Kernels (one CTA per (chunk, head, batch), no loops over tiles):
//   chunk_state : the sum in H_next (mode 0), or G = sum_i exp(cum_i) C_i (outer) dy_i (mode 1,
//                 the per-chunk term of the state gradient);   fp32 [.., N, P]
//   state pass  : the recurrence over chunks (forward) / its reverse (backward), elementwise
//   chunk_out   : y for the chunk (three MMAs: C B^T, P x, C H)
//   chunk_grad  : dx, per-head dB / dC contributions (added to fp32 buffers), and the two row
//                 scalars dy.(y - D x) and x.dx from which d(dt) and dA follow by a suffix sum.
// Decay factors are formed per element in registers (exp2 of a difference that is <= 0), never
// stored; the [128 x 128] P and dS tiles live only in shared memory as bf16 MMA operands.
#include "host.cuh"
#include "tc5.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int L = 128;      // chunk length
constexpr int NS = 128;     // state width
constexpr int PD = 64;      // head width
constexpr int BOXB = 16384; // bytes of a [128 rows][64 bf16] swizzled box
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void st_row64(uint8_t* kblock, int row, const uint32_t (&pk)[32]) {
  uint8_t* base = kblock + row * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(base + ((j ^ (row & 7)) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
}
__device__ __forceinline__ void ld_row64(const uint8_t* kblock, int row, float (&out)[64]) {
  const uint8_t* base = kblock + row * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v = *reinterpret_cast<const uint4*>(base + ((j ^ (row & 7)) << 4));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      out[8 * j + 2 * k] = f.x;
      out[8 * j + 2 * k + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void tld64(uint32_t taddr, float (&out)[64]) {
  uint32_t a[32], b[32];
  tc5::tmem_ld_x32(taddr, a);
  tc5::tmem_ld_x32(taddr + 32, b);
  tc5::tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) { out[j] = __uint_as_float(a[j]); out[32 + j] = __uint_as_float(b[j]); }
}

// Inclusive scan of `a` over the 128 threads of the CTA; cum[] and dts[] (shared, 128 floats
// each) receive every row's value.  Returns this thread's inclusive sum.
__device__ __forceinline__ float chunk_scan(float a, float dt, float* cum, float* dts, float* warp_tot) {
  const int r = threadIdx.x, lane = r & 31, w = r >> 5;
  float v = a;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_tot[w] = v;
  __syncthreads();
  float off = 0.f;
  for (int k = 0; k < w; ++k) off += warp_tot[k];
  v += off;
  cum[r] = v;
  dts[r] = dt;
  __syncthreads();
  return v;
}

struct SsdParams {
  const float* dt;     // [B, T, H] (after softplus)
  const float* A;      // [H] (negative)
  const float* Dskip;  // [H] or null
  int B, T, H, nc;
  // chunk_state
  float* S_out;        // [B, nc, H, NS, PD] fp32
  float* gamma_out;    // [B, nc, H] or null
  // chunk_out
  bf16* y;             // [B, T, H, PD]
  const bf16* x_raw;   // x for the D skip and row scalars (token stride ldx elements, head offset h*PD)
  long ldx;
  // chunk_grad
  const bf16* y_in;    // [B, T, H, PD]
  const bf16* dy_raw;  // [B, T, H, PD]
  bf16* dx;            // [B, T, H, PD]
  float* dB_acc;       // [B, T, NS] fp32 (pre-zeroed, summed over heads)
  float* dC_acc;       // [B, T, NS]
  bf16* dB_heads;      // [B, T, H, NS] per-head results written with plain stores (null: use the fp32 reductions above);
  bf16* dC_heads;      //   the caller sums over heads: 64 heads adding into one row contend for the same L2 lines otherwise
  float* q_out;        // [B, T, H]  dy . (y - D x)
  float* k_out;        // [B, T, H]  x . dx (without the D term)
  float* r_out;        // [B, T, H]  dy . x (gradient of the skip weight D before the sum over tokens), or null
  KernelStatus* status;
};

// ---------------------------------------------------------------------------------------
// chunk_state.  MODE 0: rows of Bm scaled by exp(tot - cum_j) dt_j, values = x.
//               MODE 1: rows of Cm scaled by exp(cum_i),            values = dy.
// out[N, P] = scaled^T [N x 128] * values [128 x P]
// ---------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(128, 2)
ssd_chunk_state_kernel(const __grid_constant__ CUtensorMap tm_bc, const __grid_constant__ CUtensorMap tm_v,
                       const SsdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sBC = smem;                 // [2 chunks][128 t][64]  raw rows, then scaled in place
  uint8_t* sV = sBC + 2 * BOXB;        // [128 t][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + BOXB);
  uint64_t* full = bars;
  uint64_t* done = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* cum = reinterpret_cast<float*>(bars + 4);
  float* dts = cum + L;
  float* warp_tot = dts + L;

  const int r = threadIdx.x, warp = r >> 5;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = c * L;
  if (r == 0) {
    *abort_flag = 0;
    tc5::mbar_init(full, 1);
    tc5::mbar_init(done, 1);
    tc5::fence_barrier_init();
    tc5::mbar_expect_tx(full, 3 * BOXB);
    tc5::tma_load_3d(sBC, &tm_bc, full, 0, t0, b);
    tc5::tma_load_3d(sBC + BOXB, &tm_bc, full, 64, t0, b);
    tc5::tma_load_4d(sV, &tm_v, full, 0, h, t0, b);
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 64); tc5::tmem_relinquish(); }
  const int t = t0 + r;
  const float dt = t < p.T ? p.dt[(static_cast<long>(b) * p.T + t) * p.H + h] : 0.f;
  const float a = dt * p.A[h];
  const float cm = chunk_scan(a, dt, cum, dts, warp_tot);
  const float tot = cum[L - 1];
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool ok = tc5::mbar_wait(full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
  if (ok) {
    const float sc = MODE == 0 ? exp2f((tot - cm) * LOG2E) * dt : exp2f(cm * LOG2E);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float v[64];
      ld_row64(sBC + half * BOXB, r, v);
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) pk[j] = tc5::pack_bf16(v[2 * j] * sc, v[2 * j + 1] * sc);
      st_row64(sBC + half * BOXB, r, pk);
    }
  }
  tc5::fence_proxy_async();
  tc5::fence_before_sync();
  if (__syncthreads_or(!ok)) ok = false;
  if (ok && warp == 0) {
    // the whole warp stays converged and one elected lane issues: descriptors then live in uniform
    // registers and an MMA costs the issuing thread a few cycles instead of 70 to 100
    const bool lead = tc5::elect_one();
    tc5::fence_after_sync();
    constexpr uint32_t idesc = tc5::make_idesc_bf16(128, PD, 1, 1);
    const uint64_t a0 = tc5::desc_mnmajor(tc5::smem_u32(sBC), BOXB), v0 = tc5::desc_mnmajor(tc5::smem_u32(sV), BOXB);
    if (lead) {
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk)
        tc5::mma_ss(tmem, a0 + static_cast<uint64_t>((kk * 2048) >> 4), v0 + static_cast<uint64_t>((kk * 2048) >> 4), idesc, kk > 0 ? 1u : 0u);
      tc5::mma_commit(done);
    }
    __syncwarp();
  }
  if (ok && !tc5::mbar_wait(done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
  if (!__syncthreads_or(!ok)) {
    tc5::fence_after_sync();
    float o[64];
    tld64(tmem + (static_cast<uint32_t>(warp * 32) << 16), o);
    float4* dst = reinterpret_cast<float4*>(p.S_out + (((static_cast<long>(b) * p.nc + c) * p.H + h) * NS + r) * PD);
#pragma unroll
    for (int j = 0; j < 16; ++j) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
    if (MODE == 0 && r == 0 && p.gamma_out) p.gamma_out[(static_cast<long>(b) * p.nc + c) * p.H + h] = exp2f(tot * LOG2E);
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 64); }
}

// ---------------------------------------------------------------------------------------
// chunk_out: y = P x + exp(cum) (C H) + D x  for one (chunk, head, batch).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
ssd_chunk_out_kernel(const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_h,
                     const __grid_constant__ CUtensorMap tm_y, const SsdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;                  // [2 k-blocks][128][64]
  uint8_t* sB = sC + 2 * BOXB;
  uint8_t* sX = sB + 2 * BOXB;         // [128 t][64]
  uint8_t* sH = sX + BOXB;             // [128 n][64]
  uint8_t* sP = sH + BOXB;             // [2 k-blocks][128][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * BOXB);
  uint64_t* full = bars;
  uint64_t* m1 = bars + 1;
  uint64_t* m2 = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* cum = reinterpret_cast<float*>(bars + 4);
  float* dts = cum + L;
  float* warp_tot = dts + L;

  const int r = threadIdx.x, warp = r >> 5;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = c * L;
  if (r == 0) {
    *abort_flag = 0;
    tc5::mbar_init(full, 1);
    tc5::mbar_init(m1, 1);
    tc5::mbar_init(m2, 1);
    tc5::fence_barrier_init();
    tc5::mbar_expect_tx(full, 6 * BOXB);
    tc5::tma_load_3d(sC, &tm_c, full, 0, t0, b);
    tc5::tma_load_3d(sC + BOXB, &tm_c, full, 64, t0, b);
    tc5::tma_load_3d(sB, &tm_b, full, 0, t0, b);
    tc5::tma_load_3d(sB + BOXB, &tm_b, full, 64, t0, b);
    tc5::tma_load_4d(sX, &tm_x, full, 0, h, t0, b);
    tc5::tma_load_2d(sH, &tm_h, full, 0, ((b * p.nc + c) * p.H + h) * NS);
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 256); tc5::tmem_relinquish(); }
  const int t = t0 + r;
  const bool row_ok = t < p.T;
  const float dt = row_ok ? p.dt[(static_cast<long>(b) * p.T + t) * p.H + h] : 0.f;
  const float cm = chunk_scan(dt * p.A[h], dt, cum, dts, warp_tot);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t cS = 0, cYi = 128, cYo = 192;
  constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t id_y = tc5::make_idesc_bf16(128, PD, 0, 1);
  bool ok = true;
  if (warp == 0) {
    // converged warp, elected lane issues (see ssd_chunk_state_kernel)
    const bool lead = tc5::elect_one();
    if (__all_sync(0xffffffffu, tc5::mbar_wait(full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL))) {
      tc5::fence_after_sync();
      const uint64_t cc = tc5::desc_kmajor(tc5::smem_u32(sC)), bb = tc5::desc_kmajor(tc5::smem_u32(sB));
      const uint64_t hh = tc5::desc_mnmajor(tc5::smem_u32(sH), BOXB);
      if (lead) {
#pragma unroll
        for (int kk = 0; kk < NS / 16; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4);
          tc5::mma_ss(tmem + cS, cc + off, bb + off, id_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < NS / 16; ++kk)
          tc5::mma_ss(tmem + cYi, cc + static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4),
                      hh + static_cast<uint64_t>((kk * 2048) >> 4), id_y, kk > 0 ? 1u : 0u);
        tc5::mma_commit(m1);
      }
    }
    __syncwarp();
  }
  if (!tc5::mbar_wait(m1, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
  if (__syncthreads_or(!ok)) ok = false;
  if (ok) {
    tc5::fence_after_sync();
    const float ci = cm * LOG2E;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[64];
      tld64(tmem + lane_off + cS + half * 64, s);
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        // operands fetched and the weight computed for every j, then selected: a conditional around
        // the loads costs a branch per element
        const int j0 = half * 64 + j;
        const float2 cj = *reinterpret_cast<const float2*>(cum + j0), dj = *reinterpret_cast<const float2*>(dts + j0);
        const float w0 = exp2f(fminf(ci - cj.x * LOG2E, 0.f)) * dj.x, w1 = exp2f(fminf(ci - cj.y * LOG2E, 0.f)) * dj.y;
        const float p0 = j0 <= r ? s[j] * w0 : 0.f;
        const float p1 = j0 + 1 <= r ? s[j + 1] * w1 : 0.f;
        pk[j / 2] = tc5::pack_bf16(p0, p1);
      }
      st_row64(sP + half * BOXB, r, pk);
    }
  }
  tc5::fence_proxy_async();
  tc5::fence_before_sync();
  __syncthreads();
  if (ok && warp == 0) {
    const bool lead = tc5::elect_one();
    tc5::fence_after_sync();
    const uint64_t pp = tc5::desc_kmajor(tc5::smem_u32(sP)), xx = tc5::desc_mnmajor(tc5::smem_u32(sX), BOXB);
    if (lead) {
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk)
        tc5::mma_ss(tmem + cYo, pp + static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4),
                    xx + static_cast<uint64_t>((kk * 2048) >> 4), id_y, kk > 0 ? 1u : 0u);
      tc5::mma_commit(m2);
    }
    __syncwarp();
  }
  if (ok && !tc5::mbar_wait(m2, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
  if (!__syncthreads_or(!ok)) {
    tc5::fence_after_sync();
    // y leaves through shared memory and one TMA store (a thread owns a token row, so direct stores
    // would write 16 bytes per thread into 32 different rows per instruction); x comes from its tile
    float yo[64], yi[64];
    tld64(tmem + lane_off + cYo, yo);
    tld64(tmem + lane_off + cYi, yi);
    const float e = exp2f(cm * LOG2E);
    const float dsk = p.Dskip ? p.Dskip[h] : 0.f;
    uint32_t o[32];
    {
      float xf[64];
      ld_row64(sX, r, xf);
#pragma unroll
      for (int i = 0; i < 64; i += 2)
        o[i / 2] = tc5::pack_bf16(yo[i] + e * yi[i] + dsk * xf[i], yo[i + 1] + e * yi[i + 1] + dsk * xf[i + 1]);
    }
    st_row64(sP, r, o);                 // the P tile is free once the second MMA is complete
    tc5::fence_proxy_async();
    __syncthreads();
    if (r == 0) {                       // rows past T are clipped by the copy engine
      tc5::tma_store_4d(&tm_y, sP, 0, h, t0, b);
      tc5::tma_store_commit();
      tc5::tma_store_wait_read<0>();
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 256); }
}

// ---------------------------------------------------------------------------------------
// chunk_grad for one (chunk, head, batch), given dy, the state entering the chunk (H) and
// the gradient of the state leaving it (dHn):
//   S = C B^T, R = dy x^T;  P = S w, dS = R w  with w_ij = exp(cum_i - cum_j) dt_j (j <= i)
//   dx_j  = sum_i P_ij dy_i + s_j B_j dHn + D dy_j          (s_j = exp(tot - cum_j) dt_j)
//   dC_i  = sum_j dS_ij B_j + exp(cum_i) dy_i H^T
//   dB_j  = sum_i dS_ij C_i + s_j x_j dHn^T
// dB / dC are summed over heads with fp32 vector reductions.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
ssd_chunk_grad_kernel(const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                      const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_dh,
                      const __grid_constant__ CUtensorMap tm_dx, const __grid_constant__ CUtensorMap tm_dbh,
                      const __grid_constant__ CUtensorMap tm_dch, const SsdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;                  // 2 boxes
  uint8_t* sB = sC + 2 * BOXB;         // 2 boxes
  uint8_t* sX = sB + 2 * BOXB;         // 1
  uint8_t* sDY = sX + BOXB;            // 1
  uint8_t* sH = sDY + BOXB;            // 1   [n][p]
  uint8_t* sDH = sH + BOXB;            // 1   [n][p]
  uint8_t* sP = sDH + BOXB;            // 2
  uint8_t* sDS = sP + 2 * BOXB;        // 2
  uint8_t* sXS = sDS + 2 * BOXB;       // 1   x rows scaled by s_j
  uint64_t* bars = reinterpret_cast<uint64_t*>(sXS + BOXB);
  uint64_t* full = bars;
  uint64_t* m1 = bars + 1;
  uint64_t* m2 = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* cum = reinterpret_cast<float*>(bars + 4);
  float* dts = cum + L;
  float* warp_tot = dts + L;

  const int r = threadIdx.x, warp = r >> 5;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int t0 = c * L;
  if (r == 0) {
    *abort_flag = 0;
    tc5::mbar_init(full, 1);
    tc5::mbar_init(m1, 1);
    tc5::mbar_init(m2, 1);
    tc5::fence_barrier_init();
    tc5::mbar_expect_tx(full, 8 * BOXB);
    tc5::tma_load_3d(sC, &tm_c, full, 0, t0, b);
    tc5::tma_load_3d(sC + BOXB, &tm_c, full, 64, t0, b);
    tc5::tma_load_3d(sB, &tm_b, full, 0, t0, b);
    tc5::tma_load_3d(sB + BOXB, &tm_b, full, 64, t0, b);
    tc5::tma_load_4d(sX, &tm_x, full, 0, h, t0, b);
    tc5::tma_load_4d(sDY, &tm_dy, full, 0, h, t0, b);
    const int srow = ((b * p.nc + c) * p.H + h) * NS;
    tc5::tma_load_2d(sH, &tm_h, full, 0, srow);
    tc5::tma_load_2d(sDH, &tm_dh, full, 0, srow);
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  const int t = t0 + r;
  const bool row_ok = t < p.T;
  const float dt = row_ok ? p.dt[(static_cast<long>(b) * p.T + t) * p.H + h] : 0.f;
  const float cm = chunk_scan(dt * p.A[h], dt, cum, dts, warp_tot);
  const float tot = cum[L - 1];
  const float s_row = exp2f((tot - cm) * LOG2E) * dt;
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  // TMEM columns: S / dC [0,128)  R / dB [128,256)  dX [256,320)  dXi [320,384)  dCi [384,512)
  const uint32_t cS = 0, cR = 128, cDX = 256, cDXI = 320, cDCI = 384;
  constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 128, 0, 0);     // K-major x K-major -> [128 x 128]
  constexpr uint32_t id_kn64 = tc5::make_idesc_bf16(128, PD, 0, 1);   // K-major A, MN-major B -> [128 x 64]
  constexpr uint32_t id_tn64 = tc5::make_idesc_bf16(128, PD, 1, 1);   // MN-major A, MN-major B -> [128 x 64]
  constexpr uint32_t id_kn128 = tc5::make_idesc_bf16(128, NS, 0, 1);  // K-major A, MN-major B -> [128 x 128]
  constexpr uint32_t id_tn128 = tc5::make_idesc_bf16(128, NS, 1, 1);  // MN-major A, MN-major B -> [128 x 128]
  bool ok = true;
  if (warp == 0) {
    // converged warp, elected lane issues (see ssd_chunk_state_kernel)
    const bool lead = tc5::elect_one();
    if (__all_sync(0xffffffffu, tc5::mbar_wait(full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL))) {
      tc5::fence_after_sync();
      const uint64_t cc = tc5::desc_kmajor(tc5::smem_u32(sC)), bb = tc5::desc_kmajor(tc5::smem_u32(sB));
      const uint64_t xx = tc5::desc_kmajor(tc5::smem_u32(sX)), dy = tc5::desc_kmajor(tc5::smem_u32(sDY));
      const uint64_t hh = tc5::desc_kmajor(tc5::smem_u32(sH)), dhm = tc5::desc_mnmajor(tc5::smem_u32(sDH), BOXB);
      if (lead) {
#pragma unroll
        for (int kk = 0; kk < NS / 16; ++kk) {             // S = C B^T
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4);
          tc5::mma_ss(tmem + cS, cc + off, bb + off, id_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < PD / 16; ++kk)               // R = dy x^T
          tc5::mma_ss(tmem + cR, dy + static_cast<uint64_t>((kk * 32) >> 4), xx + static_cast<uint64_t>((kk * 32) >> 4), id_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < NS / 16; ++kk)               // dXi = B dHn   (row scale s_j applied later)
          tc5::mma_ss(tmem + cDXI, bb + static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4),
                      dhm + static_cast<uint64_t>((kk * 2048) >> 4), id_kn64, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < PD / 16; ++kk)               // dCi = dy H^T  (row scale exp(cum_i) applied later)
          tc5::mma_ss(tmem + cDCI, dy + static_cast<uint64_t>((kk * 32) >> 4), hh + static_cast<uint64_t>((kk * 32) >> 4), id_s, kk > 0 ? 1u : 0u);
        tc5::mma_commit(m1);
      }
    }
    __syncwarp();
  }
  // x rows scaled by s_j (operand of the state-path part of dB) while the MMAs run
  bool landed = tc5::mbar_wait(full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
  if (landed) {
    float xv[64];
    ld_row64(sX, r, xv);
    uint32_t pk[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) pk[j] = tc5::pack_bf16(xv[2 * j] * s_row, xv[2 * j + 1] * s_row);
    st_row64(sXS, r, pk);
  } else ok = false;
  if (!tc5::mbar_wait(m1, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
  if (__syncthreads_or(!ok)) ok = false;
  float q_intra = 0.f;      // sum_j P_ij R_ij with P as rounded for the MMA: pairs exactly with x.dx
  if (ok) {
    tc5::fence_after_sync();
    const float ci = cm * LOG2E;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[64], rr[64];
      tld64(tmem + lane_off + cS + half * 64, s);
      tld64(tmem + lane_off + cR + half * 64, rr);
      uint32_t pp[32], ds[32];
#pragma unroll
      for (int j = 0; j < 64; j += 2) {
        // operands fetched and the weight computed for every j, then selected (no branch per element)
        const int j0 = half * 64 + j;
        const float2 cj = *reinterpret_cast<const float2*>(cum + j0), dj = *reinterpret_cast<const float2*>(dts + j0);
        const float e0 = exp2f(fminf(ci - cj.x * LOG2E, 0.f)) * dj.x, e1 = exp2f(fminf(ci - cj.y * LOG2E, 0.f)) * dj.y;
        const float w0 = j0 <= r ? e0 : 0.f;
        const float w1 = j0 + 1 <= r ? e1 : 0.f;
        pp[j / 2] = tc5::pack_bf16(s[j] * w0, s[j + 1] * w1);
        ds[j / 2] = tc5::pack_bf16(rr[j] * w0, rr[j + 1] * w1);
        const float2 pr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pp[j / 2]));
        q_intra += pr.x * rr[j] + pr.y * rr[j + 1];
      }
      st_row64(sP + half * BOXB, r, pp);
      st_row64(sDS + half * BOXB, r, ds);
    }
  }
  tc5::fence_proxy_async();
  tc5::fence_before_sync();
  __syncthreads();
  if (ok && warp == 0) {
    const bool lead = tc5::elect_one();
    tc5::fence_after_sync();
    const uint64_t ccm = tc5::desc_mnmajor(tc5::smem_u32(sC), BOXB), bbm = tc5::desc_mnmajor(tc5::smem_u32(sB), BOXB);
    const uint64_t dym = tc5::desc_mnmajor(tc5::smem_u32(sDY), BOXB), dh = tc5::desc_kmajor(tc5::smem_u32(sDH));
    const uint64_t ppm = tc5::desc_mnmajor(tc5::smem_u32(sP), BOXB), ds = tc5::desc_kmajor(tc5::smem_u32(sDS));
    const uint64_t dsm = tc5::desc_mnmajor(tc5::smem_u32(sDS), BOXB), xs = tc5::desc_kmajor(tc5::smem_u32(sXS));
    if (lead) {
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk)                  // dX = P^T dy
        tc5::mma_ss(tmem + cDX, ppm + static_cast<uint64_t>((kk * 2048) >> 4), dym + static_cast<uint64_t>((kk * 2048) >> 4), id_tn64, kk > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk)                  // dC = dS B
        tc5::mma_ss(tmem + cS, ds + static_cast<uint64_t>(((kk >> 2) * BOXB + (kk & 3) * 32) >> 4),
                    bbm + static_cast<uint64_t>((kk * 2048) >> 4), id_kn128, kk > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk)                  // dB = dS^T C
        tc5::mma_ss(tmem + cR, dsm + static_cast<uint64_t>((kk * 2048) >> 4), ccm + static_cast<uint64_t>((kk * 2048) >> 4), id_tn128, kk > 0 ? 1u : 0u);
#pragma unroll
      for (int kk = 0; kk < PD / 16; ++kk)                 // dB += (s x) dHn^T
        tc5::mma_ss(tmem + cR, xs + static_cast<uint64_t>((kk * 32) >> 4), dh + static_cast<uint64_t>((kk * 32) >> 4), id_s, 1u);
      tc5::mma_commit(m2);
    }
    __syncwarp();
  }
  if (ok && !tc5::mbar_wait(m2, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
  if (!__syncthreads_or(!ok)) {
    tc5::fence_after_sync();
    // Outputs leave through shared memory and TMA stores: a thread owns a token row, so direct
    // stores would write 16 bytes per thread into 32 different rows per instruction.  The operand
    // tiles are free once the second group of MMAs is complete: dx goes to the x-scaled tile, dC
    // to the P tile, dB to the dS tile.  x and dy are read back from their own tiles.
    const long tok = static_cast<long>(b) * p.T + t;
    const float e = exp2f(cm * LOG2E);
    const bool heads = p.dB_heads != nullptr;
    {
      float dxa[64], dxi[64];
      tld64(tmem + lane_off + cDX, dxa);
      tld64(tmem + lane_off + cDXI, dxi);
      const float dsk = p.Dskip ? p.Dskip[h] : 0.f;
      float kacc = 0.f, racc = 0.f;
      uint32_t o[32];
      {
        float xf[64], df[64];
        ld_row64(sX, r, xf);
        ld_row64(sDY, r, df);
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float g0 = dxa[i] + s_row * dxi[i], g1 = dxa[i + 1] + s_row * dxi[i + 1];
          kacc += xf[i] * g0 + xf[i + 1] * g1;
          racc += xf[i] * df[i] + xf[i + 1] * df[i + 1];
          o[i / 2] = tc5::pack_bf16(g0 + dsk * df[i], g1 + dsk * df[i + 1]);
        }
      }
      st_row64(sXS, r, o);
      if (row_ok) {
        p.k_out[tok * p.H + h] = kacc;
        if (p.r_out) p.r_out[tok * p.H + h] = racc;
      }
    }
    float q_inter = 0.f;    // C_i . (dy_i H^T): the state-path part of dy.(y - D x), before exp(cum_i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float dc[64], dci[64], db[64];
      tld64(tmem + lane_off + cS + half * 64, dc);
      tld64(tmem + lane_off + cDCI + half * 64, dci);
      tld64(tmem + lane_off + cR + half * 64, db);
      {
        float cv[64];
        ld_row64(sC + half * BOXB, r, cv);
#pragma unroll
        for (int j = 0; j < 64; ++j) q_inter += cv[j] * dci[j];
      }
      if (heads) {
        uint32_t vc[32], vb[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          vc[j] = tc5::pack_bf16(dc[2 * j] + e * dci[2 * j], dc[2 * j + 1] + e * dci[2 * j + 1]);
          vb[j] = tc5::pack_bf16(db[2 * j], db[2 * j + 1]);
        }
        st_row64(sP + half * BOXB, r, vc);
        st_row64(sDS + half * BOXB, r, vb);
      } else if (row_ok) {
        float4* pc = reinterpret_cast<float4*>(p.dC_acc + tok * NS + half * 64);
        float4* pb = reinterpret_cast<float4*>(p.dB_acc + tok * NS + half * 64);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          atomicAdd(pc + j, make_float4(dc[4 * j] + e * dci[4 * j], dc[4 * j + 1] + e * dci[4 * j + 1],
                                        dc[4 * j + 2] + e * dci[4 * j + 2], dc[4 * j + 3] + e * dci[4 * j + 3]));
          atomicAdd(pb + j, make_float4(db[4 * j], db[4 * j + 1], db[4 * j + 2], db[4 * j + 3]));
        }
      }
    }
    tc5::fence_proxy_async();
    __syncthreads();
    if (r == 0) {                       // rows past T are clipped by the copy engine
      tc5::tma_store_4d(&tm_dx, sXS, 0, h, t0, b);
      if (heads) {
        tc5::tma_store_4d(&tm_dch, sP, 0, h, t0, b);
        tc5::tma_store_4d(&tm_dch, sP + BOXB, 64, h, t0, b);
        tc5::tma_store_4d(&tm_dbh, sDS, 0, h, t0, b);
        tc5::tma_store_4d(&tm_dbh, sDS + BOXB, 64, h, t0, b);
      }
      tc5::tma_store_commit();
      tc5::tma_store_wait_read<0>();    // shared memory must outlive the copies' reads
    }
    if (row_ok) p.q_out[tok * p.H + h] = q_intra + e * q_inter;
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// ---------------------------------------------------------------------------------------
// State passing over chunks (elementwise).  Layout [B, nc, H, E], E = NS * PD.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ssd_state_fwd_kernel(const float* __restrict__ S, const float* __restrict__ gamma,
                                                            float* __restrict__ Hprev, bf16* __restrict__ Hprev_bf,
                                                            float* __restrict__ Hlast, int nc, int H, long E) {
  const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int h = blockIdx.y, b = blockIdx.z;
  float st = 0.f;
  for (int c = 0; c < nc; ++c) {
    const long bch = (static_cast<long>(b) * nc + c) * H + h;
    if (Hprev) Hprev[bch * E + e] = st;
    if (Hprev_bf) Hprev_bf[bch * E + e] = __float2bfloat16(st);
    st = gamma[bch] * st + S[bch * E + e];
  }
  if (Hlast) Hlast[(static_cast<long>(b) * H + h) * E + e] = st;
}
__global__ void __launch_bounds__(256) ssd_state_bwd_kernel(const float* __restrict__ dHprev, const float* __restrict__ gamma,
                                                            float* __restrict__ dS, bf16* __restrict__ dS_bf, int nc, int H, long E) {
  const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int h = blockIdx.y, b = blockIdx.z;
  float g = 0.f;
  for (int c = nc - 1; c >= 0; --c) {
    const long bch = (static_cast<long>(b) * nc + c) * H + h;
    if (dS) dS[bch * E + e] = g;
    if (dS_bf) dS_bf[bch * E + e] = __float2bfloat16(g);
    g = dHprev[bch * E + e] + gamma[bch] * g;
  }
}

int map_bc(CUtensorMap* m, const void* base, int B, int T, long ld) {
  uint64_t dims[3] = {(uint64_t)NS, (uint64_t)T, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)T * ld * 2};
  uint32_t box[3] = {64, (uint32_t)L, 1};
  return nsa::make_tmap_bf16(m, base, 3, dims, strides, box, 1);
}
int map_v(CUtensorMap* m, const void* base, int B, int T, int H, long ld) {
  uint64_t dims[4] = {(uint64_t)PD, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)PD * 2, (uint64_t)ld * 2, (uint64_t)T * ld * 2};
  uint32_t box[4] = {64, 1, (uint32_t)L, 1};
  return nsa::make_tmap_bf16(m, base, 4, dims, strides, box, 1);
}
int map_heads(CUtensorMap* m, const void* base, int B, int T, int H, bool real) {
  if (!real) return map_v(m, base, B, T, H, static_cast<long>(H) * PD);
  uint64_t dims[4] = {(uint64_t)NS, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)NS * 2, (uint64_t)H * NS * 2, (uint64_t)T * H * NS * 2};
  uint32_t box[4] = {64, 1, (uint32_t)L, 1};
  return nsa::make_tmap_bf16(m, base, 4, dims, strides, box, 1);
}
int map_state(CUtensorMap* m, const void* base, long rows) {
  return nsa::make_tmap_2d_bf16(m, base, PD, rows, PD, 64, NS);
}
template <typename K>
int smem_attr(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "ssd: shared memory attribute");
}
int check_dims(int N, int P, long ld_bc, long ld_v) {
  if (N != NS || P != PD) return nsa::fail(NSA_ERR_SHAPE, "ssd: native kernels need d_state 128 and headdim 64");
  if ((ld_bc & 7) || (ld_v & 7)) return nsa::fail(NSA_ERR_ALIGNMENT, "ssd: token strides must be multiples of 8 elements");
  return 0;
}
}  // namespace

extern "C" int nsa_ssd_state_fwd(const float* S, const float* gamma, float* Hprev, void* Hprev_bf16, float* Hlast, int B,
                                 int nc, int H, long E, cudaStream_t st) {
  dim3 grid((unsigned)((E + 255) / 256), H, B);
  ssd_state_fwd_kernel<<<grid, 256, 0, st>>>(S, gamma, Hprev, (bf16*)Hprev_bf16, Hlast, nc, H, E);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_ssd_state_bwd(const float* dHprev, const float* gamma, float* dS, void* dS_bf16, int B, int nc, int H,
                                 long E, cudaStream_t st) {
  dim3 grid((unsigned)((E + 255) / 256), H, B);
  ssd_state_bwd_kernel<<<grid, 256, 0, st>>>(dHprev, gamma, dS, (bf16*)dS_bf16, nc, H, E);
  nsa::count_launch();
  return 0;
}

// mode 0: bc = B rows, v = x -> chunk end states and gamma.  mode 1: bc = C rows, v = dy -> G.
// bc: [B, T, N] with token stride ld_bc; v: [B, T, H, P] with token stride ld_v (elements).
extern "C" int nsa_ssd_chunk_state(int mode, const void* bc, long ld_bc, const void* v, long ld_v, const float* dt,
                                   const float* A, float* S_out, float* gamma_out, int B, int T, int H, int N, int P,
                                   cudaStream_t st) {
  int rc = check_dims(N, P, ld_bc, ld_v);
  if (rc) return rc;
  CUtensorMap tb, tv;
  if ((rc = map_bc(&tb, bc, B, T, ld_bc))) return rc;
  if ((rc = map_v(&tv, v, B, T, H, ld_v))) return rc;
  SsdParams p{};
  p.dt = dt; p.A = A; p.B = B; p.T = T; p.H = H; p.nc = (T + L - 1) / L;
  p.S_out = S_out; p.gamma_out = gamma_out; p.status = nsa::status_ptr();
  const int smem = 3 * BOXB + 1024 + 2048;
  const dim3 grid(p.nc, H, B);
  if (mode == 0) {
    static bool cfg = false;
    if (!cfg) { if ((rc = smem_attr(ssd_chunk_state_kernel<0>, smem))) return rc; cfg = true; }
    ssd_chunk_state_kernel<0><<<grid, 128, smem, st>>>(tb, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = smem_attr(ssd_chunk_state_kernel<1>, smem))) return rc; cfg = true; }
    ssd_chunk_state_kernel<1><<<grid, 128, smem, st>>>(tb, tv, p);
  }
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ssd_chunk_state launch");
}

// y [B, T, H, P] contiguous.  Hprev_bf16: [B, nc, H, N, P] bf16.
extern "C" int nsa_ssd_chunk_out(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x,
                                 const void* Hprev_bf16, const float* dt, const float* A, const float* Dskip, void* y,
                                 int B, int T, int H, int N, int P, cudaStream_t st) {
  int rc = check_dims(N, P, ld_c | ld_b, ld_x);
  if (rc) return rc;
  const int nc = (T + L - 1) / L;
  CUtensorMap tc, tb, tx, th, ty;
  if ((rc = map_bc(&tc, Cm, B, T, ld_c))) return rc;
  if ((rc = map_bc(&tb, Bm, B, T, ld_b))) return rc;
  if ((rc = map_v(&tx, x, B, T, H, ld_x))) return rc;
  if ((rc = map_state(&th, Hprev_bf16, static_cast<long>(B) * nc * H * NS))) return rc;
  SsdParams p{};
  p.dt = dt; p.A = A; p.Dskip = Dskip; p.B = B; p.T = T; p.H = H; p.nc = nc;
  p.y = (bf16*)y; p.x_raw = (const bf16*)x; p.ldx = ld_x; p.status = nsa::status_ptr();
  const int smem = 8 * BOXB + 1024 + 2048;
  static bool cfg = false;
  if (!cfg) { if ((rc = smem_attr(ssd_chunk_out_kernel, smem))) return rc; cfg = true; }
  if ((rc = map_v(&ty, y, B, T, H, static_cast<long>(H) * PD))) return rc;
  ssd_chunk_out_kernel<<<dim3(nc, H, B), 128, smem, st>>>(tc, tb, tx, th, ty, p);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ssd_chunk_out launch");
}

// dB_acc / dC_acc: fp32 [B, T, N], zeroed by the caller.  q_out / k_out: fp32 [B, T, H].
static int ssd_chunk_grad_impl(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x,
                               const void* dy, const void* y, const void* Hprev_bf16, const void* dHn_bf16,
                               const float* dt, const float* A, const float* Dskip, void* dx, float* dB_acc,
                               float* dC_acc, void* dB_heads, void* dC_heads, float* q_out, float* k_out, float* r_out,
                               int B, int T, int H, int N, int P, cudaStream_t st) {
  int rc = check_dims(N, P, ld_c | ld_b, ld_x);
  if (rc) return rc;
  const int nc = (T + L - 1) / L;
  const long rows = static_cast<long>(B) * nc * H * NS;
  CUtensorMap tc, tb, tx, tdy, th, tdh, tdx, tdbh, tdch;
  if ((rc = map_bc(&tc, Cm, B, T, ld_c))) return rc;
  if ((rc = map_bc(&tb, Bm, B, T, ld_b))) return rc;
  if ((rc = map_v(&tx, x, B, T, H, ld_x))) return rc;
  if ((rc = map_v(&tdy, dy, B, T, H, static_cast<long>(H) * PD))) return rc;
  if ((rc = map_state(&th, Hprev_bf16, rows))) return rc;
  if ((rc = map_state(&tdh, dHn_bf16, rows))) return rc;
  if ((rc = map_v(&tdx, dx, B, T, H, static_cast<long>(H) * PD))) return rc;
  // per-head dB / dC [B, T, H, N]; without them the maps point at dx and are never used
  if ((rc = map_heads(&tdbh, dB_heads ? dB_heads : dx, B, T, H, dB_heads != nullptr))) return rc;
  if ((rc = map_heads(&tdch, dC_heads ? dC_heads : dx, B, T, H, dC_heads != nullptr))) return rc;
  SsdParams p{};
  p.dt = dt; p.A = A; p.Dskip = Dskip; p.B = B; p.T = T; p.H = H; p.nc = nc;
  p.x_raw = (const bf16*)x; p.ldx = ld_x; p.y_in = (const bf16*)y; p.dy_raw = (const bf16*)dy; p.dx = (bf16*)dx;
  p.dB_acc = dB_acc; p.dC_acc = dC_acc; p.q_out = q_out; p.k_out = k_out; p.status = nsa::status_ptr();
  p.dB_heads = (bf16*)dB_heads; p.dC_heads = (bf16*)dC_heads; p.r_out = r_out;
  const int smem = 13 * BOXB + 1024 + 2048;
  static bool cfg = false;
  if (!cfg) { if ((rc = smem_attr(ssd_chunk_grad_kernel, smem))) return rc; cfg = true; }
  ssd_chunk_grad_kernel<<<dim3(nc, H, B), 128, smem, st>>>(tc, tb, tx, tdy, th, tdh, tdx, tdbh, tdch, p);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_ssd_chunk_grad launch");
}

extern "C" int nsa_ssd_chunk_grad(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x,
                                  const void* dy, const void* y, const void* Hprev_bf16, const void* dHn_bf16,
                                  const float* dt, const float* A, const float* Dskip, void* dx, float* dB_acc,
                                  float* dC_acc, float* q_out, float* k_out, int B, int T, int H, int N, int P,
                                  cudaStream_t st) {
  return ssd_chunk_grad_impl(Cm, ld_c, Bm, ld_b, x, ld_x, dy, y, Hprev_bf16, dHn_bf16, dt, A, Dskip, dx, dB_acc, dC_acc,
                             nullptr, nullptr, q_out, k_out, nullptr, B, T, H, N, P, st);
}
// Same, with dB / dC written per head as bf16 [B, T, H, N] (plain stores); the caller sums over heads.
// r_out (optional, fp32 [B, T, H]) receives dy . x per token and head.
extern "C" int nsa_ssd_chunk_grad_heads(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x,
                                        const void* dy, const void* y, const void* Hprev_bf16, const void* dHn_bf16,
                                        const float* dt, const float* A, const float* Dskip, void* dx, void* dB_heads,
                                        void* dC_heads, float* q_out, float* k_out, float* r_out, int B, int T, int H,
                                        int N, int P, cudaStream_t st) {
  if (dB_heads == nullptr || dC_heads == nullptr) return nsa::fail(NSA_ERR_SHAPE, "ssd_chunk_grad_heads: null output");
  return ssd_chunk_grad_impl(Cm, ld_c, Bm, ld_b, x, ld_x, dy, y, Hprev_bf16, dHn_bf16, dt, A, Dskip, dx, nullptr, nullptr,
                             dB_heads, dC_heads, q_out, k_out, r_out, B, T, H, N, P, st);
}
