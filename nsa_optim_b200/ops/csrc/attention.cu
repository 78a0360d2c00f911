// Attention family on tcgen05: one forward kernel and one backward kernel cover dense causal
// GQA attention, sliding-window attention, and the three branches of native sparse attention
// (compressed-block attention, selected-block attention, plus the block-importance pass that
// feeds top-n selection).
//
// Tiling.  A query tile is 128 rows = R consecutive tokens x G query heads of one KV head
// (G = Hq / Hkv, R = 128 / G), so one K/V tile serves the whole GQA group.  A key tile is 128
// keys, loaded as two 64-row TMA boxes: for dense / windowed / compressed attention they are
// adjacent, for selected-block attention they are two (not necessarily adjacent) 64-key
// selection blocks from the union of the blocks chosen by the tile's R tokens; a per-entry
// bit mask says which tokens chose which block.
//
// Forward: S = Q K^T into one of two TMEM buffers (the MMA for tile j+1 is issued before the
// softmax of tile j), each thread owns one row (tcgen05.ld 32x32b): running max with lazy
// rescaling of the TMEM-resident O accumulator, P written to shared memory as bf16 in the
// swizzled K-major layout, O += P V.  Output O (bf16) and L = log2-sum-exp (fp32).
// Backward (query-tile outer): recomputes S and dP = dO V^T, forms P and dS in registers,
// accumulates dQ in TMEM and adds each tile's dK / dV contribution to fp32 global buffers
// with vector reductions.
//
// Key positions are affine in the key index (pos = idx * kp_stride + kp_off): identity for
// ordinary attention, (stride, block-1) for compressed keys, which makes "causal on block
// end" the same comparison as ordinary causality.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "host.cuh"
#include "tc5.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128;
constexpr int BN = 128;
constexpr int HALF = 8192;          // bytes of a [64 rows][64 bf16] box

struct AttnParams {
  int B, T, S;                      // query tokens and keys per batch entry
  int Hq, Hkv, G, R, D;
  float scale_log2;                 // softmax scale * log2(e)
  int causal, window;               // window 0 = unbounded
  int kp_stride, kp_off;
  // selected-block mode (null tile_blocks = contiguous key range)
  const int* tile_blocks;           // [B, Hkv, nQt, max_u] 64-key block ids, -1 = none
  const unsigned long long* tile_masks;   // [B, Hkv, nQt, max_u] bit i: token i of the tile chose the block
  const int* tile_counts;           // [B, Hkv, nQt]
  int max_u;
  bf16* O;                          // [B, T, Hq, D]
  float* L;                         // [B, T, Hq]  log2 domain
  // importance mode
  const float* L_in;
  float* imp;                       // [B, Hkv, T, nS]
  int nS, cells_per_block;          // cells_per_block = sel_block / kp_stride
  // backward
  const bf16* dO;
  const float* delta;               // [B, T, Hq]  rowsum(dO * O)
  float* dQ;                        // unused (dQ written as bf16 below)
  bf16* dQb;                        // [B, T, Hq, D]
  float* dK;                        // [B, S, Hkv, D] fp32, pre-zeroed
  float* dV;
  KernelStatus* status;
};

// Which key tiles a query tile visits, for contiguous-range modes.
__device__ __forceinline__ void key_tile_range(const AttnParams& p, int t_lo, int t_hi, int& j0, int& j1) {
  // keys with pos <= t_hi (causal) and pos > t_lo - window (window)
  long last = p.S - 1;
  if (p.causal) {
    long lim = (static_cast<long>(t_hi) - p.kp_off);
    lim = lim < 0 ? -1 : lim / p.kp_stride;
    last = lim < last ? lim : last;
  }
  long first = 0;
  if (p.window > 0) {
    long lo = static_cast<long>(t_lo) - p.window + 1 - p.kp_off;   // pos >= t_lo - window + 1
    first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
  }
  j0 = static_cast<int>(first / BN);
  j1 = last < first ? j0 : static_cast<int>(last / BN) + 1;        // exclusive
}

// --------------------------------------------------------------------------------------
// Shared pieces of the forward and backward kernels.
//
// 256 threads: thread (r, ch) with r = threadIdx.x & 127, ch = threadIdx.x >> 7 owns query row
// r and the 64 score columns of key half ch (warps w and w+4 read the same TMEM lane quarter).
// A key half is 64 consecutive keys; per (CTA, half) a uniform flag says whether any mask test
// is needed at all, so interior tiles run the mask-free path.
// --------------------------------------------------------------------------------------
struct HalfInfo {
  int s_base;        // first key index of the half, -1 = absent
  bool row_sel;      // this thread's row may see the half at all (selection bit, row validity)
  bool need_check;   // uniform: causal / window / bounds tests needed for some element
};

__device__ __forceinline__ HalfInfo half_info(const AttnParams& p, bool selected, const int* blocks,
                                              const unsigned long long* masks, int j0, int j, int ch, int q0,
                                              int t_hi, int tok_local, bool row_ok) {
  HalfInfo hi;
  if (!selected) {
    hi.s_base = (j0 + j) * BN + ch * 64;
    hi.row_sel = row_ok;
  } else {
    const int e = 2 * j + ch;
    const int blk = e < p.max_u ? blocks[e] : -1;
    hi.s_base = blk < 0 ? -1 : blk * 64;
    const unsigned long long mk = e < p.max_u ? masks[e] : 0ull;
    hi.row_sel = row_ok && blk >= 0 && ((mk >> (tok_local & 63)) & 1ull);
  }
  const int s_lo = hi.s_base, s_hi = hi.s_base + 63;
  bool need = s_hi >= p.S;
  if (p.causal) need = need || (s_hi * p.kp_stride + p.kp_off > q0);
  if (p.window > 0) need = need || (s_lo * p.kp_stride + p.kp_off <= t_hi - p.window);
  hi.need_check = need;
  return hi;
}

__device__ __forceinline__ bool key_visible(const AttnParams& p, int s, int t) {
  const int pos = s * p.kp_stride + p.kp_off;
  bool v = s < p.S;
  if (p.causal) v = v && pos <= t;
  if (p.window > 0) v = v && pos > t - p.window;
  return v;
}

// Scores of keys sb .. sb+N-1 that query position t may not see become -inf, so that the loops
// after it need no test per element (exp2 of -inf is 0).  The visible keys of a row form one index
// range [lo, hi), computed once: a test per element inside the loops costs a branch per element.
template <int N>
__device__ __forceinline__ void mask_scores(const AttnParams& p, uint32_t (&sv)[N], int sb, int t) {
  int hi = min(N, p.S - sb), lo = 0;
  if (p.causal) {                       // (sb + i) stride + off <= t
    const int num = t - p.kp_off;
    const int last = num >= 0 ? num / p.kp_stride : -1;
    hi = min(hi, last - sb + 1);
  }
  if (p.window > 0) {                   // (sb + i) stride + off > t - window
    const int w = t - p.window - p.kp_off + 1;
    const int first = w <= 0 ? 0 : (w + p.kp_stride - 1) / p.kp_stride;
    lo = max(0, first - sb);
  }
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (i < lo || i >= hi) sv[i] = 0xff800000u;
}

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&v)[64]) {
  uint32_t a[32], b[32];
  tc5::tmem_ld_x32(taddr, a);
  tc5::tmem_ld_x32(taddr + 32, b);
  tc5::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) { v[i] = a[i]; v[32 + i] = b[i]; }
}

// write 64 bf16 (32 packed pairs) as row `row` of a [128][64] swizzled k-block
__device__ __forceinline__ void store_row64(uint8_t* kblock, int row, const uint32_t (&pk)[32]) {
  uint8_t* base = kblock + row * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(base + ((j ^ (row & 7)) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
}

// --------------------------------------------------------------------------------------
// Forward.  MODE 0: attention output + L.  MODE 1: block importance from a second pass over
// compressed keys (p = exp2(s*c - L_in), summed over the G heads of a token and binned into
// selection blocks; requires sel_block = 4 * stride and cmp_block = 2 * stride).
// --------------------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(256, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr int KB = D / 64;
  constexpr int TILE = KB * 2 * HALF;
  constexpr int DH = D / 2;                  // O columns per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;
  uint8_t* sV = sK + 2 * TILE;
  uint8_t* sP = sV + 2 * TILE;               // [2 k-blocks][128][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 4 * HALF);
  uint64_t* qbar = bars;
  uint64_t* kfull = bars + 1;
  uint64_t* vfull = bars + 3;
  uint64_t* sdone = bars + 5;
  uint64_t* odone = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(bars + 10);      // [2][128]

  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, ch = tid >> 7;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int tok_local = r / p.G, g = r % p.G;
  const int t = q0 + tok_local;
  const bool row_ok = t < p.T;
  const int t_hi = min(q0 + p.R, p.T) - 1;

  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(qbar, 1);
    for (int i = 0; i < 2; ++i) { tc5::mbar_init(&kfull[i], 1); tc5::mbar_init(&vfull[i], 1); tc5::mbar_init(&sdone[i], 1); }
    tc5::mbar_init(odone, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t cO = 256;

  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int j0 = 0, j1 = 0;
  if (selected) { j1 = (p.tile_counts[tile_slot] + 1) / 2; }
  else key_tile_range(p, q0, t_hi, j0, j1);
  const int n_tiles = j1 - j0;

  auto load_kv = [&](const CUtensorMap* tm, uint8_t* dst, uint64_t* bar, int j) {
    tc5::mbar_expect_tx(bar, TILE);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int s0;
      if (!selected) s0 = (j0 + j) * BN + hh * 64;
      else { const int e = 2 * j + hh; const int blk = e < p.max_u ? blocks[e] : -1; s0 = blk < 0 ? 0 : blk * 64; }
#pragma unroll
      for (int kb = 0; kb < KB; ++kb)
        tc5::tma_load_4d(dst + kb * 2 * HALF + hh * HALF, tm, bar, kb * 64, h, s0, b);
    }
  };
  constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t id_o = tc5::make_idesc_bf16(128, D, 0, 1);
  auto issue_s = [&](int j) {
    const uint32_t q = tc5::smem_u32(sQ), k = tc5::smem_u32(sK + (j & 1) * TILE);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      tc5::mma_ss(tmem + (j & 1) * 128, tc5::desc_kmajor(q + (kk >> 2) * 2 * HALF + (kk & 3) * 32),
                  tc5::desc_kmajor(k + (kk >> 2) * 2 * HALF + (kk & 3) * 32), id_s, kk > 0 ? 1u : 0u);
    tc5::mma_commit(&sdone[j & 1]);
  };

  if (tid == 0 && n_tiles > 0) {
    tc5::mbar_expect_tx(qbar, TILE);
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, qbar, kb * 64, 0, h, q0, b);
    load_kv(&tm_k, sK, &kfull[0], 0);
    if (MODE == 0) load_kv(&tm_v, sV, &vfull[0], 0);
    if (n_tiles > 1) load_kv(&tm_k, sK + TILE, &kfull[1], 1);
  }

  float m_ref = -INFINITY, l_sum = 0.f;
  const float Lrow = (MODE == 1 && row_ok) ? p.L_in[(static_cast<long>(b) * p.T + t) * p.Hq + h * p.G + g] : 0.f;
  const float sc = p.scale_log2;
  bool ok = true;
  for (int j = 0; j < n_tiles && ok; ++j) {
    if (tid == 0) {
      bool good = true;
      if (j == 0) {
        good = tc5::mbar_wait(qbar, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
               tc5::mbar_wait(&kfull[0], 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
        if (good) { tc5::fence_after_sync(); issue_s(0); }
      }
      if (good && j + 1 < n_tiles) {
        if (tc5::mbar_wait(&kfull[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) {
          tc5::fence_after_sync();
          issue_s(j + 1);
        }
      }
    }
    const HalfInfo hi = half_info(p, selected, blocks, masks, j0, j, ch, q0, t_hi, tok_local, row_ok);
    if (!tc5::mbar_wait(&sdone[j & 1], (j >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    if (tid == 0 && j + 2 < n_tiles) load_kv(&tm_k, sK + (j & 1) * TILE, &kfull[j & 1], j + 2);

    uint32_t sv[64];
    tmem_ld64(tmem + lane_off + (j & 1) * 128 + ch * 64, sv);

    if (MODE == 0) {
      float mx = -INFINITY;
      if (hi.row_sel) {
        if (!hi.need_check) {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (key_visible(p, hi.s_base + i, t)) mx = fmaxf(mx, __uint_as_float(sv[i]));
        }
      }
      red[ch * 128 + r] = mx;
      __syncthreads();
      mx = fmaxf(red[r], red[128 + r]) * sc;
      float alpha = 1.f;
      if (mx != -INFINITY && (m_ref == -INFINITY || mx > m_ref + 8.f)) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      // probabilities (kept packed in registers until the previous P*V has released P)
      uint32_t pk[32];
      float psum = 0.f;
      if (!hi.row_sel || m_ref == -INFINITY) {
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = 0u;
      } else if (!hi.need_check) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float a = exp2f(fmaf(__uint_as_float(sv[i]), sc, -m_ref));
          const float c = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -m_ref));
          psum += a + c;
          pk[i / 2] = tc5::pack_bf16(a, c);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float a = key_visible(p, hi.s_base + i, t) ? exp2f(fmaf(__uint_as_float(sv[i]), sc, -m_ref)) : 0.f;
          const float c = key_visible(p, hi.s_base + i + 1, t) ? exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -m_ref)) : 0.f;
          psum += a + c;
          pk[i / 2] = tc5::pack_bf16(a, c);
        }
      }
      l_sum = l_sum * alpha + psum;
      if (j > 0) {
        if (!tc5::mbar_wait(odone, (j - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
        tc5::fence_after_sync();
      }
      if (tid == 0 && ok && j + 1 < n_tiles) load_kv(&tm_v, sV + ((j + 1) & 1) * TILE, &vfull[(j + 1) & 1], j + 1);
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int q4 = 0; q4 < DH / 32; ++q4) {
          uint32_t v[32];
          tc5::tmem_ld_x32(tmem + lane_off + cO + ch * DH + q4 * 32, v);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tc5::tmem_st_x32(tmem + lane_off + cO + ch * DH + q4 * 32, v);
        }
        tc5::tmem_st_wait();
      }
      store_row64(sP + ch * 2 * HALF, r, pk);
      tc5::fence_proxy_async();
      tc5::fence_before_sync();
      if (__syncthreads_or(!ok)) { ok = false; break; }
      if (tid == 0) {
        if (tc5::mbar_wait(&vfull[j & 1], (j >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) {
          tc5::fence_after_sync();
          const uint32_t pb = tc5::smem_u32(sP), vb = tc5::smem_u32(sV + (j & 1) * TILE);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            tc5::mma_ss(tmem + cO, tc5::desc_kmajor(pb + (kk >> 2) * 2 * HALF + (kk & 3) * 32),
                        tc5::desc_mnmajor(vb + kk * 2048, 2 * HALF), id_o, (j > 0 || kk > 0) ? 1u : 0u);
          tc5::mma_commit(odone);
        }
      }
    } else {
      // importance: compressed key i covers 16-token cells i and i+1; a selection block is 4 cells
      float bins[17];
#pragma unroll
      for (int i = 0; i < 17; ++i) bins[i] = 0.f;
      if (hi.row_sel) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const bool vis = !hi.need_check || key_visible(p, hi.s_base + i, t);
          const float pr = vis ? exp2f(fmaf(__uint_as_float(sv[i]), sc, -Lrow)) : 0.f;
          bins[i / 4] += pr;
          bins[(i + 1) / 4] += pr;
        }
      }
      for (int o = p.G >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < 17; ++i) bins[i] += __shfl_xor_sync(0xffffffffu, bins[i], o);
      if (g == 0 && row_ok) {
        const int jb = (j0 + j) * (BN / 4) + ch * 16;
        float* dst = p.imp + ((static_cast<long>(b) * p.Hkv + h) * p.T + t) * p.nS;
#pragma unroll
        for (int i = 0; i < 17; ++i)
          if (jb + i < p.nS && bins[i] != 0.f) atomicAdd(dst + jb + i, bins[i]);
      }
      tc5::fence_before_sync();
      __syncthreads();
    }
  }

  if (MODE == 0) {
    if (ok && n_tiles > 0) {
      if (!tc5::mbar_wait(odone, (n_tiles - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
      tc5::fence_after_sync();
    }
    red[ch * 128 + r] = l_sum;
    const bool have = !__syncthreads_or(!ok) && n_tiles > 0;
    const float l_tot = red[r] + red[128 + r];
    const long rowi = (static_cast<long>(b) * p.T + t) * p.Hq + h * p.G + g;
    const float inv = (have && l_tot > 0.f) ? 1.f / l_tot : 0.f;
    if (row_ok && ch == 0) p.L[rowi] = (have && l_tot > 0.f) ? m_ref + log2f(l_tot) : -INFINITY;
    bf16* dst = p.O + rowi * D + ch * DH;
#pragma unroll
    for (int q4 = 0; q4 < DH / 32; ++q4) {
      uint32_t v[32];
      if (have) {
        tc5::tmem_ld_x32(tmem + lane_off + cO + ch * DH + q4 * 32, v);
        tc5::tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
          o4.y = tc5::pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
          o4.z = tc5::pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
          o4.w = tc5::pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  if (!ok && tid == 0) {
    const long long t0 = clock64();
    uint64_t* pend[5] = {qbar, &kfull[0], &kfull[1], &vfull[0], &vfull[1]};
    for (int i = 0; i < 5; ++i)
      for (uint32_t n = 0; n < (1u << 16); ++n) {
        if (tc5::mbar_try_wait(pend[i], 0) || tc5::mbar_try_wait(pend[i], 1)) break;
        if (clock64() - t0 > tc5::kMaxWaitCycles) break;
      }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Forward, warp-specialised, Q and P in tensor memory (head_dim 128, output mode).  Visits are
// 64-key blocks as in the dQ kernel.  Warp 8 streams K/V through a 5-stage ring, warp 9 issues
// S = Q K^T and warp 10 issues O += P V.  Q is copied once into TMEM and each softmax group writes
// its probabilities into TMEM columns of its own, so both MMAs take their A operand from TMEM and
// shared memory carries only the K/V stream.  P has its own columns (not those of S): a group
// releases its S buffer as soon as the scores are in registers, so S of its next visit is
// computed while this visit is exponentiated and P V runs behind the softmax, not in its chain.
// The 8 softmax warps form two groups of 128 threads (one thread per query row): group g takes
// the visits with v mod 2 = g and runs its own online softmax over them, with its own running
// maximum / sum, its own S buffer, P buffer and O accumulator in TMEM, so the groups never
// exchange anything per visit; the two partial results are merged once at the end:
//   m = max(m0, m1), O = (2^(m0-m) O0 + 2^(m1-m) O1) / (2^(m0-m) l0 + 2^(m1-m) l1).
// A group waits for P V of its previous visit (p_empty) before it rescales its O accumulator in
// place or overwrites P.
// --------------------------------------------------------------------------------------
constexpr int FWT_STAGES = 5;

__global__ void __launch_bounds__(352, 1)
attn_fwd_ts_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + QT;                        // [stages][K: 2 k-blocks of [64][64] | V: same]
  float* merge = reinterpret_cast<float*>(sKV + FWT_STAGES * 4 * HALF);   // [2][128]: group 1's m and l
  uint64_t* bars = reinterpret_cast<uint64_t*>(merge + 256);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [stages]
  uint64_t* kv_empty = kv_full + FWT_STAGES;      // [stages]
  uint64_t* s_full = kv_empty + FWT_STAGES;       // [2]
  uint64_t* s_empty = s_full + 2;                // [2]
  uint64_t* p_full = s_empty + 2;                // [2]
  uint64_t* p_empty = p_full + 2;                // [2] MMA -> softmax: P V of the group's previous visit is done
  uint64_t* qt_full = p_empty + 2;               // softmax -> MMA: Q is in tensor memory
  uint64_t* acc_done = qt_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int t_hi = min(q0 + p.R, p.T) - 1;
  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int kb0 = 0, n_vis;
  if (selected) {
    n_vis = min(p.tile_counts[tile_slot], p.max_u);
  } else {
    long last = p.S - 1;
    if (p.causal) {
      long lim = static_cast<long>(t_hi) - p.kp_off;
      lim = lim < 0 ? -1 : lim / p.kp_stride;
      last = lim < last ? lim : last;
    }
    long first = 0;
    if (p.window > 0) {
      const long lo = static_cast<long>(q0) - p.window + 1 - p.kp_off;
      first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
    }
    kb0 = static_cast<int>(first / 64);
    n_vis = last < first ? 0 : static_cast<int>(last / 64) + 1 - kb0;
  }

  if (warp == 8 && lane == 0) {        // descriptor fetch off the first copy's critical path
    tc5::prefetch_tensormap(&tm_q);
    tc5::prefetch_tensormap(&tm_k);
    tc5::prefetch_tensormap(&tm_v);
  }
  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(q_full, 1);
    for (int i = 0; i < FWT_STAGES; ++i) { tc5::mbar_init(kv_full + i, 1); tc5::mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(s_full + i, 1);
      tc5::mbar_init(s_empty + i, 128);
      tc5::mbar_init(p_full + i, 128);
      tc5::mbar_init(p_empty + i, 1);
    }
    tc5::mbar_init(qt_full, 256);
    tc5::mbar_init(acc_done, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // columns: S of group g at g*64; O of group g at 128 + g*128; Q at 384; P of group g at 448 + g*32
  constexpr uint32_t cO = 128, cQ = 384, cP = 448;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_vis > 0) {
      tc5::mbar_expect_tx(q_full, QT);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, q_full, kb * 64, 0, h, q0, b);
      bool ok = true;
      int issued = 0;
      int blk_n = selected ? blocks[0] : 0;
      for (int v = 0; v < n_vis; ++v) {
        const int st = v % FWT_STAGES;
        const int blk = blk_n;
        if (selected && v + 1 < n_vis) blk_n = blocks[v + 1];
        if (!tc5::mbar_wait(kv_empty + st, ((v / FWT_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
        const int s0 = selected ? (blk < 0 ? 0 : blk * 64) : (kb0 + v) * 64;
        uint8_t* kd = sKV + st * 4 * HALF;
        tc5::mbar_expect_tx(kv_full + st, 4 * HALF);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tc5::tma_load_4d(kd + kb * HALF, &tm_k, kv_full + st, kb * 64, h, s0, b);
          tc5::tma_load_4d(kd + 2 * HALF + kb * HALF, &tm_v, kv_full + st, kb * 64, h, s0, b);
        }
        issued = v + 1;
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        for (int j = max(0, issued - FWT_STAGES); j < issued; ++j) {
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(kv_full + (j % FWT_STAGES), (j / FWT_STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full, 0)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer 1: S = Q K^T
    // Issuing one tcgen05.mma costs the issuing thread 70 to 100 cycles here (operands of 64 keys
    // give the tensor pipe only 32 to 64 cycles of work each), so one thread issuing both products
    // is the critical path of a visit.  The two products go to two warps; every dependency
    // between them already runs through an mbarrier (p_full, s_empty, kv_empty).  Each issuing warp
    // stays converged (all lanes wait, one elected lane issues).
    if (n_vis > 0) {
      const bool lead = tc5::elect_one();
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      const uint64_t bK0 = tc5::desc_kmajor(tc5::smem_u32(sKV));
      bool ok = __all_sync(0xffffffffu, tc5::mbar_wait(qt_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
      if (ok) tc5::fence_after_sync();
      for (int v = 0; v < n_vis && ok; ++v) {
        const int st = v % FWT_STAGES, g = v & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full + st, (v / FWT_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(s_empty + g, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t bK = bK0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ts(tmem + g * 64, tmem + cQ + kk * 8, bK + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s,
                        kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + g);
        }
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ MMA issuer 2: O += P V
    if (n_vis > 0) {
      const bool lead = tc5::elect_one();
      constexpr uint32_t id_o = tc5::make_idesc_bf16(128, D, 0, 1);
      const uint64_t bVmn0 = tc5::desc_mnmajor(tc5::smem_u32(sKV) + 2 * HALF, HALF);
      bool ok = true;
      for (int u = 0; u < n_vis; ++u) {
        const int st = u % FWT_STAGES, g = u & 1;
        // V of this stage: the copy that completes kv_full brings K and V together
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full + st, (u / FWT_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(p_full + g, (u >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t bV = bVmn0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)          // O_g += P V
            tc5::mma_ts(tmem + cO + g * 128, tmem + cP + g * 32 + kk * 8, bV + static_cast<uint64_t>((kk * 2048) >> 4), id_o,
                        (u > 1 || kk > 0) ? 1u : 0u);
          // a commit covers the MMAs of this thread; S of this visit completed before P could be written
          tc5::mma_commit(kv_empty + st);
          tc5::mma_commit(p_empty + g);            // the group's P columns are free, its O accumulator is at rest
        }
        __syncwarp();
      }
      if (ok && lead) tc5::mma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int r = tid & 127, grp = tid >> 7;
    const int tok_local = r / p.G, gh = r % p.G;
    const int t = q0 + tok_local;
    const bool row_ok = t < p.T;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long rowi = (static_cast<long>(b) * p.T + (row_ok ? t : 0)) * p.Hq + h * p.G + gh;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    if (n_vis > 0) {
      // Q: shared memory (swizzled [128 rows][64] k-blocks) -> TMEM; thread (r, grp) copies k-block grp of its row
      ok = __all_sync(0xffffffffu, tc5::mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL));
      if (ok) {
        uint32_t w[32];
        const uint8_t* rowp = sQ + grp * 2 * HALF + r * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 x = *reinterpret_cast<const uint4*>(rowp + ((j ^ (r & 7)) << 4));
          w[4 * j] = x.x; w[4 * j + 1] = x.y; w[4 * j + 2] = x.z; w[4 * j + 3] = x.w;
        }
        tc5::tmem_st_x32(tmem + lane_off + cQ + grp * 32, w);
        tc5::tmem_st_wait();
        tc5::fence_before_sync();
        tc5::mbar_arrive(qt_full);
      }
    }
    int blk_n = 0;
    unsigned long long msk_n = 0ull;
    if (selected && grp < n_vis) { blk_n = blocks[grp]; msk_n = masks[grp]; }
    int n_mine = 0;
    for (int v = grp; v < n_vis && ok; v += 2, ++n_mine) {
      int sb;
      bool row_sel = row_ok;
      if (!selected) sb = (kb0 + v) * 64;
      else {
        const int blk = blk_n;
        const unsigned long long msk = msk_n;
        if (v + 2 < n_vis) { blk_n = blocks[v + 2]; msk_n = masks[v + 2]; }
        sb = blk < 0 ? -1 : blk * 64;
        row_sel = row_ok && blk >= 0 && ((msk >> (tok_local & 63)) & 1ull);
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + grp, n_mine & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[64];
      tmem_ld64(tmem + lane_off + grp * 64, sv);
      tc5::fence_before_sync();
      tc5::mbar_arrive(s_empty + grp);           // S of the group's next visit may be computed while this one is exponentiated
      bool check = false;
      float mx = -INFINITY;
      if (row_sel) {
        check = sb + 63 >= p.S;
        if (p.causal) check = check || ((sb + 63) * p.kp_stride + p.kp_off > t);
        if (p.window > 0) check = check || (sb * p.kp_stride + p.kp_off <= t - p.window);
        if (check) mask_scores<64>(p, sv, sb, t);
        // four independent chains: one serial chain of 64 dependent maxima is about 250 cycles of
        // pure latency on the critical path of every visit
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
#pragma unroll
          for (int q = 0; q < 4; ++q) m4[q] = fmaxf(m4[q], __uint_as_float(sv[i + q]));
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      mx *= sc;
      float alpha = 1.f;
      if (mx != -INFINITY && (m_ref == -INFINITY || mx > m_ref + 8.f)) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      uint32_t pk[32];
      float psum = 0.f;
      if (!row_sel || m_ref == -INFINITY) {
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = 0u;
      } else {
        float s4[4] = {0.f, 0.f, 0.f, 0.f};               // independent partial sums (see the maxima above)
#pragma unroll
        for (int i = 0; i < 64; i += 2) {                 // masked scores are -inf: their probability is 0
          const float a = exp2f(fmaf(__uint_as_float(sv[i]), sc, -m_ref));
          const float c = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -m_ref));
          s4[(i >> 1) & 3] += a + c;
          pk[i / 2] = tc5::pack_bf16(a, c);
        }
        psum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      }
      l_sum = l_sum * alpha + psum;
      // P V of the group's previous visit must be done before P is overwritten or O rescaled
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(p_empty + grp, (n_mine & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      if (n_mine > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int q4 = 0; q4 < D / 32; ++q4) {
          uint32_t o[32];
          tc5::tmem_ld_x32(tmem + lane_off + cO + grp * 128 + q4 * 32, o);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc5::tmem_st_x32(tmem + lane_off + cO + grp * 128 + q4 * 32, o);
        }
        tc5::tmem_st_wait();
      }
      tc5::tmem_st_x32(tmem + lane_off + cP + grp * 32, pk);
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(p_full + grp);
    }
    // ---- merge the two groups' partial results and write O (thread (r, grp): columns grp*64..)
    const bool done = __all_sync(0xffffffffu, ok && n_vis > 0 &&
                                 tc5::mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
    if (done) tc5::fence_after_sync();
    if (grp == 1) { merge[r] = m_ref; merge[128 + r] = l_sum; }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float m0, l0, m1, l1;
    if (grp == 0) { m0 = m_ref; l0 = l_sum; m1 = merge[r]; l1 = merge[128 + r]; }
    else { m1 = m_ref; l1 = l_sum; }
    if (grp == 0) { merge[r] = m0; merge[128 + r] = l0; }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (grp == 1) { m0 = merge[r]; l0 = merge[128 + r]; }
    const float m = fmaxf(m0, m1);
    const float w0 = (l0 > 0.f) ? exp2f(m0 - m) : 0.f;
    const float w1 = (l1 > 0.f) ? exp2f(m1 - m) : 0.f;
    const float l_tot = w0 * l0 + w1 * l1;
    const bool have = done && l_tot > 0.f;
    const float f0 = have ? w0 / l_tot : 0.f, f1 = have ? w1 / l_tot : 0.f;
    if (row_ok && grp == 0) p.L[rowi] = have ? m + log2f(l_tot) : -INFINITY;
    bf16* dst = p.O + rowi * D + grp * 64;
    // every thread of a warp takes the same branches below (done, and the visit counts, are uniform)
    const bool use0 = done && n_vis > 0, use1 = done && n_vis > 1;
#pragma unroll
    for (int q4 = 0; q4 < 2; ++q4) {
      uint32_t a[32], c[32];
      if (use0) tc5::tmem_ld_x32(tmem + lane_off + cO + grp * 64 + q4 * 32, a);
      if (use1) tc5::tmem_ld_x32(tmem + lane_off + cO + 128 + grp * 64 + q4 * 32, c);
      if (use0 || use1) tc5::tmem_ld_wait();
      if (row_ok) {
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = 0.f;
          if (use0 && f0 != 0.f) x = __uint_as_float(a[i]) * f0;
          if (use1 && f1 != 0.f) x += __uint_as_float(c[i]) * f1;
          o[i] = x;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(o[8 * i], o[8 * i + 1]);
          o4.y = tc5::pack_bf16(o[8 * i + 2], o[8 * i + 3]);
          o4.z = tc5::pack_bf16(o[8 * i + 4], o[8 * i + 5]);
          o4.w = tc5::pack_bf16(o[8 * i + 6], o[8 * i + 7]);
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Block importance for top-n selection, warp-specialised (head_dim 128).  A second pass over the
// compressed keys with the row statistics L of the compressed branch: p = 2^(S c - L), summed over
// the G heads of the group and binned into selection blocks (a compressed key covers two
// 16-token cells, a selection block four cells).  Same pipeline as the forward kernel above
// without the P V product: Q in tensor memory, K stream through the shared-memory ring, the two
// softmax groups on alternate 64-key visits.
// --------------------------------------------------------------------------------------
constexpr int IMP_STAGES = 6;

__global__ void __launch_bounds__(320, 1)
attn_importance_ts_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + QT;                        // [stages][K: 2 k-blocks of [64][64] | V: same]
  float* merge = reinterpret_cast<float*>(sKV + IMP_STAGES * 2 * HALF);   // [2][128]: group 1's m and l
  uint64_t* bars = reinterpret_cast<uint64_t*>(merge + 256);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [stages]
  uint64_t* kv_empty = kv_full + IMP_STAGES;      // [stages]
  uint64_t* s_full = kv_empty + IMP_STAGES;       // [2]
  uint64_t* s_empty = s_full + 2;                // [2]
  uint64_t* p_full = s_empty + 2;                // [2]
  uint64_t* qt_full = p_full + 2;                // softmax -> MMA: Q is in tensor memory
  uint64_t* acc_done = qt_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int t_hi = min(q0 + p.R, p.T) - 1;
  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int kb0 = 0, n_vis;
  if (selected) {
    n_vis = min(p.tile_counts[tile_slot], p.max_u);
  } else {
    long last = p.S - 1;
    if (p.causal) {
      long lim = static_cast<long>(t_hi) - p.kp_off;
      lim = lim < 0 ? -1 : lim / p.kp_stride;
      last = lim < last ? lim : last;
    }
    long first = 0;
    if (p.window > 0) {
      const long lo = static_cast<long>(q0) - p.window + 1 - p.kp_off;
      first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
    }
    kb0 = static_cast<int>(first / 64);
    n_vis = last < first ? 0 : static_cast<int>(last / 64) + 1 - kb0;
  }

  if (warp == 8 && lane == 0) {        // descriptor fetch off the first copy's critical path
    tc5::prefetch_tensormap(&tm_q);
    tc5::prefetch_tensormap(&tm_k);
  }
  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(q_full, 1);
    for (int i = 0; i < IMP_STAGES; ++i) { tc5::mbar_init(kv_full + i, 1); tc5::mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(s_full + i, 1);
      tc5::mbar_init(s_empty + i, 128);
      tc5::mbar_init(p_full + i, 128);
    }
    tc5::mbar_init(qt_full, 256);
    tc5::mbar_init(acc_done, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // columns: S of group g at g*64; O of group g at 128 + g*128
  constexpr uint32_t cO = 128, cQ = 384;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_vis > 0) {
      tc5::mbar_expect_tx(q_full, QT);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, q_full, kb * 64, 0, h, q0, b);
      bool ok = true;
      int issued = 0;
      int blk_n = selected ? blocks[0] : 0;
      for (int v = 0; v < n_vis; ++v) {
        const int st = v % IMP_STAGES;
        const int blk = blk_n;
        if (selected && v + 1 < n_vis) blk_n = blocks[v + 1];
        if (!tc5::mbar_wait(kv_empty + st, ((v / IMP_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
        const int s0 = selected ? (blk < 0 ? 0 : blk * 64) : (kb0 + v) * 64;
        uint8_t* kd = sKV + st * 2 * HALF;
        tc5::mbar_expect_tx(kv_full + st, 2 * HALF);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) tc5::tma_load_4d(kd + kb * HALF, &tm_k, kv_full + st, kb * 64, h, s0, b);
        issued = v + 1;
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        for (int j = max(0, issued - IMP_STAGES); j < issued; ++j) {
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(kv_full + (j % IMP_STAGES), (j / IMP_STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full, 0)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (converged warp, elected lane issues)
    if (n_vis > 0) {
      const bool lead = tc5::elect_one();
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      const uint64_t bK0 = tc5::desc_kmajor(tc5::smem_u32(sKV));
      bool ok = __all_sync(0xffffffffu, tc5::mbar_wait(qt_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
      if (ok) tc5::fence_after_sync();
      for (int v = 0; v < n_vis && ok; ++v) {
        const int st = v % IMP_STAGES, g = v & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full + st, (v / IMP_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(s_empty + g, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t bK = bK0 + static_cast<uint64_t>((st * 2 * HALF) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ts(tmem + g * 64, tmem + cQ + kk * 8, bK + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s,
                        kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + g);
          tc5::mma_commit(kv_empty + st);          // the K stage is free once S is complete
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int r = tid & 127, grp = tid >> 7;
    const int tok_local = r / p.G, gh = r % p.G;
    const int t = q0 + tok_local;
    const bool row_ok = t < p.T;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long rowi = (static_cast<long>(b) * p.T + (row_ok ? t : 0)) * p.Hq + h * p.G + gh;
    const float sc = p.scale_log2;
    const float Lrow = row_ok ? p.L_in[rowi] : 0.f;
    const float negL = Lrow == -INFINITY ? -INFINITY : -Lrow;     // a row that sees no key: -inf - inf, not -inf + inf
    bool ok = true;
    if (n_vis > 0) {
      // Q: shared memory (swizzled [128 rows][64] k-blocks) -> TMEM; thread (r, grp) copies k-block grp of its row
      ok = __all_sync(0xffffffffu, tc5::mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL));
      if (ok) {
        uint32_t w[32];
        const uint8_t* rowp = sQ + grp * 2 * HALF + r * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 x = *reinterpret_cast<const uint4*>(rowp + ((j ^ (r & 7)) << 4));
          w[4 * j] = x.x; w[4 * j + 1] = x.y; w[4 * j + 2] = x.z; w[4 * j + 3] = x.w;
        }
        tc5::tmem_st_x32(tmem + lane_off + cQ + grp * 32, w);
        tc5::tmem_st_wait();
        tc5::fence_before_sync();
        tc5::mbar_arrive(qt_full);
      }
    }
    int n_mine = 0;
    for (int v = grp; v < n_vis && ok; v += 2, ++n_mine) {
      const int sb = (kb0 + v) * 64;
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + grp, n_mine & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[64];
      tmem_ld64(tmem + lane_off + grp * 64, sv);
      tc5::fence_before_sync();
      tc5::mbar_arrive(s_empty + grp);
      // compressed key i covers 16-token cells i and i+1; a selection block is 4 cells
      float bins[17];
#pragma unroll
      for (int i = 0; i < 17; ++i) bins[i] = 0.f;
      if (row_ok) {
        const bool check = (sb + 63 >= p.S) || ((sb + 63) * p.kp_stride + p.kp_off > t);
        if (check) mask_scores<64>(p, sv, sb, t);
#pragma unroll
        for (int i = 0; i < 64; ++i) {                    // masked scores are -inf: their probability is 0
          const float pr = exp2f(fmaf(__uint_as_float(sv[i]), sc, negL));
          bins[i / 4] += pr;
          bins[(i + 1) / 4] += pr;
        }
      }
      for (int o = p.G >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < 17; ++i) bins[i] += __shfl_xor_sync(0xffffffffu, bins[i], o);
      if (gh == 0 && row_ok) {
        // bins 1..15 receive keys of this visit only: plain stores.  Bin 0 also receives the last key
        // of the previous visit (its bin 16), so only those two go through a reduction.
        const int jb = sb / 4;
        float* dst = p.imp + ((static_cast<long>(b) * p.Hkv + h) * p.T + t) * p.nS;
#pragma unroll
        for (int i = 1; i < 16; ++i)
          if (jb + i < p.nS) dst[jb + i] = bins[i];
        if (jb < p.nS && bins[0] != 0.f) atomicAdd(dst + jb, bins[0]);
        if (jb + 16 < p.nS && bins[16] != 0.f) atomicAdd(dst + jb + 16, bins[16]);
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Forward, warp-specialised (head_dim 128, output mode).  Visits are 64-key blocks as in the
// dQ kernel.  Warp 8 streams K/V through a 4-stage ring, warp 9 issues S = Q K^T and O += P V.
// The 8 softmax warps form two groups of 128 threads (one thread per query row): group g takes
// the visits with v mod 2 = g and runs its own online softmax over them, with its own running
// maximum / sum, its own S buffer, P buffer and O accumulator in TMEM, so the groups never
// exchange anything per visit; the two partial results are merged once at the end:
//   m = max(m0, m1), O = (2^(m0-m) O0 + 2^(m1-m) O1) / (2^(m0-m) l0 + 2^(m1-m) l1).
// tcgen05 MMAs complete in issue order, and S of visit v is issued after P V of visit v-2, so a
// group that has received S_v may rescale its O accumulator in place.
// --------------------------------------------------------------------------------------
constexpr int FW_STAGES = 4;

__global__ void __launch_bounds__(320, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + QT;                        // [stages][K: 2 k-blocks of [64][64] | V: same]
  uint8_t* sP = sKV + FW_STAGES * 4 * HALF;      // [2 groups][128 rows][64 keys]
  float* merge = reinterpret_cast<float*>(sP + 4 * HALF);   // [2][128]: group 1's m and l
  uint64_t* bars = reinterpret_cast<uint64_t*>(merge + 256);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [stages]
  uint64_t* kv_empty = kv_full + FW_STAGES;      // [stages]
  uint64_t* s_full = kv_empty + FW_STAGES;       // [2]
  uint64_t* s_empty = s_full + 2;                // [2]
  uint64_t* p_full = s_empty + 2;                // [2]
  uint64_t* p_empty = p_full + 2;                // [2]
  uint64_t* acc_done = p_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int t_hi = min(q0 + p.R, p.T) - 1;
  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int kb0 = 0, n_vis;
  if (selected) {
    n_vis = min(p.tile_counts[tile_slot], p.max_u);
  } else {
    long last = p.S - 1;
    if (p.causal) {
      long lim = static_cast<long>(t_hi) - p.kp_off;
      lim = lim < 0 ? -1 : lim / p.kp_stride;
      last = lim < last ? lim : last;
    }
    long first = 0;
    if (p.window > 0) {
      const long lo = static_cast<long>(q0) - p.window + 1 - p.kp_off;
      first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
    }
    kb0 = static_cast<int>(first / 64);
    n_vis = last < first ? 0 : static_cast<int>(last / 64) + 1 - kb0;
  }

  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(q_full, 1);
    for (int i = 0; i < FW_STAGES; ++i) { tc5::mbar_init(kv_full + i, 1); tc5::mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(s_full + i, 1);
      tc5::mbar_init(s_empty + i, 128);
      tc5::mbar_init(p_full + i, 128);
      tc5::mbar_init(p_empty + i, 1);
    }
    tc5::mbar_init(acc_done, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // columns: S of group g at g*64; O of group g at 128 + g*128
  constexpr uint32_t cO = 128;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_vis > 0) {
      tc5::mbar_expect_tx(q_full, QT);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, q_full, kb * 64, 0, h, q0, b);
      bool ok = true;
      int issued = 0;
      int blk_n = selected ? blocks[0] : 0;
      for (int v = 0; v < n_vis; ++v) {
        const int st = v % FW_STAGES;
        const int blk = blk_n;
        if (selected && v + 1 < n_vis) blk_n = blocks[v + 1];
        if (!tc5::mbar_wait(kv_empty + st, ((v / FW_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
        const int s0 = selected ? (blk < 0 ? 0 : blk * 64) : (kb0 + v) * 64;
        uint8_t* kd = sKV + st * 4 * HALF;
        tc5::mbar_expect_tx(kv_full + st, 4 * HALF);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tc5::tma_load_4d(kd + kb * HALF, &tm_k, kv_full + st, kb * 64, h, s0, b);
          tc5::tma_load_4d(kd + 2 * HALF + kb * HALF, &tm_v, kv_full + st, kb * 64, h, s0, b);
        }
        issued = v + 1;
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        for (int j = max(0, issued - FW_STAGES); j < issued; ++j) {
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(kv_full + (j % FW_STAGES), (j / FW_STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full, 0)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_vis > 0) {
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t id_o = tc5::make_idesc_bf16(128, D, 0, 1);
      uint64_t aQ[D / 16];
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) aQ[kk] = tc5::desc_kmajor(tc5::smem_u32(sQ) + (kk >> 2) * 2 * HALF + (kk & 3) * 32);
      const uint64_t bK0 = tc5::desc_kmajor(tc5::smem_u32(sKV));
      const uint64_t bVmn0 = tc5::desc_mnmajor(tc5::smem_u32(sKV) + 2 * HALF, HALF);
      const uint64_t aP0 = tc5::desc_kmajor(tc5::smem_u32(sP));
      bool ok = tc5::mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
      for (int v = 0; v <= n_vis && ok; ++v) {
        if (v < n_vis) {
          const int st = v % FW_STAGES, g = v & 1;
          if (!tc5::mbar_wait(kv_full + st, (v / FW_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          if (!tc5::mbar_wait(s_empty + g, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint64_t bK = bK0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ss(tmem + g * 64, aQ[kk], bK + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s,
                        kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + g);
        }
        if (v >= 1) {
          const int u = v - 1, st = u % FW_STAGES, g = u & 1;
          if (!tc5::mbar_wait(p_full + g, (u >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint64_t aP = aP0 + static_cast<uint64_t>((g * 2 * HALF) >> 4);
          const uint64_t bV = bVmn0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)          // O_g += P V  (64 keys per visit)
            tc5::mma_ss(tmem + cO + g * 128, aP + static_cast<uint64_t>((kk * 32) >> 4), bV + static_cast<uint64_t>((kk * 2048) >> 4),
                        id_o, (u > 1 || kk > 0) ? 1u : 0u);
          tc5::mma_commit(kv_empty + st);
          tc5::mma_commit(p_empty + g);
        }
      }
      if (ok) tc5::mma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax groups
    const int r = tid & 127, grp = tid >> 7;
    const int tok_local = r / p.G, gh = r % p.G;
    const int t = q0 + tok_local;
    const bool row_ok = t < p.T;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long rowi = (static_cast<long>(b) * p.T + (row_ok ? t : 0)) * p.Hq + h * p.G + gh;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    int blk_n = 0;
    unsigned long long msk_n = 0ull;
    if (selected && grp < n_vis) { blk_n = blocks[grp]; msk_n = masks[grp]; }
    int n_mine = 0;
    for (int v = grp; v < n_vis; v += 2, ++n_mine) {
      int sb;
      bool row_sel = row_ok;
      if (!selected) sb = (kb0 + v) * 64;
      else {
        const int blk = blk_n;
        const unsigned long long msk = msk_n;
        if (v + 2 < n_vis) { blk_n = blocks[v + 2]; msk_n = masks[v + 2]; }
        sb = blk < 0 ? -1 : blk * 64;
        row_sel = row_ok && blk >= 0 && ((msk >> (tok_local & 63)) & 1ull);
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + grp, n_mine & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[64];
      tmem_ld64(tmem + lane_off + grp * 64, sv);
      tc5::fence_before_sync();
      tc5::mbar_arrive(s_empty + grp);
      bool check = false;
      float mx = -INFINITY;
      if (row_sel) {
        check = sb + 63 >= p.S;
        if (p.causal) check = check || ((sb + 63) * p.kp_stride + p.kp_off > t);
        if (p.window > 0) check = check || (sb * p.kp_stride + p.kp_off <= t - p.window);
        if (check) mask_scores<64>(p, sv, sb, t);
        // four independent chains: one serial chain of 64 dependent maxima is about 250 cycles of
        // pure latency on the critical path of every visit
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
#pragma unroll
          for (int q = 0; q < 4; ++q) m4[q] = fmaxf(m4[q], __uint_as_float(sv[i + q]));
        }
        mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      }
      mx *= sc;
      float alpha = 1.f;
      if (mx != -INFINITY && (m_ref == -INFINITY || mx > m_ref + 8.f)) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
      }
      uint32_t pk[32];
      float psum = 0.f;
      if (!row_sel || m_ref == -INFINITY) {
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = 0u;
      } else {
        float s4[4] = {0.f, 0.f, 0.f, 0.f};               // independent partial sums (see the maxima above)
#pragma unroll
        for (int i = 0; i < 64; i += 2) {                 // masked scores are -inf: their probability is 0
          const float a = exp2f(fmaf(__uint_as_float(sv[i]), sc, -m_ref));
          const float c = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -m_ref));
          s4[(i >> 1) & 3] += a + c;
          pk[i / 2] = tc5::pack_bf16(a, c);
        }
        psum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      }
      l_sum = l_sum * alpha + psum;
      // O_g is quiescent here: P V of this group's previous visit completed before S of this visit
      if (n_mine > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int q4 = 0; q4 < D / 32; ++q4) {
          uint32_t o[32];
          tc5::tmem_ld_x32(tmem + lane_off + cO + grp * 128 + q4 * 32, o);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc5::tmem_st_x32(tmem + lane_off + cO + grp * 128 + q4 * 32, o);
        }
        tc5::tmem_st_wait();
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(p_empty + grp, (n_mine & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY))) {
        ok = false;
        break;
      }
      store_row64(sP + grp * 2 * HALF, r, pk);
      tc5::fence_proxy_async();
      tc5::fence_before_sync();
      tc5::mbar_arrive(p_full + grp);
    }
    // ---- merge the two groups' partial results and write O (thread (r, grp): columns grp*64..)
    const bool done = __all_sync(0xffffffffu, ok && n_vis > 0 &&
                                 tc5::mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
    if (done) tc5::fence_after_sync();
    if (grp == 1) { merge[r] = m_ref; merge[128 + r] = l_sum; }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float m0, l0, m1, l1;
    if (grp == 0) { m0 = m_ref; l0 = l_sum; m1 = merge[r]; l1 = merge[128 + r]; }
    else { m1 = m_ref; l1 = l_sum; }
    if (grp == 0) { merge[r] = m0; merge[128 + r] = l0; }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (grp == 1) { m0 = merge[r]; l0 = merge[128 + r]; }
    const float m = fmaxf(m0, m1);
    const float w0 = (l0 > 0.f) ? exp2f(m0 - m) : 0.f;
    const float w1 = (l1 > 0.f) ? exp2f(m1 - m) : 0.f;
    const float l_tot = w0 * l0 + w1 * l1;
    const bool have = done && l_tot > 0.f;
    const float f0 = have ? w0 / l_tot : 0.f, f1 = have ? w1 / l_tot : 0.f;
    if (row_ok && grp == 0) p.L[rowi] = have ? m + log2f(l_tot) : -INFINITY;
    bf16* dst = p.O + rowi * D + grp * 64;
    // every thread of a warp takes the same branches below (done, and the visit counts, are uniform)
    const bool use0 = done && n_vis > 0, use1 = done && n_vis > 1;
#pragma unroll
    for (int q4 = 0; q4 < 2; ++q4) {
      uint32_t a[32], c[32];
      if (use0) tc5::tmem_ld_x32(tmem + lane_off + cO + grp * 64 + q4 * 32, a);
      if (use1) tc5::tmem_ld_x32(tmem + lane_off + cO + 128 + grp * 64 + q4 * 32, c);
      if (use0 || use1) tc5::tmem_ld_wait();
      if (row_ok) {
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = 0.f;
          if (use0 && f0 != 0.f) x = __uint_as_float(a[i]) * f0;
          if (use1 && f1 != 0.f) x += __uint_as_float(c[i]) * f1;
          o[i] = x;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(o[8 * i], o[8 * i + 1]);
          o4.y = tc5::pack_bf16(o[8 * i + 2], o[8 * i + 3]);
          o4.z = tc5::pack_bf16(o[8 * i + 4], o[8 * i + 5]);
          o4.w = tc5::pack_bf16(o[8 * i + 6], o[8 * i + 7]);
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Backward, query-tile outer.  Per key tile: S = Q K^T and dP = dO V^T (TMEM), then in
// registers P = exp2(S c - L), dS = P (dP - delta) scale; then dQ += dS K (TMEM resident),
// and the tile's dV = P^T dO, dK = dS^T Q are added to fp32 global buffers.
// --------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const AttnParams p, const float scale) {
  constexpr int KB = D / 64;
  constexpr int TILE = KB * 2 * HALF;
  constexpr int DH = D / 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sK = sDO + TILE;
  uint8_t* sV = sK + TILE;
  uint8_t* sP = sV + TILE;
  uint8_t* sDS = sP + 4 * HALF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 4 * HALF);
  uint64_t* qbar = bars;
  uint64_t* kvbar = bars + 1;
  uint64_t* m1 = bars + 2;
  uint64_t* m2 = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127, ch = tid >> 7;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int tok_local = r / p.G, g = r % p.G;
  const int t = q0 + tok_local;
  const bool row_ok = t < p.T;
  const int t_hi = min(q0 + p.R, p.T) - 1;

  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(qbar, 1);
    tc5::mbar_init(kvbar, 1);
    tc5::mbar_init(m1, 1);
    tc5::mbar_init(m2, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 0) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t cS = 0, cDP = 128, cDQ = 256, cDV = 384, cDK = 0;   // dK reuses the S columns

  const bool selected = p.tile_blocks != nullptr;
  const bool with_dkv = p.dK != nullptr;          // null: dK / dV come from the key-stationary kernel
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int j0 = 0, j1 = 0;
  if (selected) { j1 = (p.tile_counts[tile_slot] + 1) / 2; }
  else key_tile_range(p, q0, t_hi, j0, j1);
  const int n_tiles = j1 - j0;

  const long rowi = (static_cast<long>(b) * p.T + t) * p.Hq + h * p.G + g;
  const float Lrow = row_ok ? p.L[rowi] : 0.f;
  const float drow = row_ok ? p.delta[rowi] : 0.f;
  const float sc = p.scale_log2;

  if (tid == 0 && n_tiles > 0) {
    tc5::mbar_expect_tx(qbar, 2 * TILE);
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, qbar, kb * 64, 0, h, q0, b);
      tc5::tma_load_5d(sDO + kb * 2 * HALF, &tm_do, qbar, kb * 64, 0, h, q0, b);
    }
  }
  constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t id_q = tc5::make_idesc_bf16(128, D, 0, 1);
  constexpr uint32_t id_t = tc5::make_idesc_bf16(128, D, 1, 1);
  bool ok = true;
  for (int j = 0; j < n_tiles && ok; ++j) {
    const HalfInfo hi = half_info(p, selected, blocks, masks, j0, j, ch, q0, t_hi, tok_local, row_ok);
    if (tid == 0) {
      tc5::mbar_expect_tx(kvbar, 2 * TILE);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int s0;
        if (!selected) s0 = (j0 + j) * BN + hh * 64;
        else { const int e = 2 * j + hh; const int blk = e < p.max_u ? blocks[e] : -1; s0 = blk < 0 ? 0 : blk * 64; }
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tc5::tma_load_4d(sK + kb * 2 * HALF + hh * HALF, &tm_k, kvbar, kb * 64, h, s0, b);
          tc5::tma_load_4d(sV + kb * 2 * HALF + hh * HALF, &tm_v, kvbar, kb * 64, h, s0, b);
        }
      }
      bool good = true;
      if (j == 0) good = tc5::mbar_wait(qbar, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
      if (good && tc5::mbar_wait(kvbar, j & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) {
        tc5::fence_after_sync();
        const uint32_t q = tc5::smem_u32(sQ), dob = tc5::smem_u32(sDO), k = tc5::smem_u32(sK), v = tc5::smem_u32(sV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 2 * HALF + (kk & 3) * 32;
          tc5::mma_ss(tmem + cS, tc5::desc_kmajor(q + off), tc5::desc_kmajor(k + off), id_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 2 * HALF + (kk & 3) * 32;
          tc5::mma_ss(tmem + cDP, tc5::desc_kmajor(dob + off), tc5::desc_kmajor(v + off), id_s, kk > 0 ? 1u : 0u);
        }
        tc5::mma_commit(m1);
      }
    }
    if (!tc5::mbar_wait(m1, j & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    {
      uint32_t sv[64], dv[64], pp[32], ds[32];
      tmem_ld64(tmem + lane_off + cS + ch * 64, sv);
      tmem_ld64(tmem + lane_off + cDP + ch * 64, dv);
      if (!hi.row_sel) {
#pragma unroll
        for (int i = 0; i < 32; ++i) { pp[i] = 0u; ds[i] = 0u; }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const bool v0 = !hi.need_check || key_visible(p, hi.s_base + i, t);
          const bool v1 = !hi.need_check || key_visible(p, hi.s_base + i + 1, t);
          const float p0 = v0 ? exp2f(fmaf(__uint_as_float(sv[i]), sc, -Lrow)) : 0.f;
          const float p1 = v1 ? exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -Lrow)) : 0.f;
          pp[i / 2] = tc5::pack_bf16(p0, p1);
          ds[i / 2] = tc5::pack_bf16(p0 * (__uint_as_float(dv[i]) - drow) * scale,
                                     p1 * (__uint_as_float(dv[i + 1]) - drow) * scale);
        }
      }
      store_row64(sP + ch * 2 * HALF, r, pp);
      store_row64(sDS + ch * 2 * HALF, r, ds);
    }
    tc5::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc5::fence_after_sync();
      const uint32_t q = tc5::smem_u32(sQ), dob = tc5::smem_u32(sDO), k = tc5::smem_u32(sK);
      const uint32_t pb = tc5::smem_u32(sP), dsb = tc5::smem_u32(sDS);
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk)      // dQ += dS K
        tc5::mma_ss(tmem + cDQ, tc5::desc_kmajor(dsb + (kk >> 2) * 2 * HALF + (kk & 3) * 32),
                    tc5::desc_mnmajor(k + kk * 2048, 2 * HALF), id_q, (j > 0 || kk > 0) ? 1u : 0u);
      if (with_dkv) {
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)      // dV_tile = P^T dO
          tc5::mma_ss(tmem + cDV, tc5::desc_mnmajor(pb + kk * 2048, 2 * HALF),
                      tc5::desc_mnmajor(dob + kk * 2048, 2 * HALF), id_t, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk)      // dK_tile = dS^T Q
          tc5::mma_ss(tmem + cDK, tc5::desc_mnmajor(dsb + kk * 2048, 2 * HALF),
                      tc5::desc_mnmajor(q + kk * 2048, 2 * HALF), id_t, kk > 0 ? 1u : 0u);
      }
      tc5::mma_commit(m2);
    }
    // thread (r, ch) owns key row r of the tile, D-half ch
    int sb_r;
    if (!selected) sb_r = (j0 + j) * BN + (r >> 6) * 64;
    else { const int e = 2 * j + (r >> 6); const int blk = e < p.max_u ? blocks[e] : -1; sb_r = blk < 0 ? -1 : blk * 64; }
    const int s_r = sb_r + (r & 63);
    const bool key_ok = sb_r >= 0 && s_r < p.S;
    const long krow = ((static_cast<long>(b) * p.S + (key_ok ? s_r : 0)) * p.Hkv + h) * D + ch * DH;
    if (!tc5::mbar_wait(m2, j & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc5::fence_after_sync();
    if (with_dkv)
#pragma unroll
    for (int q4 = 0; q4 < DH / 32; ++q4) {
      uint32_t a[32], c[32];
      tc5::tmem_ld_x32(tmem + lane_off + cDV + ch * DH + q4 * 32, a);
      tc5::tmem_ld_x32(tmem + lane_off + cDK + ch * DH + q4 * 32, c);
      tc5::tmem_ld_wait();
      if (key_ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          atomicAdd(reinterpret_cast<float4*>(p.dV + krow + q4 * 32) + i,
                    make_float4(__uint_as_float(a[4 * i]), __uint_as_float(a[4 * i + 1]),
                                __uint_as_float(a[4 * i + 2]), __uint_as_float(a[4 * i + 3])));
          atomicAdd(reinterpret_cast<float4*>(p.dK + krow + q4 * 32) + i,
                    make_float4(__uint_as_float(c[4 * i]), __uint_as_float(c[4 * i + 1]),
                                __uint_as_float(c[4 * i + 2]), __uint_as_float(c[4 * i + 3])));
        }
      }
    }
    tc5::fence_before_sync();
    __syncthreads();
  }
  {
    const bool have = !__syncthreads_or(!ok) && n_tiles > 0;
    bf16* dst = p.dQb + rowi * D + ch * DH;
#pragma unroll
    for (int q4 = 0; q4 < DH / 32; ++q4) {
      uint32_t v[32];
      if (have) {
        tc5::tmem_ld_x32(tmem + lane_off + cDQ + ch * DH + q4 * 32, v);
        tc5::tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1]));
          o4.y = tc5::pack_bf16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
          o4.z = tc5::pack_bf16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
          o4.w = tc5::pack_bf16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  if (!ok && tid == 0) {
    const long long t0 = clock64();
    uint64_t* pend[2] = {qbar, kvbar};
    for (int i = 0; i < 2; ++i)
      for (uint32_t n = 0; n < (1u << 16); ++n) {
        if (tc5::mbar_try_wait(pend[i], 0) || tc5::mbar_try_wait(pend[i], 1)) break;
        if (clock64() - t0 > tc5::kMaxWaitCycles) break;
      }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Backward for dQ with the stationary operands in tensor memory.  The shared-memory variant
// below re-reads Q and dO (4 KB per MMA) for every 64-key visit and writes dS through shared
// memory: about 176 KB of shared-memory traffic per visit, which bounds it.  Here Q and dO are
// copied once into TMEM (bf16 pairs, 64 columns each) and used as the A operand of
// tcgen05.mma; dS is written back into the S columns it was computed from (each thread into the
// first half of its own column range) and is the A operand of dQ += dS K.  Shared memory then
// carries only the K/V stream.  Same roles as the dK/dV kernel below:
// warps 0-7 turn S and dP into dS, warp 8 streams 64-key K/V blocks through a 5-stage ring,
// warps 9, 10 and 11 issue S = Q K^T, dP = dO V^T (double-buffered in TMEM) and dQ += dS K
// (resident in TMEM).  Visits are 64-key blocks: the contiguous range allowed by causality / window, or the
// entries of the tile's union list (selected mode, with the per-token bit masks).
// Needs D = 128.
// --------------------------------------------------------------------------------------
constexpr int DQT_STAGES = 5;

__global__ void __launch_bounds__(384, 1)
attn_bwd_dq_ts_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const AttnParams p, const float scale) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + QT;
  uint8_t* sKV = sDO + QT;                       // [stages][K: 2 k-blocks of [64][64] | V: same]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + DQT_STAGES * 4 * HALF);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [stages] TMA -> MMA
  uint64_t* kv_empty = kv_full + DQT_STAGES;      // [stages] MMA -> TMA
  uint64_t* s_full = kv_empty + DQT_STAGES;       // [2] MMA -> softmax
  uint64_t* s_empty = s_full + 2;                // [2] softmax -> MMA
  // One dS barrier per S buffer: warps whose rows are all masked finish a visit early and may
  // already be in the next visit (other buffer); with a single barrier their second arrival
  // would complete the phase of the visit the slower warps are still writing.
  uint64_t* ds_full = s_empty + 2;               // [2] softmax -> MMA
  uint64_t* qt_full = ds_full + 2;               // softmax -> MMA: Q and dO are in tensor memory
  uint64_t* acc_done = qt_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int t_hi = min(q0 + p.R, p.T) - 1;
  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int kb0 = 0, n_vis;
  if (selected) {
    n_vis = min(p.tile_counts[tile_slot], p.max_u);
  } else {
    long last = p.S - 1;
    if (p.causal) {
      long lim = static_cast<long>(t_hi) - p.kp_off;
      lim = lim < 0 ? -1 : lim / p.kp_stride;
      last = lim < last ? lim : last;
    }
    long first = 0;
    if (p.window > 0) {
      const long lo = static_cast<long>(q0) - p.window + 1 - p.kp_off;
      first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
    }
    kb0 = static_cast<int>(first / 64);
    n_vis = last < first ? 0 : static_cast<int>(last / 64) + 1 - kb0;
  }

  if (warp == 8 && lane == 0) {        // descriptor fetch off the first copy's critical path
    tc5::prefetch_tensormap(&tm_q);
    tc5::prefetch_tensormap(&tm_do);
    tc5::prefetch_tensormap(&tm_k);
    tc5::prefetch_tensormap(&tm_v);
  }
  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(q_full, 1);
    for (int i = 0; i < DQT_STAGES; ++i) { tc5::mbar_init(kv_full + i, 1); tc5::mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) { tc5::mbar_init(s_full + i, 2); tc5::mbar_init(s_empty + i, 1); }
    tc5::mbar_init(ds_full, 256);
    tc5::mbar_init(ds_full + 1, 256);
    tc5::mbar_init(qt_full, 256);
    tc5::mbar_init(acc_done, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cDQ = 256, cQ = 384, cDO = 448;   // S/dP of buffer i at i*128 + {0, 64}

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_vis > 0) {
      tc5::mbar_expect_tx(q_full, 2 * QT);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, q_full, kb * 64, 0, h, q0, b);
        tc5::tma_load_5d(sDO + kb * 2 * HALF, &tm_do, q_full, kb * 64, 0, h, q0, b);
      }
      bool ok = true;
      int issued = 0;
      int blk_n = selected ? blocks[0] : 0;
      for (int v = 0; v < n_vis; ++v) {
        const int st = v % DQT_STAGES;
        const int blk = blk_n;
        if (selected && v + 1 < n_vis) blk_n = blocks[v + 1];
        if (!tc5::mbar_wait(kv_empty + st, ((v / DQT_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
        int s0;
        if (!selected) s0 = (kb0 + v) * 64;
        else s0 = blk < 0 ? 0 : blk * 64;
        uint8_t* kd = sKV + st * 4 * HALF;
        tc5::mbar_expect_tx(kv_full + st, 4 * HALF);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tc5::tma_load_4d(kd + kb * HALF, &tm_k, kv_full + st, kb * 64, h, s0, b);
          tc5::tma_load_4d(kd + 2 * HALF + kb * HALF, &tm_v, kv_full + st, kb * 64, h, s0, b);
        }
        issued = v + 1;
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        for (int j = max(0, issued - DQT_STAGES); j < issued; ++j) {
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(kv_full + (j % DQT_STAGES), (j / DQT_STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full, 0)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers 1 and 2: S = Q K^T, dP = dO V^T
    // Three issuing warps, each converged with one elected lane issuing (see the forward kernel):
    // warp 9 issues S, warp 10 dP, warp 11 dQ += dS K.  s_full counts one commit of each of the
    // first two.  The address field (bits 0-13, address >> 4) of a shared-memory descriptor is
    // advanced by adding the byte offset >> 4.
    if (n_vis > 0) {
      const bool lead = tc5::elect_one();
      const bool is_dp = warp == 10;
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      const uint64_t b0 = tc5::desc_kmajor(tc5::smem_u32(sKV) + (is_dp ? 2 * HALF : 0));   // stage 0, K or V, k-step 0
      const uint32_t acol = is_dp ? cDO : cQ, dcol = is_dp ? 64u : 0u;
      bool ok = __all_sync(0xffffffffu, tc5::mbar_wait(qt_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
      if (ok) tc5::fence_after_sync();
      for (int v = 0; v < n_vis && ok; ++v) {
        const int st = v % DQT_STAGES, buf = v & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full + st, (v / DQT_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(s_empty + buf, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t bB = b0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)      // a k-step of 16 bf16 is 8 TMEM columns of the A operand
            tc5::mma_ts(tmem + buf * 128 + dcol, tmem + acol + kk * 8, bB + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4),
                        id_s, kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + buf);
        }
        __syncwarp();
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------ MMA issuer 3: dQ += dS K
    if (n_vis > 0) {
      const bool lead = tc5::elect_one();
      constexpr uint32_t id_q = tc5::make_idesc_bf16(128, D, 0, 1);
      const uint64_t bKmn0 = tc5::desc_mnmajor(tc5::smem_u32(sKV), HALF);    // the K tile as an MN-major operand
      bool ok = true;
      for (int u = 0; u < n_vis; ++u) {
        const int st = u % DQT_STAGES, buf = u & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full + st, (u / DQT_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(ds_full + buf, (u >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t bKmn = bKmn0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)          // dQ += dS K: keys 0-31 sit in columns 0-15, keys 32-63 in columns 32-47
            tc5::mma_ts(tmem + cDQ, tmem + buf * 128 + (kk >> 1) * 32 + (kk & 1) * 8, bKmn + static_cast<uint64_t>((kk * 2048) >> 4),
                        id_q, (u > 0 || kk > 0) ? 1u : 0u);
          // S and dP of this visit completed before dS could be written, so the commits of this warp
          // alone release the stage and the buffer
          tc5::mma_commit(kv_empty + st);
          tc5::mma_commit(s_empty + buf);          // the S / dP / dS columns of this buffer are free again
        }
        __syncwarp();
      }
      if (ok && lead) tc5::mma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int r = tid & 127, ch = tid >> 7;
    const int tok_local = r / p.G, g = r % p.G;
    const int t = q0 + tok_local;
    const bool row_ok = t < p.T;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long rowi = (static_cast<long>(b) * p.T + (row_ok ? t : 0)) * p.Hq + h * p.G + g;
    const float Lrow = row_ok ? p.L[rowi] : 0.f;
    const float negL = Lrow == -INFINITY ? -INFINITY : -Lrow;     // a row that sees no key: -inf - inf, not -inf + inf
    const float drow = row_ok ? p.delta[rowi] : 0.f;
    const float nds = -drow * scale;
    const float sc = p.scale_log2;
    bool ok = true;
    if (n_vis > 0) {
      // Q and dO: shared memory (swizzled [128 rows][64] k-blocks) -> TMEM, thread (r, ch) copies the
      // 64 elements of k-block ch of its row as 32 packed words
      ok = __all_sync(0xffffffffu, tc5::mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL));
      if (ok) {
        uint32_t w[32];
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint8_t* rowp = (which ? sDO : sQ) + ch * 2 * HALF + r * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 x = *reinterpret_cast<const uint4*>(rowp + ((j ^ (r & 7)) << 4));
            w[4 * j] = x.x; w[4 * j + 1] = x.y; w[4 * j + 2] = x.z; w[4 * j + 3] = x.w;
          }
          tc5::tmem_st_x32(tmem + lane_off + (which ? cDO : cQ) + ch * 32, w);
          tc5::tmem_st_wait();                     // before the registers are reused for the second operand
        }
        tc5::fence_before_sync();
        tc5::mbar_arrive(qt_full);
      }
    }
    // selected mode: the block id and token mask of visit v+1 are fetched during visit v, so the
    // global-memory latency is off the per-visit critical path
    int blk_n = (selected && n_vis > 0) ? blocks[0] : 0;
    unsigned long long msk_n = (selected && n_vis > 0) ? masks[0] : 0ull;
    for (int v = 0; v < n_vis && ok; ++v) {
      const int buf = v & 1;
      int sb;
      bool row_sel = row_ok;
      if (!selected) sb = (kb0 + v) * 64 + ch * 32;
      else {
        const int blk = blk_n;
        const unsigned long long msk = msk_n;
        if (v + 1 < n_vis) { blk_n = blocks[v + 1]; msk_n = masks[v + 1]; }
        sb = blk < 0 ? -1 : blk * 64 + ch * 32;
        row_sel = row_ok && blk >= 0 && ((msk >> (tok_local & 63)) & 1ull);
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + buf, (v >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[32], dv[32], ds[16];
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + ch * 32, sv);
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + 64 + ch * 32, dv);
      tc5::tmem_ld_wait();
      if (!row_sel) {
#pragma unroll
        for (int i = 0; i < 16; ++i) ds[i] = 0u;
      } else {
        bool check = sb + 31 >= p.S;
        if (p.causal) check = check || ((sb + 31) * p.kp_stride + p.kp_off > t);
        if (p.window > 0) check = check || (sb * p.kp_stride + p.kp_off <= t - p.window);
        if (check) mask_scores<32>(p, sv, sb, t);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {                 // masked scores are -inf: their probability is 0
          const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sc, negL));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, negL));
          ds[i / 2] = tc5::pack_bf16(p0 * fmaf(__uint_as_float(dv[i]), scale, nds),
                                     p1 * fmaf(__uint_as_float(dv[i + 1]), scale, nds));
        }
      }
      // dS replaces the first half of this thread's own S columns
      tc5::tmem_st_x16(tmem + lane_off + buf * 128 + ch * 32, ds);
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(ds_full + buf);
    }
    // ---- dQ: thread (r, ch) stores D-half ch of row r
    const bool have = __all_sync(0xffffffffu, ok && n_vis > 0 &&
                                 tc5::mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
    if (have) tc5::fence_after_sync();
    bf16* dst = p.dQb + rowi * D + ch * 64;
#pragma unroll
    for (int q4 = 0; q4 < 2; ++q4) {
      uint32_t a[32];
      if (have) {
        tc5::tmem_ld_x32(tmem + lane_off + cDQ + ch * 64 + q4 * 32, a);
        tc5::tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) a[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(__uint_as_float(a[8 * i]), __uint_as_float(a[8 * i + 1]));
          o4.y = tc5::pack_bf16(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3]));
          o4.z = tc5::pack_bf16(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5]));
          o4.w = tc5::pack_bf16(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7]));
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Backward for dQ, query-tile stationary, pipelined.  Same roles as the dK/dV kernel below:
// warps 0-7 turn S and dP into dS, warp 8 streams 64-key K/V blocks through a 5-stage ring,
// warps 9, 10 and 11 issue S = Q K^T, dP = dO V^T (double-buffered in TMEM) and dQ += dS K
// (resident in TMEM).  Visits are 64-key blocks: the contiguous range allowed by causality / window, or the
// entries of the tile's union list (selected mode, with the per-token bit masks).
// Needs D = 128.
// --------------------------------------------------------------------------------------
constexpr int DQ_STAGES = 4;

__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const AttnParams p, const float scale) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + QT;
  uint8_t* sKV = sDO + QT;                       // [stages][K: 2 k-blocks of [64][64] | V: same]
  uint8_t* sDS = sKV + DQ_STAGES * 4 * HALF;     // [128 rows][64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * HALF);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                  // [stages] TMA -> MMA
  uint64_t* kv_empty = kv_full + DQ_STAGES;      // [stages] MMA -> TMA
  uint64_t* s_full = kv_empty + DQ_STAGES;       // [2] MMA -> softmax
  uint64_t* s_empty = s_full + 2;                // [2] softmax -> MMA
  uint64_t* ds_full = s_empty + 2;               // softmax -> MMA
  uint64_t* ds_empty = ds_full + 1;              // MMA -> softmax
  uint64_t* acc_done = ds_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * p.R;
  const int t_hi = min(q0 + p.R, p.T) - 1;
  const bool selected = p.tile_blocks != nullptr;
  const long tile_slot = (static_cast<long>(b) * p.Hkv + h) * gridDim.x + qt;
  const int* blocks = selected ? p.tile_blocks + tile_slot * p.max_u : nullptr;
  const unsigned long long* masks = selected ? p.tile_masks + tile_slot * p.max_u : nullptr;
  int kb0 = 0, n_vis;
  if (selected) {
    n_vis = min(p.tile_counts[tile_slot], p.max_u);
  } else {
    long last = p.S - 1;
    if (p.causal) {
      long lim = static_cast<long>(t_hi) - p.kp_off;
      lim = lim < 0 ? -1 : lim / p.kp_stride;
      last = lim < last ? lim : last;
    }
    long first = 0;
    if (p.window > 0) {
      const long lo = static_cast<long>(q0) - p.window + 1 - p.kp_off;
      first = lo <= 0 ? 0 : (lo + p.kp_stride - 1) / p.kp_stride;
    }
    kb0 = static_cast<int>(first / 64);
    n_vis = last < first ? 0 : static_cast<int>(last / 64) + 1 - kb0;
  }

  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(q_full, 1);
    for (int i = 0; i < DQ_STAGES; ++i) { tc5::mbar_init(kv_full + i, 1); tc5::mbar_init(kv_empty + i, 1); }
    for (int i = 0; i < 2; ++i) { tc5::mbar_init(s_full + i, 1); tc5::mbar_init(s_empty + i, 256); }
    tc5::mbar_init(ds_full, 256);
    tc5::mbar_init(ds_empty, 1);
    tc5::mbar_init(acc_done, 1);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cDQ = 256;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_vis > 0) {
      tc5::mbar_expect_tx(q_full, 2 * QT);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        tc5::tma_load_5d(sQ + kb * 2 * HALF, &tm_q, q_full, kb * 64, 0, h, q0, b);
        tc5::tma_load_5d(sDO + kb * 2 * HALF, &tm_do, q_full, kb * 64, 0, h, q0, b);
      }
      bool ok = true;
      int issued = 0;
      int blk_n = selected ? blocks[0] : 0;
      for (int v = 0; v < n_vis; ++v) {
        const int st = v % DQ_STAGES;
        const int blk = blk_n;
        if (selected && v + 1 < n_vis) blk_n = blocks[v + 1];
        if (!tc5::mbar_wait(kv_empty + st, ((v / DQ_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY)) { ok = false; break; }
        int s0;
        if (!selected) s0 = (kb0 + v) * 64;
        else s0 = blk < 0 ? 0 : blk * 64;
        uint8_t* kd = sKV + st * 4 * HALF;
        tc5::mbar_expect_tx(kv_full + st, 4 * HALF);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tc5::tma_load_4d(kd + kb * HALF, &tm_k, kv_full + st, kb * 64, h, s0, b);
          tc5::tma_load_4d(kd + 2 * HALF + kb * HALF, &tm_v, kv_full + st, kb * 64, h, s0, b);
        }
        issued = v + 1;
      }
      if (!ok) {
        // let the copies already issued land before the CTA's shared memory is released
        for (int j = max(0, issued - DQ_STAGES); j < issued; ++j) {
          const long long t0 = clock64();
          for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
            if (tc5::mbar_try_wait(kv_full + (j % DQ_STAGES), (j / DQ_STAGES) & 1)) break;
            if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
          }
        }
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full, 0)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_vis > 0) {
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t id_q = tc5::make_idesc_bf16(128, D, 0, 1);
      // Every shared-memory descriptor is built once.  The address field (bits 0-13, address >> 4) of
      // a descriptor can be advanced by adding the byte offset >> 4, so the per-visit work of this
      // thread is one add per operand and the MMA itself: with 64-key MMAs of about 32 cycles the
      // issuing thread's instruction count, not the tensor pipe, sets the pace otherwise.
      uint64_t aQ[D / 16], aDO[D / 16], aDS[4];
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t a_off = (kk >> 2) * 2 * HALF + (kk & 3) * 32;
        aQ[kk] = tc5::desc_kmajor(tc5::smem_u32(sQ) + a_off);
        aDO[kk] = tc5::desc_kmajor(tc5::smem_u32(sDO) + a_off);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) aDS[kk] = tc5::desc_kmajor(tc5::smem_u32(sDS) + kk * 32);
      const uint64_t bK0 = tc5::desc_kmajor(tc5::smem_u32(sKV));             // stage 0, K, k-step 0
      const uint64_t bKmn0 = tc5::desc_mnmajor(tc5::smem_u32(sKV), HALF);    // same tile as an MN-major operand
      bool ok = tc5::mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL);
      for (int v = 0; v <= n_vis && ok; ++v) {
        if (v < n_vis) {
          const int st = v % DQ_STAGES, buf = v & 1;
          if (!tc5::mbar_wait(kv_full + st, (v / DQ_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          if (!tc5::mbar_wait(s_empty + buf, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint64_t bK = bK0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
          const uint64_t bV = bK + static_cast<uint64_t>((2 * HALF) >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ss(tmem + buf * 128, aQ[kk], bK + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s,
                        kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ss(tmem + buf * 128 + 64, aDO[kk], bV + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s,
                        kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + buf);
        }
        if (v >= 1) {
          const int u = v - 1, st = u % DQ_STAGES;
          if (!tc5::mbar_wait(ds_full, u & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint64_t bKmn = bKmn0 + static_cast<uint64_t>((st * 4 * HALF) >> 4);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)          // dQ += dS K  (64 keys per visit)
            tc5::mma_ss(tmem + cDQ, aDS[kk], bKmn + static_cast<uint64_t>((kk * 2048) >> 4), id_q, (u > 0 || kk > 0) ? 1u : 0u);
          tc5::mma_commit(kv_empty + st);
          tc5::mma_commit(ds_empty);
        }
      }
      if (ok) tc5::mma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int r = tid & 127, ch = tid >> 7;
    const int tok_local = r / p.G, g = r % p.G;
    const int t = q0 + tok_local;
    const bool row_ok = t < p.T;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const long rowi = (static_cast<long>(b) * p.T + (row_ok ? t : 0)) * p.Hq + h * p.G + g;
    const float Lrow = row_ok ? p.L[rowi] : 0.f;
    const float negL = Lrow == -INFINITY ? -INFINITY : -Lrow;     // a row that sees no key: -inf - inf, not -inf + inf
    const float drow = row_ok ? p.delta[rowi] : 0.f;
    const float nds = -drow * scale;
    const float sc = p.scale_log2;
    bool ok = true;
    // selected mode: the block id and token mask of visit v+1 are fetched during visit v, so the
    // global-memory latency is off the per-visit critical path
    int blk_n = (selected && n_vis > 0) ? blocks[0] : 0;
    unsigned long long msk_n = (selected && n_vis > 0) ? masks[0] : 0ull;
    for (int v = 0; v < n_vis; ++v) {
      const int buf = v & 1;
      int sb;
      bool row_sel = row_ok;
      if (!selected) sb = (kb0 + v) * 64 + ch * 32;
      else {
        const int blk = blk_n;
        const unsigned long long msk = msk_n;
        if (v + 1 < n_vis) { blk_n = blocks[v + 1]; msk_n = masks[v + 1]; }
        sb = blk < 0 ? -1 : blk * 64 + ch * 32;
        row_sel = row_ok && blk >= 0 && ((msk >> (tok_local & 63)) & 1ull);
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + buf, (v >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[32], dv[32], ds[16];
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + ch * 32, sv);
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + 64 + ch * 32, dv);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(s_empty + buf);
      if (!row_sel) {
#pragma unroll
        for (int i = 0; i < 16; ++i) ds[i] = 0u;
      } else {
        bool check = sb + 31 >= p.S;
        if (p.causal) check = check || ((sb + 31) * p.kp_stride + p.kp_off > t);
        if (p.window > 0) check = check || (sb * p.kp_stride + p.kp_off <= t - p.window);
        if (check) mask_scores<32>(p, sv, sb, t);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {                 // masked scores are -inf: their probability is 0
          const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sc, negL));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, negL));
          ds[i / 2] = tc5::pack_bf16(p0 * fmaf(__uint_as_float(dv[i]), scale, nds),
                                     p1 * fmaf(__uint_as_float(dv[i + 1]), scale, nds));
        }
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(ds_empty, (v & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY))) {
        ok = false;
        break;
      }
      {
        uint8_t* rd = sDS + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(rd + (((ch * 4 + j) ^ (r & 7)) << 4)) = make_uint4(ds[4 * j], ds[4 * j + 1], ds[4 * j + 2], ds[4 * j + 3]);
      }
      tc5::fence_proxy_async();
      tc5::mbar_arrive(ds_full);
    }
    // ---- dQ: thread (r, ch) stores D-half ch of row r
    const bool have = __all_sync(0xffffffffu, ok && n_vis > 0 &&
                                 tc5::mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL));
    if (have) tc5::fence_after_sync();
    bf16* dst = p.dQb + rowi * D + ch * 64;
#pragma unroll
    for (int q4 = 0; q4 < 2; ++q4) {
      uint32_t a[32];
      if (have) {
        tc5::tmem_ld_x32(tmem + lane_off + cDQ + ch * 64 + q4 * 32, a);
        tc5::tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) a[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o4;
          o4.x = tc5::pack_bf16(__uint_as_float(a[8 * i]), __uint_as_float(a[8 * i + 1]));
          o4.y = tc5::pack_bf16(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3]));
          o4.z = tc5::pack_bf16(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5]));
          o4.w = tc5::pack_bf16(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7]));
          reinterpret_cast<uint4*>(dst + q4 * 32)[i] = o4;
        }
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Backward for dK / dV, key-block stationary.  A CTA owns one 64-key block of one KV head and
// walks over "visits": query tiles of 128 rows (R tokens x G heads) that can see the block.
//   contiguous modes: the visits are the query tiles of an analytic range (causality, window),
//     split into chunks of `visits_per_cta` along grid.x;
//   selected mode: the visits come from the inverse selection map: for every (batch, KV head,
//     block) the ascending list of tokens that selected it, R tokens per visit, each token's
//     G query rows fetched by its own TMA box.
// dV^T (D x 64) += dO^T P and dK^T (D x 64) += Q^T dS stay in TMEM for the whole walk, so global
// memory sees one fp32 reduction per CTA instead of one per (query tile, key tile) pair.
// Roles: warps 0-7 softmax (thread (r, ch) = row r, 32 key columns), warp 8 TMA producer,
// warps 9-11 MMA issuers.  Q/dO are double-buffered in shared memory and S/dP in TMEM: while the
// softmax warps work on visit v the tensor pipe runs S/dP of visit v+1 and dV/dK of visit v-1.
// Needs D = 128 (the accumulators put D on the 128 TMEM lanes).
// --------------------------------------------------------------------------------------
struct KvWalk {
  int visits_per_cta;
  const int* tok_list;      // selected mode: tokens grouped by (b, h, block), ascending inside a group
  const int* list_start;    // [n_lists + 1]
  const int* item_start;    // [n_lists + 1] exclusive prefix of CTAs per list
  int n_lists, nS;
};

constexpr int KV_THREADS = 384;

__global__ void __launch_bounds__(KV_THREADS, 1)
attn_bwd_kv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_q1, const __grid_constant__ CUtensorMap tm_do1,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const AttnParams p, const KvWalk w, const float scale) {
  constexpr int D = 128;
  constexpr int QT = 4 * HALF;                   // one [128 rows][128] bf16 operand: two 64-column k-blocks
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                            // [2 k-blocks][64 keys][64]
  uint8_t* sV = sK + 2 * HALF;
  uint8_t* sQ = sV + 2 * HALF;                   // [2 buffers][QT]
  uint8_t* sDO = sQ + 2 * QT;
  uint8_t* sP = sDO + 2 * QT;                    // [128 rows][64 keys]
  uint8_t* sDS = sP + 2 * HALF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * HALF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                   // [2] TMA -> MMA
  uint64_t* q_empty = bars + 3;                  // [2] MMA -> TMA
  uint64_t* s_full = bars + 5;                   // [2] MMA -> softmax
  uint64_t* s_empty = bars + 7;                  // [2] softmax -> MMA
  uint64_t* p_full = bars + 9;                   // softmax -> MMA
  uint64_t* p_empty = bars + 10;                 // MMA -> softmax
  uint64_t* acc_done = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool selected = w.tok_list != nullptr;
  // ---- which block, which visits (uniform over the CTA; CTAs without work leave before any setup)
  int b, h, s0, v0, n_vis, lst0 = 0, cnt = 0;
  if (selected) {
    const int item = blockIdx.x;
    if (item >= w.item_start[w.n_lists]) return;
    int lo = 0, hi = w.n_lists;                  // largest l with item_start[l] <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (w.item_start[mid] <= item) lo = mid; else hi = mid;
    }
    const int l = lo;
    const int bh = l / w.nS;
    b = bh / p.Hkv; h = bh - b * p.Hkv;
    s0 = (l - bh * w.nS) * 64;
    lst0 = w.list_start[l];
    cnt = w.list_start[l + 1] - lst0;
    v0 = (item - w.item_start[l]) * w.visits_per_cta;
    n_vis = min(w.visits_per_cta, (cnt + p.R - 1) / p.R - v0);
  } else {
    const int bh = blockIdx.z;
    b = bh / p.Hkv; h = bh - b * p.Hkv;
    s0 = blockIdx.x * 64;                         // key block fastest: concurrent CTAs share a Q/dO range in L2
    const int s_hi = min(s0 + 63, p.S - 1);
    const int n_qt = (p.T + p.R - 1) / p.R;
    int qt_lo = 0, qt_hi = n_qt;
    if (p.causal) qt_lo = max(0, (s0 * p.kp_stride + p.kp_off) / p.R);
    if (p.window > 0) qt_hi = min(n_qt, (s_hi * p.kp_stride + p.kp_off + p.window - 1) / p.R + 1);
    if (p.window > 0) {                          // short ranges: chunks counted from the block's first tile
      v0 = qt_lo + blockIdx.y * w.visits_per_cta;
      n_vis = min(w.visits_per_cta, qt_hi - v0);
    } else {                                     // long ranges: absolute chunks, the same Q/dO range for every key block
      v0 = max(qt_lo, static_cast<int>(blockIdx.y) * w.visits_per_cta);
      n_vis = min(qt_hi, (static_cast<int>(blockIdx.y) + 1) * w.visits_per_cta) - v0;
    }
  }
  if (n_vis <= 0) return;

  if (tid == 0) {
    *abort_flag = 0;
    tc5::mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc5::mbar_init(q_full + i, 1);
      tc5::mbar_init(q_empty + i, 2);
      tc5::mbar_init(s_full + i, 1);
      tc5::mbar_init(s_empty + i, 256);
    }
    tc5::mbar_init(p_full, 256);
    tc5::mbar_init(p_empty, 2);
    tc5::mbar_init(acc_done, 2);
    tc5::fence_barrier_init();
  }
  if (warp == 9) { tc5::tmem_alloc(tmem_slot, 512); tc5::tmem_relinquish(); }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cDV = 256, cDK = 320;       // S/dP of buffer i at columns i*128 + {0, 64}

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    bool ok = true;
    if (lane == 0) {
      tc5::mbar_expect_tx(kv_full, 4 * HALF);
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        tc5::tma_load_4d(sK + kb * HALF, &tm_k, kv_full, kb * 64, h, s0, b);
        tc5::tma_load_4d(sV + kb * HALF, &tm_v, kv_full, kb * 64, h, s0, b);
      }
    }
    int issued = 0;
    for (int v = 0; v < n_vis; ++v) {
      const int buf = v & 1;
      if (lane == 0) {
        ok = tc5::mbar_wait(q_empty + buf, ((v >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY);
        if (ok) tc5::mbar_expect_tx(q_full + buf, 2 * QT);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      uint8_t* dq_ = sQ + buf * QT;
      uint8_t* dd_ = sDO + buf * QT;
      if (!selected) {
        if (lane == 0) {
          const int q0 = (v0 + v) * p.R;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            tc5::tma_load_5d(dq_ + kb * 2 * HALF, &tm_q, q_full + buf, kb * 64, 0, h, q0, b);
            tc5::tma_load_5d(dd_ + kb * 2 * HALF, &tm_do, q_full + buf, kb * 64, 0, h, q0, b);
          }
        }
      } else {
        for (int j = lane; j < p.R; j += 32) {
          const int li = (v0 + v) * p.R + j;
          const int tok = li < cnt ? __ldg(w.tok_list + lst0 + li) : 0;   // rows past the list read token 0 and are masked
          const int off = j * p.G * 128;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
            tc5::tma_load_5d(dq_ + kb * 2 * HALF + off, &tm_q1, q_full + buf, kb * 64, 0, h, tok, b);
            tc5::tma_load_5d(dd_ + kb * 2 * HALF + off, &tm_do1, q_full + buf, kb * 64, 0, h, tok, b);
          }
        }
      }
      __syncwarp();
      issued = v + 1;
    }
    if (!ok && lane == 0) {
      // let the copies already issued land before the CTA's shared memory is released
      for (int j = max(0, issued - 2); j < issued; ++j) {
        const long long t0 = clock64();
        for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
          if (tc5::mbar_try_wait(q_full + (j & 1), (j >> 1) & 1)) break;
          if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
        }
      }
      const long long t0 = clock64();
      for (uint32_t i = 0; i < tc5::kMaxPolls; ++i) {
        if (tc5::mbar_try_wait(kv_full, 0)) break;
        if ((i & 255u) == 255u && clock64() - t0 > tc5::kMaxWaitCycles) break;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer 1: S = Q K^T, dP = dO V^T
    // Three issuing warps, each converged with one elected lane issuing (see the forward kernel):
    // warp 9 issues S and dP, warp 10 dV^T += dO^T P, warp 11 dK^T += Q^T dS.  q_empty, p_empty and
    // acc_done count one commit of each of the last two.  (A thirteenth warp would put four warps on
    // one scheduler and cap every thread at 128 registers.)
    {
      const bool lead = tc5::elect_one();
      constexpr uint32_t id_s = tc5::make_idesc_bf16(128, 64, 0, 0);
      const uint64_t aQ0 = tc5::desc_kmajor(tc5::smem_u32(sQ)), aDO0 = tc5::desc_kmajor(tc5::smem_u32(sDO));
      const uint64_t bK0 = tc5::desc_kmajor(tc5::smem_u32(sK)), bV0 = tc5::desc_kmajor(tc5::smem_u32(sV));
      bool ok = __all_sync(0xffffffffu, tc5::mbar_wait(kv_full, 0, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL));
      for (int v = 0; v < n_vis && ok; ++v) {
        const int buf = v & 1;
        const uint32_t ph = (v >> 1) & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(q_full + buf, ph, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL) &&
                                     tc5::mbar_wait(s_empty + buf, ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t aQ = aQ0 + static_cast<uint64_t>((buf * QT) >> 4), aDO = aDO0 + static_cast<uint64_t>((buf * QT) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ss(tmem + buf * 128, aQ + static_cast<uint64_t>(((kk >> 2) * 2 * HALF + (kk & 3) * 32) >> 4),
                        bK0 + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s, kk > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            tc5::mma_ss(tmem + buf * 128 + 64, aDO + static_cast<uint64_t>(((kk >> 2) * 2 * HALF + (kk & 3) * 32) >> 4),
                        bV0 + static_cast<uint64_t>(((kk >> 2) * HALF + (kk & 3) * 32) >> 4), id_s, kk > 0 ? 1u : 0u);
          tc5::mma_commit(s_full + buf);
        }
        __syncwarp();
      }
    }
  } else if (warp == 10 || warp == 11) {
    // ------------------------------------------------------------------ MMA issuers 2 and 3: dV^T += dO^T P, dK^T += Q^T dS
    {
      const bool lead = tc5::elect_one();
      const bool is_dk = warp == 11;
      constexpr uint32_t id_t = tc5::make_idesc_bf16(128, 64, 1, 1);
      const uint64_t a0 = tc5::desc_mnmajor(tc5::smem_u32(is_dk ? sQ : sDO), 2 * HALF);
      const uint64_t b0 = tc5::desc_mnmajor(tc5::smem_u32(is_dk ? sDS : sP), 2 * HALF);
      const uint32_t dcol = is_dk ? cDK : cDV;
      bool ok = true;
      for (int u = 0; u < n_vis; ++u) {
        const int buf = u & 1;
        ok = __all_sync(0xffffffffu, tc5::mbar_wait(p_full, u & 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_FULL));
        if (!ok) break;
        tc5::fence_after_sync();
        const uint64_t aA = a0 + static_cast<uint64_t>((buf * QT) >> 4);
        if (lead) {
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk)
            tc5::mma_ss(tmem + dcol, aA + static_cast<uint64_t>((kk * 2048) >> 4), b0 + static_cast<uint64_t>((kk * 2048) >> 4), id_t,
                        (u > 0 || kk > 0) ? 1u : 0u);
          // S and dP of this visit completed before P and dS could be written, so the commits of these
          // two warps alone release the Q / dO buffer and the P / dS tiles
          tc5::mma_commit(q_empty + buf);
          tc5::mma_commit(p_empty);
        }
        __syncwarp();
      }
      if (ok && lead) tc5::mma_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int r = tid & 127, ch = tid >> 7;
    const int tok_local = r / p.G, g = r % p.G;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const float sc = p.scale_log2;
    const int sb = s0 + ch * 32;                   // this thread's first key
    bool ok = true;
    // The row's token (selected mode: from the inverse list) and its L / delta are fetched one and
    // two visits ahead, so the two dependent global loads are off the per-visit critical path.
    auto token_of = [&](int v) -> int {
      if (v >= n_vis) return -1;
      if (selected) {
        const int li = (v0 + v) * p.R + tok_local;
        return li < cnt ? w.tok_list[lst0 + li] : -1;
      }
      const int tt = (v0 + v) * p.R + tok_local;
      return tt < p.T ? tt : -1;
    };
    int t_cur = token_of(0), t_nxt = token_of(1);
    float L_cur = 0.f, d_cur = 0.f;
    if (t_cur >= 0) {
      const long rowi = (static_cast<long>(b) * p.T + t_cur) * p.Hq + h * p.G + g;
      L_cur = p.L[rowi];
      d_cur = p.delta[rowi];
    }
    for (int v = 0; v < n_vis; ++v) {
      const int buf = v & 1;
      const int t = t_cur;
      const float Lrow = L_cur, nds = -d_cur * scale;
      const float negL = Lrow == -INFINITY ? -INFINITY : -Lrow;   // a row that sees no key: -inf - inf, not -inf + inf
      {
        float Ln = 0.f, dn = 0.f;
        if (t_nxt >= 0) {
          const long rowi = (static_cast<long>(b) * p.T + t_nxt) * p.Hq + h * p.G + g;
          Ln = p.L[rowi];
          dn = p.delta[rowi];
        }
        t_cur = t_nxt; L_cur = Ln; d_cur = dn;
        t_nxt = token_of(v + 2);
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(s_full + buf, (v >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc5::fence_after_sync();
      uint32_t sv[32], dv[32], pp[16], ds[16];
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + ch * 32, sv);
      tc5::tmem_ld_x32(tmem + lane_off + buf * 128 + 64 + ch * 32, dv);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      tc5::mbar_arrive(s_empty + buf);
      if (t < 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) { pp[i] = 0u; ds[i] = 0u; }
      } else {
        bool check = sb + 31 >= p.S;
        if (p.causal) check = check || ((sb + 31) * p.kp_stride + p.kp_off > t);
        if (p.window > 0) check = check || (sb * p.kp_stride + p.kp_off <= t - p.window);
        if (check) mask_scores<32>(p, sv, sb, t);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {                 // masked scores are -inf: their probability is 0
          const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sc, negL));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, negL));
          pp[i / 2] = tc5::pack_bf16(p0, p1);
          ds[i / 2] = tc5::pack_bf16(p0 * fmaf(__uint_as_float(dv[i]), scale, nds),
                                     p1 * fmaf(__uint_as_float(dv[i + 1]), scale, nds));
        }
      }
      if (!__all_sync(0xffffffffu, tc5::mbar_wait(p_empty, (v & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_SMEM_EMPTY))) {
        ok = false;
        break;
      }
      {
        uint8_t* rp = sP + r * 128;
        uint8_t* rd = sDS + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = ((ch * 4 + j) ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(rp + c) = make_uint4(pp[4 * j], pp[4 * j + 1], pp[4 * j + 2], pp[4 * j + 3]);
          *reinterpret_cast<uint4*>(rd + c) = make_uint4(ds[4 * j], ds[4 * j + 1], ds[4 * j + 2], ds[4 * j + 3]);
        }
      }
      tc5::fence_proxy_async();
      tc5::mbar_arrive(p_full);
    }
    // ---- accumulators -> global: lane = d, columns = keys; one fp32 reduction per element
    if (__all_sync(0xffffffffu, ok && tc5::mbar_wait(acc_done, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL))) {
      tc5::fence_after_sync();
      const int d = (warp & 3) * 32 + lane;
      float* dst = (warp < 4 ? p.dV : p.dK) + ((static_cast<long>(b) * p.S + s0) * p.Hkv + h) * D + d;
      const uint32_t col = warp < 4 ? cDV : cDK;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t a[32];
        tc5::tmem_ld_x32(tmem + lane_off + col + c0, a);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (s0 + c0 + i < p.S) atomicAdd(dst + static_cast<long>(c0 + i) * p.Hkv * D, __uint_as_float(a[i]));
      }
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 9) { tc5::fence_after_sync(); tc5::tmem_dealloc(tmem, 512); }
}

// --------------------------------------------------------------------------------------
// Top-n block selection.  One warp per (batch, KV head, token) row of the importance tensor:
// block 0, the token's own block and the one before it are always taken; the remaining slots go
// to the causal blocks of highest importance (ties: lower block index first); slots that cannot
// be filled hold -1.  Lane l keeps blocks l, l + 32, ... in registers; every round is a
// lane-local scan plus a five-step warp arg-max.
// --------------------------------------------------------------------------------------
template <int PER_LANE>
__global__ void __launch_bounds__(256) nsa_select_kernel(const float* __restrict__ imp, int* __restrict__ idx, long rows,
                                                         int T, int nS, int sel_block, int top_n) {
  const int lane = threadIdx.x & 31;
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int t = static_cast<int>(row % T);
  const int own = min(t / sel_block, nS - 1);
  const float* src = imp + row * nS;
  float v[PER_LANE];
#pragma unroll
  for (int k = 0; k < PER_LANE; ++k) {
    const int j = lane + 32 * k;
    v[k] = (j <= own) ? src[j] : -INFINITY;
    if (j == 0 || j == own || j == own - 1) v[k] = -INFINITY;       // forced blocks are emitted below
  }
  int* dst = idx + row * top_n;
  int n_out = 0;
  if (lane == 0) {
    dst[n_out] = 0;
    if (own > 0 && n_out + 1 < top_n) dst[n_out + 1] = own;
    if (own > 1 && n_out + 2 < top_n) dst[n_out + 2] = own - 1;
  }
  n_out = min(top_n, 1 + (own > 0 ? 1 : 0) + (own > 1 ? 1 : 0));
  const int candidates = max(0, own + 1 - n_out);                     // causal blocks that are not forced
  const int rounds = min(top_n - n_out, candidates);
  for (int rd = 0; rd < rounds; ++rd) {
    float best = -INFINITY;
    int bk = -1;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k)
      if (v[k] > best) {                                              // strict: the lowest index wins a tie
        best = v[k];
        bk = k;
      }
    int bj = bk < 0 ? 0x7fffffff : lane + 32 * bk;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
      if (ob > best || (ob == best && oj < bj)) { best = ob; bj = oj; }
    }
    if (bj == 0x7fffffff) break;                                      // only -inf importances left (cannot happen for finite input)
    if ((bj & 31) == lane) {
#pragma unroll
      for (int k = 0; k < PER_LANE; ++k)
        if (k == (bj >> 5)) v[k] = -INFINITY;
    }
    if (lane == 0) dst[n_out] = bj;
    ++n_out;
  }
  for (int i = n_out + lane; i < top_n; i += 32) dst[i] = -1;
}

// --------------------------------------------------------------------------------------
// Helper kernels
// --------------------------------------------------------------------------------------
// delta[row] = sum_d dO[row, d] * O[row, d]; one warp per row.
__global__ void __launch_bounds__(256) attn_delta_kernel(const bf16* __restrict__ O, const bf16* __restrict__ dO,
                                                         float* __restrict__ delta, long rows, int D) {
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(O + row * D + c));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dO + row * D + c));
    s += a.x * d.x + a.y * d.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[row] = s;
}

// Union of the selection blocks chosen by the R tokens of each query tile.
// --------------------------------------------------------------------------------------
// Inverse of the selection map: for every (batch, kv head, block) the ascending list of tokens that
// selected the block (what the key-stationary dK/dV pass walks).  Counting, scanning and filling,
// with no sort and no atomics on global memory, so the lists are the same on every run:
//   1. one warp per (b*h, chunk of INV_CHUNK tokens) builds the chunk's histogram over blocks;
//   2. per list, an exclusive scan of the histograms along the chunks gives each chunk's offset
//      inside the list, and the total gives the list's length;
//   3. one thread block scans the lengths into list starts (and the CTA counts per list);
//   4. the warps of step 1 walk their tokens again in the same order and write them.
// An entry is dropped if it is negative, out of range or repeats an earlier entry of the same token.
// --------------------------------------------------------------------------------------
constexpr int INV_CHUNK = 256;

// mode 0: hist[(bh * chunks + chunk) * nS + blk] = entries of the chunk; mode 1: fill tok_list.
// The warp takes the chunk's tokens one after the other, lane j looking at entry j of the token's
// list (n <= 32): a token's valid entries name distinct blocks, so the lanes touch distinct counters,
// and tokens reach every list in ascending order.
__global__ void __launch_bounds__(32) nsa_inverse_walk_kernel(const int* __restrict__ idx, int* __restrict__ hist,
                                                              const int* __restrict__ chunk_off,
                                                              const int* __restrict__ list_start, int* __restrict__ tok_list,
                                                              int T, int n, int nS, int chunks, int mode) {
  extern __shared__ int bins[];                   // nS running counts of this chunk
  const int chunk = blockIdx.x, lane = threadIdx.x;
  const long bh = blockIdx.y;
  for (int i = lane; i < nS; i += 32) bins[i] = 0;
  __syncwarp();
  const long slot = (bh * chunks + chunk) * nS;
  const int t_end = min(T, (chunk + 1) * INV_CHUNK);
  int v_next = (lane < n && chunk * INV_CHUNK < t_end) ? idx[(bh * T + chunk * INV_CHUNK) * n + lane] : -1;
  for (int t = chunk * INV_CHUNK; t < t_end; ++t) {
    const int v = v_next;
    if (t + 1 < t_end && lane < n) v_next = idx[(bh * T + t + 1) * n + lane];      // next token's entry, ahead of use
    const bool in_range = lane < n && v >= 0 && v < nS;
    const unsigned same = __match_any_sync(0xffffffffu, in_range ? v : -1 - lane);
    const bool first = (same & ((1u << lane) - 1u)) == 0u;                          // not a repeat of an earlier entry
    if (in_range && first) {
      const int before = bins[v];
      if (mode == 1) tok_list[list_start[bh * nS + v] + chunk_off[slot + v] + before] = t;
      bins[v] = before + 1;
    }
    __syncwarp();
  }
  if (mode == 0)
    for (int i = lane; i < nS; i += 32) hist[slot + i] = bins[i];
}

// one thread per list: offsets of the chunks inside the list (in place over hist) and the length
__global__ void __launch_bounds__(256) nsa_inverse_offsets_kernel(int* __restrict__ hist, int* __restrict__ count, long lists,
                                                                 int nS, int chunks) {
  const long l = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (l >= lists) return;
  const long bh = l / nS;
  const int blk = static_cast<int>(l - bh * nS);
  int run = 0;
  for (int c = 0; c < chunks; ++c) {
    int* p = hist + (bh * chunks + c) * nS + blk;
    const int v = *p;
    *p = run;
    run += v;
  }
  count[l] = run;
}

// single CTA: list_start[l] = sum of count[< l]; item_start[l] = sum of ceil(ceil(count / R) / vpc)
__global__ void __launch_bounds__(1024) nsa_inverse_scan_kernel(const int* __restrict__ count, int* __restrict__ list_start,
                                                               int* __restrict__ item_start, long lists, int R, int vpc) {
  __shared__ int sa[1024], sb[1024];
  __shared__ int base_a, base_b;
  if (threadIdx.x == 0) { base_a = 0; base_b = 0; }
  __syncthreads();
  for (long l0 = 0; l0 < lists; l0 += 1024) {
    const long l = l0 + threadIdx.x;
    const int c = l < lists ? count[l] : 0;
    const int it = ((c + R - 1) / R + vpc - 1) / vpc;
    sa[threadIdx.x] = c;
    sb[threadIdx.x] = it;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {           // inclusive scan, Hillis-Steele
      const int va = threadIdx.x >= o ? sa[threadIdx.x - o] : 0;
      const int vb = threadIdx.x >= o ? sb[threadIdx.x - o] : 0;
      __syncthreads();
      sa[threadIdx.x] += va;
      sb[threadIdx.x] += vb;
      __syncthreads();
    }
    if (l < lists) {
      list_start[l] = base_a + sa[threadIdx.x] - c;
      item_start[l] = base_b + sb[threadIdx.x] - it;
    }
    __syncthreads();
    if (threadIdx.x == 1023) { base_a += sa[1023]; base_b += sb[1023]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { list_start[lists] = base_a; item_start[lists] = base_b; }
}

// idx: [B, Hkv, T, top_n] int32 block ids (-1 = none).  Outputs per (b, h, tile): ascending
// block list, per-entry token bit masks, and the entry count.  One CTA per tile.
__global__ void __launch_bounds__(128) nsa_union_kernel(const int* __restrict__ idx, int* __restrict__ tile_blocks,
                                                        unsigned long long* __restrict__ tile_masks,
                                                        int* __restrict__ tile_counts, int T, int R, int top_n,
                                                        int nS, int max_u, KernelStatus* status) {
  extern __shared__ unsigned int sh[];          // bitmap words, then per-word prefix counts
  const int words = (nS + 31) / 32;
  unsigned int* bitmap = sh;
  unsigned int* prefix = sh + words;
  const int qt = blockIdx.x;
  const long bh = blockIdx.y;                   // b * Hkv + h
  const long slot = bh * gridDim.x + qt;
  int* ob = tile_blocks + slot * max_u;
  unsigned long long* om = tile_masks + slot * max_u;
  for (int i = threadIdx.x; i < words; i += blockDim.x) bitmap[i] = 0u;
  for (int i = threadIdx.x; i < max_u; i += blockDim.x) { ob[i] = -1; om[i] = 0ull; }
  __syncthreads();
  const int q0 = qt * R;
  const int n_cand = R * top_n;
  for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
    const int tl = i / top_n, t = q0 + tl;
    if (t >= T) continue;
    const int blk = idx[(bh * T + t) * top_n + (i - tl * top_n)];
    NSA_CHECK_INDEX(blk >= -1 && blk < nS && blk * 64 <= t, status, blk);     // in range and not after the query
    if (blk >= 0 && blk < nS) atomicOr(&bitmap[blk >> 5], 1u << (blk & 31));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int run = 0;
    for (int wd = 0; wd < words; ++wd) { prefix[wd] = run; run += __popc(bitmap[wd]); }
    tile_counts[slot] = static_cast<int>(run < static_cast<unsigned>(max_u) ? run : max_u);
  }
  __syncthreads();
  for (int wd = threadIdx.x; wd < words; wd += blockDim.x) {
    unsigned int bits = bitmap[wd];
    unsigned int pos = prefix[wd];
    while (bits) {
      const int bpos = __ffs(bits) - 1;
      bits &= bits - 1;
      if (pos < static_cast<unsigned>(max_u)) ob[pos] = wd * 32 + bpos;
      ++pos;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_cand; i += blockDim.x) {
    const int tl = i / top_n, t = q0 + tl;
    if (t >= T) continue;
    const int blk = idx[(bh * T + t) * top_n + (i - tl * top_n)];
    if (blk < 0 || blk >= nS) continue;
    const unsigned int below = bitmap[blk >> 5] & ((1u << (blk & 31)) - 1u);
    const unsigned int pos = prefix[blk >> 5] + __popc(below);
    if (pos < static_cast<unsigned>(max_u)) atomicOr(&om[pos], 1ull << tl);
  }
}

// box_tokens 0: a whole query tile (128 / G tokens); otherwise that many tokens per box
int make_q_map(CUtensorMap* m, const void* base, int B, int T, int Hq, int Hkv, int D, int box_tokens = 0) {
  const int G = Hq / Hkv, R = box_tokens > 0 ? box_tokens : BM / G;
  uint64_t dims[5] = {(uint64_t)D, (uint64_t)G, (uint64_t)Hkv, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {(uint64_t)D * 2, (uint64_t)G * D * 2, (uint64_t)Hq * D * 2, (uint64_t)T * Hq * D * 2};
  uint32_t box[5] = {64, (uint32_t)G, 1, (uint32_t)R, 1};
  return nsa::make_tmap_bf16(m, base, 5, dims, strides, box, 1);
}
int make_kv_map(CUtensorMap* m, const void* base, int B, int S, int Hkv, int D) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)S * Hkv * D * 2};
  uint32_t box[4] = {64, 1, 64, 1};
  return nsa::make_tmap_bf16(m, base, 4, dims, strides, box, 1);
}

int check_shape(int Hq, int Hkv, int D, const int* tile_blocks) {
  if (D != 64 && D != 128) return nsa::fail(NSA_ERR_SHAPE, "attention: head_dim must be 64 or 128");
  if (Hkv <= 0 || Hq % Hkv) return nsa::fail(NSA_ERR_SHAPE, "attention: query heads must be a multiple of KV heads");
  const int G = Hq / Hkv;
  if (G > 128 || (G & (G - 1))) return nsa::fail(NSA_ERR_SHAPE, "attention: GQA group must be a power of two <= 128");
  if (tile_blocks && BM / G > 64) return nsa::fail(NSA_ERR_SHAPE, "selected attention needs a GQA group of at least 2");
  return 0;
}

template <typename K>
int set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "attention: shared memory attribute");
}

void fill_params(AttnParams& p, int B, int T, int S, int Hq, int Hkv, int D, float scale, int causal, int window,
                 int kp_stride, int kp_off, const int* tb, const unsigned long long* tmk, const int* tc, int max_u) {
  p = AttnParams{};
  p.B = B; p.T = T; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.R = BM / p.G; p.D = D;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal; p.window = window; p.kp_stride = kp_stride; p.kp_off = kp_off;
  p.tile_blocks = tb; p.tile_masks = tmk; p.tile_counts = tc; p.max_u = max_u;
  p.status = nsa::status_ptr();
}
}  // namespace

extern "C" int nsa_attn_fwd(const void* q, const void* k, const void* v, void* o, float* L, int B, int T, int S,
                            int Hq, int Hkv, int D, float scale, int causal, int window, int kp_stride, int kp_off,
                            const int* tile_blocks, const unsigned long long* tile_masks, const int* tile_counts,
                            int max_u, cudaStream_t st) {
  int rc = check_shape(Hq, Hkv, D, tile_blocks);
  if (rc) return rc;
  CUtensorMap tq, tk, tv;
  if ((rc = make_q_map(&tq, q, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tk, k, B, S, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tv, v, B, S, Hkv, D))) return rc;
  AttnParams p;
  fill_params(p, B, T, S, Hq, Hkv, D, scale, causal, window, kp_stride, kp_off, tile_blocks, tile_masks, tile_counts, max_u);
  p.O = (bf16*)o; p.L = L;
  const dim3 grid((T + p.R - 1) / p.R, Hkv, B);
  const int smem = (D / 64) * 2 * HALF * 5 + 4 * HALF + 1024 + 2048;
  static const bool legacy = [] { const char* e = getenv("NSA_B200_ATTN_FWD"); return e && !strcmp(e, "legacy"); }();
  static const bool smem_operands = [] { const char* e = getenv("NSA_B200_ATTN_FWD"); return e && !strcmp(e, "smem"); }();
  if (D == 128 && !legacy && !smem_operands) {
    const int smem_ts = (4 + 4 * FWT_STAGES) * HALF + 1024 + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_ts_kernel, smem_ts))) return rc; cfg = true; }
    attn_fwd_ts_kernel<<<grid, 352, smem_ts, st>>>(tq, tk, tv, p);
  } else if (D == 128 && !legacy) {
    const int smem_ws = (4 + 4 * FW_STAGES + 4) * HALF + 1024 + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_ws_kernel, smem_ws))) return rc; cfg = true; }
    attn_fwd_ws_kernel<<<grid, 320, smem_ws, st>>>(tq, tk, tv, p);
  } else if (D == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_kernel<128, 0>, smem))) return rc; cfg = true; }
    attn_fwd_kernel<128, 0><<<grid, 256, smem, st>>>(tq, tk, tv, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_kernel<64, 0>, smem))) return rc; cfg = true; }
    attn_fwd_kernel<64, 0><<<grid, 256, smem, st>>>(tq, tk, tv, p);
  }
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_attn_fwd launch");
}

// Block importance for top-n selection: imp[b,h,t,j] (pre-zeroed) += sum over the G heads of the
// compressed-branch probabilities, binned into selection blocks of 4 strides; compressed blocks
// span 2 strides.  L_in is the compressed branch's L from nsa_attn_fwd.
extern "C" int nsa_attn_importance(const void* q, const void* k_cmp, const float* L_in, float* imp, int B, int T, int S,
                                   int Hq, int Hkv, int D, float scale, int kp_stride, int kp_off, int nS,
                                   cudaStream_t st) {
  int rc = check_shape(Hq, Hkv, D, nullptr);
  if (rc) return rc;
  if (Hq / Hkv > 32) return nsa::fail(NSA_ERR_SHAPE, "importance: GQA group above 32 is not supported");
  if (kp_off + 1 != 2 * kp_stride) return nsa::fail(NSA_ERR_SHAPE, "importance: compressed block must span two strides");
  CUtensorMap tq, tk;
  if ((rc = make_q_map(&tq, q, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tk, k_cmp, B, S, Hkv, D))) return rc;
  AttnParams p;
  fill_params(p, B, T, S, Hq, Hkv, D, scale, 1, 0, kp_stride, kp_off, nullptr, nullptr, nullptr, 0);
  p.L_in = L_in; p.imp = imp; p.nS = nS; p.cells_per_block = 4;
  const dim3 grid((T + p.R - 1) / p.R, Hkv, B);
  const int smem = (D / 64) * 2 * HALF * 5 + 4 * HALF + 1024 + 2048;
  static const bool legacy = [] { const char* e = getenv("NSA_B200_ATTN_IMP"); return e && !strcmp(e, "legacy"); }();
  if (D == 128 && !legacy && 128 % (Hq / Hkv) == 0) {
    const int smem_ts = (4 + 2 * IMP_STAGES) * HALF + 1024 + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_importance_ts_kernel, smem_ts))) return rc; cfg = true; }
    attn_importance_ts_kernel<<<grid, 320, smem_ts, st>>>(tq, tk, tk, p);
  } else if (D == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_kernel<128, 1>, smem))) return rc; cfg = true; }
    attn_fwd_kernel<128, 1><<<grid, 256, smem, st>>>(tq, tk, tk, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_fwd_kernel<64, 1>, smem))) return rc; cfg = true; }
    attn_fwd_kernel<64, 1><<<grid, 256, smem, st>>>(tq, tk, tk, p);
  }
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_attn_importance launch");
}

// delta: scratch [B*T*Hq] fp32 (written here).  dK, dV: fp32 [B,S,Hkv,D], zeroed by the caller.
extern "C" int nsa_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* L,
                            float* delta, void* dq, float* dk, float* dv, int B, int T, int S, int Hq, int Hkv, int D,
                            float scale, int causal, int window, int kp_stride, int kp_off, const int* tile_blocks,
                            const unsigned long long* tile_masks, const int* tile_counts, int max_u, cudaStream_t st) {
  int rc = check_shape(Hq, Hkv, D, tile_blocks);
  if (rc) return rc;
  CUtensorMap tq, tdo, tk, tv;
  if ((rc = make_q_map(&tq, q, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_q_map(&tdo, d_o, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tk, k, B, S, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tv, v, B, S, Hkv, D))) return rc;
  const long rows = static_cast<long>(B) * T * Hq;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)o, (const bf16*)d_o, delta, rows, D);
  AttnParams p;
  fill_params(p, B, T, S, Hq, Hkv, D, scale, causal, window, kp_stride, kp_off, tile_blocks, tile_masks, tile_counts, max_u);
  p.L = const_cast<float*>(L); p.delta = delta; p.dQb = (bf16*)dq; p.dK = dk; p.dV = dv;
  const dim3 grid((T + p.R - 1) / p.R, Hkv, B);
  const int smem = (D / 64) * 2 * HALF * 4 + 8 * HALF + 1024 + 256;
  if (D == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_bwd_kernel<128>, smem))) return rc; cfg = true; }
    attn_bwd_kernel<128><<<grid, 256, smem, st>>>(tq, tdo, tk, tv, p, scale);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_bwd_kernel<64>, smem))) return rc; cfg = true; }
    attn_bwd_kernel<64><<<grid, 256, smem, st>>>(tq, tdo, tk, tv, p, scale);
  }
  nsa::count_launch(2);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_attn_bwd launch");
}

// Backward in two kernels without per-tile global reductions: dQ from the query-tile-outer
// kernel (its dK / dV part switched off) and dK / dV from the key-block-stationary kernel.
// Selected mode additionally takes the inverse selection map: tok_list (tokens grouped by
// (b, h, block), ascending), list_start / item_start ([B*Hkv*nS + 1] exclusive prefixes of list
// lengths and of CTAs per list, a CTA covering visits_per_cta * (128 / G) tokens) and
// item_bound >= item_start[last].  head_dim 128 only; selected mode needs G >= 8.
extern "C" int nsa_attn_bwd_split(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                  const float* L, float* delta, void* dq, float* dk, float* dv, int B, int T, int S,
                                  int Hq, int Hkv, int D, float scale, int causal, int window, int kp_stride, int kp_off,
                                  const int* tile_blocks, const unsigned long long* tile_masks, const int* tile_counts,
                                  int max_u, const int* tok_list, const int* list_start, const int* item_start, int nS,
                                  int item_bound, int visits_per_cta, cudaStream_t st) {
  int rc = check_shape(Hq, Hkv, D, tile_blocks);
  if (rc) return rc;
  const int G = Hq / Hkv;
  if (D != 128) return nsa::fail(NSA_ERR_SHAPE, "attn_bwd_split: head_dim must be 128");
  if (tile_blocks && (G < 8 || tok_list == nullptr))
    return nsa::fail(NSA_ERR_SHAPE, "attn_bwd_split: selected mode needs a GQA group of at least 8 and the inverse map");
  if (visits_per_cta <= 0) return nsa::fail(NSA_ERR_SHAPE, "attn_bwd_split: visits_per_cta must be positive");
  CUtensorMap tq, tdo, tq1, tdo1, tk, tv;
  if ((rc = make_q_map(&tq, q, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_q_map(&tdo, d_o, B, T, Hq, Hkv, D))) return rc;
  if ((rc = make_q_map(&tq1, q, B, T, Hq, Hkv, D, 1))) return rc;
  if ((rc = make_q_map(&tdo1, d_o, B, T, Hq, Hkv, D, 1))) return rc;
  if ((rc = make_kv_map(&tk, k, B, S, Hkv, D))) return rc;
  if ((rc = make_kv_map(&tv, v, B, S, Hkv, D))) return rc;
  const long rows = static_cast<long>(B) * T * Hq;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)o, (const bf16*)d_o, delta, rows, D);
  AttnParams p;
  fill_params(p, B, T, S, Hq, Hkv, D, scale, causal, window, kp_stride, kp_off, tile_blocks, tile_masks, tile_counts, max_u);
  p.L = const_cast<float*>(L); p.delta = delta; p.dQb = (bf16*)dq; p.dK = nullptr; p.dV = nullptr;
  {
    const dim3 grid((T + p.R - 1) / p.R, Hkv, B);
    static const bool smem_operands = [] { const char* e = getenv("NSA_B200_ATTN_DQ"); return e && !strcmp(e, "smem"); }();
    if (!smem_operands) {
      const int smem = (8 + 4 * DQT_STAGES) * HALF + 1024 + 256;
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(attn_bwd_dq_ts_kernel, smem))) return rc; cfg = true; }
      attn_bwd_dq_ts_kernel<<<grid, 384, smem, st>>>(tq, tdo, tk, tv, p, scale);
    } else {
      const int smem = (8 + 4 * DQ_STAGES + 2) * HALF + 1024 + 256;
      static bool cfg = false;
      if (!cfg) { if ((rc = set_smem(attn_bwd_dq_kernel, smem))) return rc; cfg = true; }
      attn_bwd_dq_kernel<<<grid, 320, smem, st>>>(tq, tdo, tk, tv, p, scale);
    }
  }
  p.dK = dk; p.dV = dv;
  KvWalk w{};
  w.visits_per_cta = visits_per_cta;
  dim3 grid;
  if (tile_blocks) {
    w.tok_list = tok_list; w.list_start = list_start; w.item_start = item_start; w.n_lists = B * Hkv * nS; w.nS = nS;
    if (item_bound <= 0) return nsa::fail(NSA_ERR_SHAPE, "attn_bwd_split: item_bound must be positive");
    grid = dim3(item_bound, 1, 1);
  } else {
    const int n_qt = (T + p.R - 1) / p.R;
    int max_vis = n_qt;
    if (window > 0) max_vis = std::min(n_qt, (63 * kp_stride + window - 1) / p.R + 2);
    grid = dim3((S + 63) / 64, (max_vis + visits_per_cta - 1) / visits_per_cta, B * Hkv);
  }
  {
    const int smem = 24 * HALF + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if ((rc = set_smem(attn_bwd_kv_kernel, smem))) return rc; cfg = true; }
    attn_bwd_kv_kernel<<<grid, KV_THREADS, smem, st>>>(tq, tdo, tq1, tdo1, tk, tv, p, w, scale);
  }
  nsa::count_launch(3);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_attn_bwd_split launch");
}

// imp [B, Hkv, T, nS] fp32 -> idx [B, Hkv, T, top_n] int32 (see nsa_select_kernel).  nS <= 2048.
extern "C" int nsa_select_blocks(const float* imp, int* idx, long rows, int T, int nS, int sel_block, int top_n,
                                 cudaStream_t st) {
  if (nS <= 0 || nS > 2048 || top_n <= 0 || sel_block <= 0) return nsa::fail(NSA_ERR_SHAPE, "select_blocks: nS must be in 1..2048");
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  if (nS <= 1024) nsa_select_kernel<32><<<grid, 256, 0, st>>>(imp, idx, rows, T, nS, sel_block, top_n);
  else nsa_select_kernel<64><<<grid, 256, 0, st>>>(imp, idx, rows, T, nS, sel_block, top_n);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_select_blocks launch");
}

// idx [B, Hkv, T, top_n] int32 -> per query tile (R = 128 / G tokens): block list, token masks, count.
extern "C" int nsa_union_blocks(const int* idx, int* tile_blocks, unsigned long long* tile_masks, int* tile_counts,
                                int B, int T, int Hkv, int G, int top_n, int nS, int max_u, cudaStream_t st) {
  const int R = BM / G;
  if (R > 64) return nsa::fail(NSA_ERR_SHAPE, "union: more than 64 tokens per tile");
  const int words = (nS + 31) / 32;
  const dim3 grid((T + R - 1) / R, B * Hkv);
  nsa_union_kernel<<<grid, 128, words * 8, st>>>(idx, tile_blocks, tile_masks, tile_counts, T, R, top_n, nS, max_u, nsa::status_ptr());
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_union_blocks launch");
}

// Inverse selection map (see nsa_inverse_walk_kernel).  idx: [B*Hkv, T, n] int32.  Outputs: tok_list
// (capacity B*Hkv*T*n), list_start and item_start (lists + 1 entries, lists = B*Hkv*nS).  Scratch:
// hist with B*Hkv*chunks*nS ints (chunks = ceil(T / 256)) and count with `lists` ints.
extern "C" int nsa_inverse_blocks(const int* idx, int* tok_list, int* list_start, int* item_start, int* hist, int* count,
                                  int BH, int T, int n, int nS, int R, int visits_per_cta, cudaStream_t st) {
  if (BH <= 0 || T <= 0 || n <= 0 || nS <= 0 || R <= 0 || visits_per_cta <= 0)
    return nsa::fail(NSA_ERR_SHAPE, "nsa_inverse_blocks: empty problem");
  if (nS * 4 > 48 * 1024 || n > 32) return nsa::fail(NSA_ERR_SHAPE, "nsa_inverse_blocks: at most 12288 selection blocks and 32 entries per token");
  const int chunks = (T + INV_CHUNK - 1) / INV_CHUNK;
  const long lists = static_cast<long>(BH) * nS;
  const dim3 grid(chunks, BH);
  nsa_inverse_walk_kernel<<<grid, 32, nS * 4, st>>>(idx, hist, nullptr, nullptr, nullptr, T, n, nS, chunks, 0);
  nsa_inverse_offsets_kernel<<<(unsigned)((lists + 255) / 256), 256, 0, st>>>(hist, count, lists, nS, chunks);
  nsa_inverse_scan_kernel<<<1, 1024, 0, st>>>(count, list_start, item_start, lists, R, visits_per_cta);
  nsa_inverse_walk_kernel<<<grid, 32, nS * 4, st>>>(idx, nullptr, hist, list_start, tok_list, T, n, nS, chunks, 1);
  nsa::count_launch(4);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_inverse_blocks launch");
}
