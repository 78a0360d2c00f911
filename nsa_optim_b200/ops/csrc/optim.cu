// Optimizer and loss kernels.
//   * fused AdamW (decoupled weight decay, bias correction, optional fp32 master copy);
//   * 8-bit AdamW: moments stored as uint8 codes of a 256-entry dynamic-tree code book with
//     one fp32 absmax per 256-element block (signed map for the first moment, unsigned for
//     the second); one CTA per block: dequantise, update, block absmax, requantise;
//   * sum of squares for the global gradient norm (deterministic two-stage reduction);
//   * softmax cross-entropy over a (rows, vocab) bf16 logits block: per-row loss and the
//     logits overwritten in place by d(loss)/d(logits).
// Gradients may be bf16 or fp32; an optional device scalar `grad_scale` multiplies them
// (clip coefficient), so no host synchronisation is needed between norm and update.
#include <algorithm>

#include "codebook.cuh"
#include "host.cuh"
#include <cuda_bf16.h>

namespace {
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt;   // bc1 = 1-beta1^t, bc2_sqrt = sqrt(1-beta2^t)
};

template <typename PT, typename GT>
__global__ void __launch_bounds__(256) adamw_kernel(PT* __restrict__ p, const GT* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, float* __restrict__ master,
                                                    const float* __restrict__ grad_scale, long n, AdamArgs a) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gr = static_cast<float>(g[i]) * gs;
    float w = master ? master[i] : static_cast<float>(p[i]);
    w *= (1.f - a.lr * a.wd);
    const float mm = a.beta1 * m[i] + (1.f - a.beta1) * gr;
    const float vv = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
    m[i] = mm;
    v[i] = vv;
    w -= (a.lr / a.bc1) * mm / (sqrtf(vv) / a.bc2_sqrt + a.eps);
    if (master) master[i] = w;
    p[i] = static_cast<PT>(w);
  }
}

__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
  const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
  v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  uint2 x;
  *reinterpret_cast<__nv_bfloat162*>(&x.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&x.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = x;
}

// A CTA of 256 threads takes four 256-element quantisation blocks per iteration: 64 threads per
// block, four consecutive elements per thread (8- or 16-byte loads of p and g, 4-byte loads of
// the state codes).
template <typename PT, typename GT>
__global__ void __launch_bounds__(256) adamw8bit_kernel(PT* __restrict__ p, const GT* __restrict__ g,
                                                        uint8_t* __restrict__ mq, float* __restrict__ mabs,
                                                        uint8_t* __restrict__ vq, float* __restrict__ vabs,
                                                        const float* __restrict__ cb_signed,
                                                        const float* __restrict__ cb_unsigned,
                                                        const float* __restrict__ grad_scale, long nblocks, AdamArgs a) {
  __shared__ float cs[256], cu[256];
  __shared__ uint8_t ts[cbk::kTable], tu[cbk::kTable];
  __shared__ float red_m[8], red_v[8];
  cs[threadIdx.x] = cb_signed[threadIdx.x];
  cu[threadIdx.x] = cb_unsigned[threadIdx.x];
  __syncthreads();
  cbk::build_table(cs, ts);
  cbk::build_table(cu, tu);
  __syncthreads();
  const float gs = grad_scale ? *grad_scale : 1.f;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int grp = threadIdx.x >> 6, t64 = threadIdx.x & 63;
  const long quads = (nblocks + 3) / 4;
  const float decay = 1.f - a.lr * a.wd, step_size = a.lr / a.bc1;
  for (long q = blockIdx.x; q < quads; q += gridDim.x) {
    const long b = q * 4 + grp;
    const bool live = b < nblocks;
    const long i = b * 256 + t64 * 4;
    float mm[4], vv[4];
    float am = 0.f, av = 0.f;
    if (live) {
      float gr[4], wt[4];
      load4(g + i, gr);
      load4(p + i, wt);
      const uchar4 mc = *reinterpret_cast<const uchar4*>(mq + i);
      const uchar4 vc = *reinterpret_cast<const uchar4*>(vq + i);
      const float ms = mabs[b], vs = vabs[b];
      const float m0[4] = {cs[mc.x], cs[mc.y], cs[mc.z], cs[mc.w]};
      const float v0[4] = {cu[vc.x], cu[vc.y], cu[vc.z], cu[vc.w]};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float x = gr[k] * gs;
        mm[k] = a.beta1 * (m0[k] * ms) + (1.f - a.beta1) * x;
        vv[k] = a.beta2 * (v0[k] * vs) + (1.f - a.beta2) * x * x;
        wt[k] = wt[k] * decay - step_size * mm[k] / (sqrtf(vv[k]) / a.bc2_sqrt + a.eps);
        am = fmaxf(am, fabsf(mm[k]));
        av = fmaxf(av, vv[k]);
      }
      store4(p + i, wt);
    }
    am = warp_max(am);
    av = warp_max(av);
    __syncthreads();               // previous iteration's readers of red_* are done
    if (l == 0) { red_m[w] = am; red_v[w] = av; }
    __syncthreads();
    am = fmaxf(red_m[2 * grp], red_m[2 * grp + 1]);
    av = fmaxf(red_v[2 * grp], red_v[2 * grp + 1]);
    if (live) {
      const float dm = fmaxf(am, 1e-30f), dv = fmaxf(av, 1e-30f);
      uchar4 mc, vc;
      mc.x = static_cast<uint8_t>(cbk::nearest_code(cs, ts, mm[0] / dm));
      mc.y = static_cast<uint8_t>(cbk::nearest_code(cs, ts, mm[1] / dm));
      mc.z = static_cast<uint8_t>(cbk::nearest_code(cs, ts, mm[2] / dm));
      mc.w = static_cast<uint8_t>(cbk::nearest_code(cs, ts, mm[3] / dm));
      vc.x = static_cast<uint8_t>(cbk::nearest_code(cu, tu, vv[0] / dv));
      vc.y = static_cast<uint8_t>(cbk::nearest_code(cu, tu, vv[1] / dv));
      vc.z = static_cast<uint8_t>(cbk::nearest_code(cu, tu, vv[2] / dv));
      vc.w = static_cast<uint8_t>(cbk::nearest_code(cu, tu, vv[3] / dv));
      *reinterpret_cast<uchar4*>(mq + i) = mc;
      *reinterpret_cast<uchar4*>(vq + i) = vc;
      if (t64 == 0) { mabs[b] = am; vabs[b] = av; }
    }
  }
}

template <typename GT>
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const GT* __restrict__ g, long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float s = 0.f;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float x = static_cast<float>(g[i]);
    s += x * x;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < 8; ++k) t += red[k];
    partial[blockIdx.x] = t;
  }
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int parts, float* __restrict__ out, int accumulate) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float t = accumulate ? *out : 0.f;
    for (int k = 0; k < parts; ++k) t += partial[k];
    *out = t;
  }
}

// One CTA per row.  loss_out[row] = lse - logit[label] (0 for ignored rows); the row is then
// overwritten with (softmax - onehot) * (*inv_count) (zeros for ignored rows).
__global__ void __launch_bounds__(256) cross_entropy_kernel(bf16* __restrict__ logits, const long* __restrict__ labels,
                                                            float* __restrict__ loss_out, const float* __restrict__ inv_count,
                                                            int V, long ld, long ignore_index, int write_grad,
                                                            KernelStatus* status) {
  __shared__ float red[8], red2[8];
  const long row = blockIdx.x;
  bf16* lp = logits + row * ld;
  const long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  if (threadIdx.x == 0) NSA_CHECK_INDEX(label == ignore_index || (label >= 0 && label < V), status, label);
  const int V8 = V / 8;
  // pass 1: online max / sum-exp
  float mx = -INFINITY, sum = 0.f;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = *reinterpret_cast<const uint4*>(lp + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    float x[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); x[2 * k] = f.x; x[2 * k + 1] = f.y; }
    float lm = x[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, x[k]);
    const float nm = fmaxf(mx, lm);
    float ls = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ls += __expf(x[k] - nm);
    sum = sum * __expf(mx - nm) + ls;
    mx = nm;
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float x = __bfloat162float(lp[i]);
    const float nm = fmaxf(mx, x);
    sum = sum * __expf(mx - nm) + __expf(x - nm);
    mx = nm;
  }
  // combine across the CTA
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float gm = warp_max(mx);
  if (l == 0) red[w] = gm;
  __syncthreads();
  gm = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) gm = fmaxf(gm, red[k]);
  float s = (mx == -INFINITY) ? 0.f : sum * __expf(mx - gm);
  s = warp_sum(s);
  if (l == 0) red2[w] = s;
  __syncthreads();
  s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += red2[k];
  const float lse = gm + __logf(s);
  if (threadIdx.x == 0) loss_out[row] = ignored ? 0.f : lse - __bfloat162float(lp[label]);
  if (!write_grad) return;
  __syncthreads();      // the label logit has been read before anyone overwrites it
  const float scale = ignored ? 0.f : *inv_count;
  for (int i = threadIdx.x; i < V8; i += blockDim.x) {
    uint4 u = *reinterpret_cast<const uint4*>(lp + i * 8);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      const int c = i * 8 + 2 * k;
      f.x = (__expf(f.x - lse) - (c == label ? 1.f : 0.f)) * scale;
      f.y = (__expf(f.y - lse) - (c + 1 == label ? 1.f : 0.f)) * scale;
      h[k] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(lp + i * 8) = u;
  }
  for (int i = V8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float x = __bfloat162float(lp[i]);
    lp[i] = __float2bfloat16((__expf(x - lse) - (i == label ? 1.f : 0.f)) * scale);
  }
}

inline int grid_cap(long want, int per_sm) {
  long cap = static_cast<long>(nsa::sm_count()) * per_sm;
  return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
}
AdamArgs make_args(int step, float lr, float b1, float b2, float eps, float wd) {
  AdamArgs a;
  a.lr = lr; a.beta1 = b1; a.beta2 = b2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(b1, (float)step);
  a.bc2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  return a;
}
// ------------------------------------------------------------------------------------
// Asymmetric affine block quantisation of SOAP's eigenbases: every row is cut into blocks of
// q_block columns; a block stores uint8 codes q = round(x / scale + zero) with
// scale = (max - min) / (2^bits - 1) and zero = round(-min / scale) kept as a float.  One warp per block.
// Divisions are IEEE (not the fast-math approximations) so the codes match the PyTorch form.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) affine_quant_kernel(const float* __restrict__ t, uint8_t* __restrict__ q,
                                                           float* __restrict__ scale, float* __restrict__ zero, long rows,
                                                           int cols, int q_block, int nblk, float qmax) {
  const int lane = threadIdx.x & 31;
  const long wid = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (wid >= rows * nblk) return;
  const long row = wid / nblk;
  const int blk = static_cast<int>(wid - row * nblk);
  const float* src = t + row * cols;
  const int c0 = blk * q_block;
  float lo = INFINITY, hi = -INFINITY;
  for (int j = lane; j < q_block; j += 32) {
    const int c = min(c0 + j, cols - 1);            // the padded tail repeats the last column
    const float x = src[c];
    lo = fminf(lo, x);
    hi = fmaxf(hi, x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  const float sc = fmaxf(__fdiv_rn(hi - lo, qmax), 1e-12f);
  const float zp = rintf(__fdiv_rn(-lo, sc));        // not clamped: a one-signed block has its zero outside the code range
  if (lane == 0) { scale[wid] = sc; zero[wid] = zp; }
  uint8_t* dst = q + (row * nblk + blk) * static_cast<long>(q_block);
  for (int j = lane; j < q_block; j += 32) {
    const int c = min(c0 + j, cols - 1);
    const float v = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(src[c], sc), zp)), 0.f), qmax);
    dst[j] = static_cast<uint8_t>(v);
  }
}
__global__ void __launch_bounds__(256) affine_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                                                             const float* __restrict__ zero, float* __restrict__ out,
                                                             long rows, int cols, int q_block, int nblk) {
  const long n = rows * cols;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long row = i / cols;
    const int c = static_cast<int>(i - row * cols);
    const long b = row * nblk + c / q_block;
    out[i] = (static_cast<float>(q[row * static_cast<long>(nblk) * q_block + c]) - zero[b]) * scale[b];
  }
}
}  // namespace

// p: bf16 (p_fp32 = 0) or fp32; g: bf16 (g_fp32 = 0) or fp32; m, v fp32; master fp32 or null.
extern "C" int nsa_adamw_step(void* p, const void* g, float* m, float* v, float* master, const float* grad_scale,
                              long n, int p_fp32, int g_fp32, int step, float lr, float b1, float b2, float eps, float wd,
                              cudaStream_t st) {
  if (n <= 0) return 0;
  const AdamArgs a = make_args(step, lr, b1, b2, eps, wd);
  const int grid = grid_cap((n + 255) / 256, 16);
  if (p_fp32 && g_fp32) adamw_kernel<float, float><<<grid, 256, 0, st>>>((float*)p, (const float*)g, m, v, master, grad_scale, n, a);
  else if (p_fp32) adamw_kernel<float, bf16><<<grid, 256, 0, st>>>((float*)p, (const bf16*)g, m, v, master, grad_scale, n, a);
  else if (g_fp32) adamw_kernel<bf16, float><<<grid, 256, 0, st>>>((bf16*)p, (const float*)g, m, v, master, grad_scale, n, a);
  else adamw_kernel<bf16, bf16><<<grid, 256, 0, st>>>((bf16*)p, (const bf16*)g, m, v, master, grad_scale, n, a);
  nsa::count_launch();
  return 0;
}

// n must be a multiple of 256.  cb_signed / cb_unsigned: device pointers to 256 fp32 entries.
extern "C" int nsa_adamw8bit_step(void* p, const void* g, uint8_t* mq, float* mabs, uint8_t* vq, float* vabs,
                                  const float* cb_signed, const float* cb_unsigned, const float* grad_scale, long n,
                                  int p_fp32, int g_fp32, int step, float lr, float b1, float b2, float eps, float wd,
                                  cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 256) return nsa::fail(NSA_ERR_SHAPE, "adamw8bit: element count must be a multiple of 256");
  const AdamArgs a = make_args(step, lr, b1, b2, eps, wd);
  const long nb = n / 256;
  const int grid = grid_cap((nb + 3) / 4, 8);
  if (p_fp32 && g_fp32) adamw8bit_kernel<float, float><<<grid, 256, 0, st>>>((float*)p, (const float*)g, mq, mabs, vq, vabs, cb_signed, cb_unsigned, grad_scale, nb, a);
  else if (p_fp32) adamw8bit_kernel<float, bf16><<<grid, 256, 0, st>>>((float*)p, (const bf16*)g, mq, mabs, vq, vabs, cb_signed, cb_unsigned, grad_scale, nb, a);
  else if (g_fp32) adamw8bit_kernel<bf16, float><<<grid, 256, 0, st>>>((bf16*)p, (const float*)g, mq, mabs, vq, vabs, cb_signed, cb_unsigned, grad_scale, nb, a);
  else adamw8bit_kernel<bf16, bf16><<<grid, 256, 0, st>>>((bf16*)p, (const bf16*)g, mq, mabs, vq, vabs, cb_signed, cb_unsigned, grad_scale, nb, a);
  nsa::count_launch();
  return 0;
}

// out (device scalar) = [out +] sum(g^2).  partial: scratch of nsa_sumsq_parts() floats.
extern "C" int nsa_sumsq_parts() { return nsa::sm_count() * 4; }
extern "C" int nsa_sumsq(const void* g, long n, int g_fp32, float* partial, float* out, int accumulate, cudaStream_t st) {
  const int parts = grid_cap((n + 255) / 256, 4);
  if (g_fp32) sumsq_partial_kernel<float><<<parts, 256, 0, st>>>((const float*)g, n, partial);
  else sumsq_partial_kernel<bf16><<<parts, 256, 0, st>>>((const bf16*)g, n, partial);
  sumsq_final_kernel<<<1, 32, 0, st>>>(partial, parts, out, accumulate);
  nsa::count_launch(2);
  return 0;
}

extern "C" int nsa_cross_entropy(void* logits, const long* labels, float* loss_rows, const float* inv_count, long rows,
                                 int V, long ld, long ignore_index, int write_grad, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ld % 8) return nsa::fail(NSA_ERR_SHAPE, "cross_entropy: row pitch must be a multiple of 8");
  cross_entropy_kernel<<<(unsigned)rows, 256, 0, st>>>((bf16*)logits, labels, loss_rows, inv_count, V, ld, ignore_index, write_grad,
                                                       nsa::status_ptr());
  nsa::count_launch();
  return 0;
}

// t: [rows, cols] fp32 -> q: [rows, nblk * q_block] uint8, scale / zero: [rows, nblk] with nblk = ceil(cols / q_block).
extern "C" int nsa_affine_quant(const float* t, uint8_t* q, float* scale, float* zero, long rows, int cols, int q_block,
                                int bits, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || q_block <= 0 || bits < 1 || bits > 8) return nsa::fail(NSA_ERR_SHAPE, "affine_quant: bad shape");
  const int nblk = (cols + q_block - 1) / q_block;
  const long warps = rows * nblk;
  affine_quant_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(t, q, scale, zero, rows, cols, q_block, nblk,
                                                                   static_cast<float>((1 << bits) - 1));
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_affine_dequant(const uint8_t* q, const float* scale, const float* zero, float* out, long rows, int cols,
                                  int q_block, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || q_block <= 0) return nsa::fail(NSA_ERR_SHAPE, "affine_dequant: bad shape");
  const int nblk = (cols + q_block - 1) / q_block;
  const long n = rows * cols;
  const long blocks = std::min<long>((n + 255) / 256, 148L * 16);
  affine_dequant_kernel<<<(unsigned)blocks, 256, 0, st>>>(q, scale, zero, out, rows, cols, q_block, nblk);
  nsa::count_launch();
  return 0;
}
