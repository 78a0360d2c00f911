// Bandwidth-bound kernels: RMSNorm / gated RMSNorm / L2 norm (forward + backward),
// SwiGLU, rotary embedding, causal depthwise conv1d (+SiLU), embedding gather and its
// deterministic scatter-add backward.  bf16 storage, fp32 arithmetic, 16-byte accesses.
//
// Row kernels keep a whole row in registers (one global read per element).  Rows up to 512
// elements use one warp per row, longer rows (up to 8192) use one 256-thread CTA per row.
// Weight gradients of the norms and the convolution are reduced deterministically:
// a persistent grid accumulates per-CTA partial sums into a scratch buffer
// [grid, width] (fp32) that a second kernel adds up in a fixed order.
#include "host.cuh"
#include <cuda_bf16.h>

namespace {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8(const uint4& u, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
// d/dx silu(x)
__device__ __forceinline__ float dsilu_f(float x) {
  float s = sigmoid_f(x);
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over the TPR threads that share a row.  TPR == 32: warp; TPR == 256: whole CTA.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < TPR / 32; ++i) t += red[i];
  return t;
}

// ------------------------------------------------------------------------------------
// (gated) RMSNorm.  MODE 0: y = x*rstd*w.   MODE 1: y = x*rstd*w * silu(g)   (norm, then gate)
//                   MODE 2: u = x*silu(g); y = u*rstd(u)*w                    (gate, then norm)
// ------------------------------------------------------------------------------------
template <int TPR, int NV, int MODE>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ g,
                                                          const bf16* __restrict__ w, bf16* __restrict__ y,
                                                          float* __restrict__ rstd_out, long rows, int d, float eps,
                                                          long ldg) {
  __shared__ float red[8];
  const int rows_per_cta = 256 / TPR;
  const long row = static_cast<long>(blockIdx.x) * rows_per_cta + threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const bool active = row < rows;
  float xv[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * TPR) * 8;
    if (active && c < d) {
      load8(x + row * d + c, xv[i]);
      if (MODE == 2) {
        float gv[8];
        load8(g + row * ldg + c, gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) xv[i][j] *= silu_f(gv[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += xv[i][j] * xv[i][j];
    }
  }
  ss = row_sum<TPR>(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (active && t == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * TPR) * 8;
    if (active && c < d) {
      float wv[8], o[8];
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = xv[i][j] * rstd * wv[j];
      if (MODE == 1) {
        float gv[8];
        load8(g + row * ldg + c, gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= silu_f(gv[j]);
      }
      store8(y + row * d + c, o);
    }
  }
}

// Residual add fused into the plain norm: h = x + r (rounded to bf16, written out because the
// residual stream continues from it) and y = h * rstd(h) * w, one read of x and r, one write of
// h and y.  The statistics use the rounded h, so the result equals add-then-norm to the bit.
template <int TPR, int NV>
__global__ void __launch_bounds__(256) rmsnorm_add_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ r,
                                                              const bf16* __restrict__ w, bf16* __restrict__ h,
                                                              bf16* __restrict__ y, float* __restrict__ rstd_out,
                                                              long rows, int d, float eps) {
  __shared__ float red[8];
  const int rows_per_cta = 256 / TPR;
  const long row = static_cast<long>(blockIdx.x) * rows_per_cta + threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const bool active = row < rows;
  float hv[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * TPR) * 8;
    if (active && c < d) {
      float rv[8];
      load8(x + row * d + c, hv[i]);
      load8(r + row * d + c, rv);
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[i][j] = __bfloat162float(__float2bfloat16(hv[i][j] + rv[j]));
      store8(h + row * d + c, hv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += hv[i][j] * hv[i][j];
    }
  }
  ss = row_sum<TPR>(ss, red);
  const float rstd = rsqrtf(ss / d + eps);
  if (active && t == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * TPR) * 8;
    if (active && c < d) {
      float wv[8], o[8];
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = hv[i][j] * rstd * wv[j];
      store8(y + row * d + c, o);
    }
  }
}

// Backward.  Persistent over rows; writes dx (and dg for gated modes) and per-CTA partial
// dw into `partial[gridDim.x][d]`.  `dres` (may be null) is a gradient that reaches the norm's
// input by another route (the residual stream); it is added into dx here instead of by a
// separate pass over both tensors.
template <int TPR, int NV, int MODE>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ g,
                                                          const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                                          const float* __restrict__ rstd_in, bf16* __restrict__ dx,
                                                          bf16* __restrict__ dg, float* __restrict__ partial,
                                                          long rows, int d, const bf16* __restrict__ dres = nullptr,
                                                          long ldg = 0) {
  __shared__ float red[8];
  __shared__ float dw_sh[(TPR == 32) ? 512 : 1];
  const int rows_per_cta = 256 / TPR;
  const int sub = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  float dwacc[NV][8];
  float wv[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * TPR) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (c < d) load8(w + c, wv[i]);
  }
  for (long base = static_cast<long>(blockIdx.x) * rows_per_cta; base < rows; base += static_cast<long>(gridDim.x) * rows_per_cta) {
    const long row = base + sub;
    const bool active = row < rows;
    const float rstd = active ? rstd_in[row] : 0.f;
    float xn[NV][8], wdy[NV][8], gv[NV][8], sg[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (t + i * TPR) * 8;
      if (active && c < d) {
        float xv[8], dv[8];
        load8(x + row * d + c, xv);
        load8(dy + row * d + c, dv);
        if (MODE != 0) load8(g + row * (ldg ? ldg : d) + c, gv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float xin = xv[j];
          float dout = dv[j];
          if (MODE == 2) { sg[i][j] = silu_f(gv[i][j]); xin *= sg[i][j]; }
          xn[i][j] = xin * rstd;
          if (MODE == 1) {
            // y = n*w*silu(g): dg = dy*n*w*dsilu(g); upstream for the norm is dy*silu(g)
            const float s = silu_f(gv[i][j]);
            sg[i][j] = dout * xn[i][j] * wv[i][j] * dsilu_f(gv[i][j]);   // dg
            dout *= s;
          }
          dwacc[i][j] += dout * xn[i][j];
          wdy[i][j] = dout * wv[i][j];
          dot += wdy[i][j] * xn[i][j];
        }
      }
    }
    dot = row_sum<TPR>(dot, red) / d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (t + i * TPR) * 8;
      if (active && c < d) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (wdy[i][j] - xn[i][j] * dot);   // d/d(norm input)
        if (MODE == 2) {
          // norm input u = x*silu(g): dx = du*silu(g), dg = du*x*dsilu(g)
          float xv[8], og[8];
          load8(x + row * d + c, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            og[j] = o[j] * xv[j] * dsilu_f(gv[i][j]);
            o[j] *= sg[i][j];
          }
          store8(dg + row * d + c, og);
        } else if (MODE == 1) {
          store8(dg + row * d + c, sg[i]);
        }
        if (dres != nullptr) {
          float rv[8];
          load8(dres + row * d + c, rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rv[j];
        }
        store8(dx + row * d + c, o);
      }
    }
  }
  // per-CTA partial dw
  if (TPR == 32) {
    // 8 sub-rows share columns: combine through shared memory in a fixed order
    for (int i = 0; i < NV; ++i) {
      const int c = (t + i * TPR) * 8;
      for (int s = 0; s < rows_per_cta; ++s) {
        __syncthreads();
        if (sub == s && c < d) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dw_sh[c + j] = (s == 0 ? 0.f : dw_sh[c + j]) + dwacc[i][j];
        }
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < d; c += 256) partial[static_cast<long>(blockIdx.x) * d + c] = dw_sh[c];
  } else {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (t + i * TPR) * 8;
      if (c < d) {
#pragma unroll
        for (int j = 0; j < 8; ++j) partial[static_cast<long>(blockIdx.x) * d + c + j] = dwacc[i][j];
      }
    }
  }
}

// out[c] = sum_p partial[p][c], p ascending (deterministic); bf16 or fp32 output.
__global__ void reduce_partials_kernel(const float* __restrict__ partial, int parts, int width,
                                       bf16* __restrict__ out_bf16, float* __restrict__ out_f32) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<long>(p) * width + c];
  if (out_bf16) out_bf16[c] = __float2bfloat16(s);
  if (out_f32) out_f32[c] = s;
}

// out[o][i] = sum_p in[o][p][i] over bf16 partial results, summed in fp32 in ascending p (the same
// bits on every run), 8 elements per thread.
__global__ void __launch_bounds__(256) sum_parts_bf16_kernel(const bf16* __restrict__ in, bf16* __restrict__ out,
                                                             int parts, long n8, long outer) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8 * outer;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long o = i / n8, e = i - o * n8;
    const uint4* src = reinterpret_cast<const uint4*>(in) + (o * parts) * n8 + e;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int p = 0; p < parts; ++p) {
      float v[8];
      unpack8(src[static_cast<long>(p) * n8], v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
    store8(out + i * 8, acc);
  }
}

// Rows of D bf16 between head-major (B, H, Ts, D) and token-major (B, Tt, H, D) storage, one warp per
// row: to_token = 1 reads (b, h, t) and writes (b, t, h); to_token = 0 the reverse.  Only t < min(Ts, Tt)
// is copied; when the destination is head-major and longer, its rows t >= Tt are zeroed.
__global__ void __launch_bounds__(256) permute_rows_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, int B, int H,
                                                           int Th, int Tt, int D, int to_token) {
  const int d8 = D / 8;
  const int Tloop = to_token ? Tt : Th;            // rows of the destination per (b, h)
  const long rows = static_cast<long>(B) * H * Tloop;
  const int lane = threadIdx.x & 31;
  for (long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += static_cast<long>(gridDim.x) * 8) {
    long b, h, t;
    if (to_token) { b = row / (static_cast<long>(Tt) * H); const long r2 = row - b * Tt * H; t = r2 / H; h = r2 - t * H; }
    else { b = row / (static_cast<long>(H) * Th); const long r2 = row - b * H * Th; h = r2 / Th; t = r2 - h * Th; }
    const bf16* hp = (to_token ? src : dst) + ((b * H + h) * Th + t) * D;     // head-major address
    const bf16* tp = (to_token ? dst : src) + ((b * Tt + t) * H + h) * D;     // token-major address
    if (to_token) {
      if (t < Th)
        for (int j = lane; j < d8; j += 32) reinterpret_cast<uint4*>(const_cast<bf16*>(tp))[j] = reinterpret_cast<const uint4*>(hp)[j];
    } else {
      for (int j = lane; j < d8; j += 32)
        reinterpret_cast<uint4*>(const_cast<bf16*>(hp))[j] = t < Tt ? reinterpret_cast<const uint4*>(tp)[j] : make_uint4(0, 0, 0, 0);
    }
  }
}

// ------------------------------------------------------------------------------------
// L2 norm over the last dimension (d <= 512, warp per row)
// ------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y,
                                                         float* __restrict__ rinv_out, long rows, int d, float eps) {
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int t = threadIdx.x & 31;
  if (row >= rows) return;
  float xv[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * 32) * 8;
    if (c < d) {
      load8(x + row * d + c, xv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += xv[i][j] * xv[i][j];
    }
  }
  ss = warp_sum(ss);
  const float rinv = rsqrtf(ss + eps);
  if (t == 0) rinv_out[row] = rinv;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * 32) * 8;
    if (c < d) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = xv[i][j] * rinv;
      store8(y + row * d + c, o);
    }
  }
}
template <int NV>
__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const bf16* __restrict__ y, const bf16* __restrict__ dy,
                                                         const float* __restrict__ rinv_in, bf16* __restrict__ dx,
                                                         long rows, int d) {
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int t = threadIdx.x & 31;
  if (row >= rows) return;
  float yv[NV][8], dv[NV][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * 32) * 8;
    if (c < d) {
      load8(y + row * d + c, yv[i]);
      load8(dy + row * d + c, dv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += yv[i][j] * dv[i][j];
    }
  }
  dot = warp_sum(dot);
  const float rinv = rinv_in[row];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (t + i * 32) * 8;
    if (c < d) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rinv * (dv[i][j] - yv[i][j] * dot);
      store8(dx + row * d + c, o);
    }
  }
}

// ------------------------------------------------------------------------------------
// SwiGLU
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u,
                                                         bf16* __restrict__ y, long n8, int cols8, long ldg8, long ldu8) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / cols8, c = i - r * cols8;
    float gv[8], uv[8], o[8];
    load8(g + (r * ldg8 + c) * 8, gv);
    load8(u + (r * ldu8 + c) * 8, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu_f(gv[j]) * uv[j];
    store8(y + i * 8, o);
  }
}
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ u,
                                                         const bf16* __restrict__ dy, bf16* __restrict__ dg,
                                                         bf16* __restrict__ du, long n8, int cols8, long ldg8, long ldu8,
                                                         long ldo8) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / cols8, c = i - r * cols8;
    float gv[8], uv[8], dv[8], o1[8], o2[8];
    load8(g + (r * ldg8 + c) * 8, gv);
    load8(u + (r * ldu8 + c) * 8, uv);
    load8(dy + i * 8, dv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o1[j] = dv[j] * uv[j] * dsilu_f(gv[j]);
      o2[j] = dv[j] * silu_f(gv[j]);
    }
    store8(dg + (r * ldo8 + c) * 8, o1);
    store8(du + (r * ldo8 + c) * 8, o2);
  }
}

// ------------------------------------------------------------------------------------
// Gated combine of the three sparse-attention branches: o = g1 o1 + g2 o2 + g3 o3 with one gate
// per (token, head) row.  Backward: do_i = g_i do and dg_i = sum_d do * o_i.  LANES = D / 8 threads
// share a row (8 elements each); LANES is a power of two <= 32 so a row never straddles a warp.
// ------------------------------------------------------------------------------------
template <int LANES>
__global__ void __launch_bounds__(256) gate_combine_fwd_kernel(const bf16* __restrict__ o1, const bf16* __restrict__ o2,
                                                               const bf16* __restrict__ o3, const bf16* __restrict__ g1,
                                                               const bf16* __restrict__ g2, const bf16* __restrict__ g3,
                                                               bf16* __restrict__ o, long n8, int Hq, long ldg, int sig) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long row = i / LANES;
    const long gi = (row / Hq) * ldg + row % Hq;           // gates: [tokens, Hq] with row pitch ldg
    float a = __bfloat162float(g1[gi]), b = __bfloat162float(g2[gi]), c = __bfloat162float(g3[gi]);
    if (sig) { a = sigmoid_f(a); b = sigmoid_f(b); c = sigmoid_f(c); }   // gates given as logits
    float x[8], y[8], z[8], r[8];
    load8(o1 + i * 8, x);
    load8(o2 + i * 8, y);
    load8(o3 + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = a * x[j] + b * y[j] + c * z[j];
    store8(o + i * 8, r);
  }
}
template <int LANES>
__global__ void __launch_bounds__(256) gate_combine_bwd_kernel(const bf16* __restrict__ o1, const bf16* __restrict__ o2,
                                                               const bf16* __restrict__ o3, const bf16* __restrict__ g1,
                                                               const bf16* __restrict__ g2, const bf16* __restrict__ g3,
                                                               const bf16* __restrict__ d_o, bf16* __restrict__ do1,
                                                               bf16* __restrict__ do2, bf16* __restrict__ do3,
                                                               bf16* __restrict__ dg1, bf16* __restrict__ dg2,
                                                               bf16* __restrict__ dg3, long n8, int Hq, long ldg, int sig) {
  // the grid is sized so that every thread handles exactly one vector (rows stay inside a warp)
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = i < n8;
  const long row = (live ? i : 0) / LANES;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const long gi = (row / Hq) * ldg + row % Hq;
  float a = 0.f, b = 0.f, c = 0.f;
  if (live) {
    a = __bfloat162float(g1[gi]); b = __bfloat162float(g2[gi]); c = __bfloat162float(g3[gi]);
    if (sig) { a = sigmoid_f(a); b = sigmoid_f(b); c = sigmoid_f(c); }
    float x[8], y[8], z[8], d[8], r[8];
    load8(o1 + i * 8, x);
    load8(o2 + i * 8, y);
    load8(o3 + i * 8, z);
    load8(d_o + i * 8, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) { s1 += d[j] * x[j]; s2 += d[j] * y[j]; s3 += d[j] * z[j]; }
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = a * d[j];
    store8(do1 + i * 8, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = b * d[j];
    store8(do2 + i * 8, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = c * d[j];
    store8(do3 + i * 8, r);
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    s3 += __shfl_xor_sync(0xffffffffu, s3, o);
  }
  if (live && (threadIdx.x % LANES) == 0) {
    // gates given as logits: the gradient goes back through the sigmoid here
    if (sig) { s1 *= a * (1.f - a); s2 *= b * (1.f - b); s3 *= c * (1.f - c); }
    dg1[gi] = __float2bfloat16(s1);
    dg2[gi] = __float2bfloat16(s2);
    dg3[gi] = __float2bfloat16(s3);
  }
}

// ------------------------------------------------------------------------------------
// Mean pooling of keys / values into compressed blocks (native sparse attention):
//   y[b, i, :] = mean over t in [i*stride, i*stride + block) of x[b, t, :]
// x rows are `width` = Hkv * D elements with row pitch ldx; y is contiguous [B, nC, width].
// Backward: dx[b, t, :] = (1/block) * sum of dy[b, i, :] over the windows i that contain t.
// One thread per 8 elements; fp32 accumulation in a fixed order.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) nsa_pool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, int T, int nC,
                                                           int width8, long ldx, int block, int stride, long n) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(i % width8);
    const long r = i / width8;
    const int ci = static_cast<int>(r % nC);
    const long b = r / nC;
    const bf16* src = x + (b * T + static_cast<long>(ci) * stride) * ldx + c8 * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int t = 0; t < block; ++t) {
      float v[8];
      load8(src + t * ldx, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    const float inv = 1.f / block;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
    store8(y + i * 8, acc);
  }
}
__global__ void __launch_bounds__(256) nsa_pool_bwd_kernel(const bf16* __restrict__ dy, bf16* __restrict__ dx, int T, int nC,
                                                           int width8, int block, int stride, long n) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(i % width8);
    const long r = i / width8;
    const int t = static_cast<int>(r % T);
    const long b = r / T;
    int lo = t - block + 1;
    lo = lo <= 0 ? 0 : (lo + stride - 1) / stride;
    int hi = t / stride;
    hi = hi < nC - 1 ? hi : nC - 1;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int ci = lo; ci <= hi; ++ci) {
      float v[8];
      load8(dy + ((b * nC + ci) * width8 + c8) * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    const float inv = 1.f / block;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv;
    store8(dx + i * 8, acc);
  }
}

// ------------------------------------------------------------------------------------
// Gated DeltaNet layout pass.  q, k (B, T, H, 128) and v (B, T, H, V) arrive token-major; the
// chunk kernels want head-major rows (B*H, Tp, .) with Tp the padded length.  One warp per row
// writes the copies qh, kh, vh and the decay-scaled operands qd = q * sq, kt = k * sk in one pass
// (rows >= T are zero).  The backward folds the five incoming gradients back to token-major and
// reduces d sq = sum(dqd * q), d sk = sum(dkt * k).
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gdn_pack_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                           const bf16* __restrict__ v, const float* __restrict__ sq,
                                                           const float* __restrict__ sk, bf16* __restrict__ qh,
                                                           bf16* __restrict__ kh, bf16* __restrict__ vh,
                                                           bf16* __restrict__ qd, bf16* __restrict__ kt, int B, int T,
                                                           int Tp, int H, int V) {
  constexpr int K = 128;
  const int lane = threadIdx.x & 31;
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);     // (b*H + h) * Tp + t
  if (row >= static_cast<long>(B) * H * Tp) return;
  const int t = static_cast<int>(row % Tp);
  const long bh = row / Tp;
  const int h = static_cast<int>(bh % H);
  const long b = bh / H;
  const bool live = t < T;
  const long tok = (b * T + (live ? t : 0)) * H + h;
  float x[8], y[8];
  const int part = lane >> 4, c = (lane & 15) * 8;                             // lanes 0-15: q, 16-31: k
  const bf16* src = (part ? k : q) + tok * K + c;
  const float s = live ? (part ? sk : sq)[row] : 0.f;
  if (live) load8(src, x);
  else {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = 0.f;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = x[j] * s;
  store8((part ? kh : qh) + row * K + c, x);
  store8((part ? kt : qd) + row * K + c, y);
  for (int cv = lane * 8; cv < V; cv += 256) {
    if (live) load8(v + tok * V + cv, x);
    store8(vh + row * V + cv, x);            // x is zero on padded rows
  }
}
__global__ void __launch_bounds__(256) gdn_pack_bwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                           const float* __restrict__ sq, const float* __restrict__ sk,
                                                           const bf16* __restrict__ dqh, const bf16* __restrict__ dkh,
                                                           const bf16* __restrict__ dvh, const bf16* __restrict__ dqd,
                                                           const bf16* __restrict__ dkt, bf16* __restrict__ dq,
                                                           bf16* __restrict__ dk, bf16* __restrict__ dv,
                                                           float* __restrict__ dsq, float* __restrict__ dsk, int B, int T,
                                                           int Tp, int H, int V) {
  constexpr int K = 128;
  const int lane = threadIdx.x & 31;
  const long row = static_cast<long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= static_cast<long>(B) * H * Tp) return;
  const int t = static_cast<int>(row % Tp);
  const long bh = row / Tp;
  const int h = static_cast<int>(bh % H);
  const long b = bh / H;
  const int part = lane >> 4, c = (lane & 15) * 8;
  if (t >= T) {                                                                // padded row: no token, zero scale gradients
    if ((lane & 15) == 0) (part ? dsk : dsq)[row] = 0.f;
    return;
  }
  const long tok = (b * T + t) * H + h;
  float x[8], g1[8], g2[8], o[8];
  load8((part ? k : q) + tok * K + c, x);
  const bf16* a = part ? dkh : dqh;
  const bf16* d = part ? dkt : dqd;
  if (a) load8(a + row * K + c, g1);
  else {
#pragma unroll
    for (int j = 0; j < 8; ++j) g1[j] = 0.f;
  }
  if (d) load8(d + row * K + c, g2);
  else {
#pragma unroll
    for (int j = 0; j < 8; ++j) g2[j] = 0.f;
  }
  const float s = (part ? sk : sq)[row];
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    o[j] = g1[j] + g2[j] * s;
    dot += g2[j] * x[j];
  }
  store8((part ? dk : dq) + tok * K + c, o);
#pragma unroll
  for (int m = 8; m > 0; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);   // within each half-warp
  if ((lane & 15) == 0) (part ? dsk : dsq)[row] = dot;
  for (int cv = lane * 8; cv < V; cv += 256) {
    if (dvh) load8(dvh + row * V + cv, o);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
    }
    store8(dv + tok * V + cv, o);
  }
}

// ------------------------------------------------------------------------------------
// Gated DeltaNet per-chunk matrices (chunk 64), one CTA of 64 threads per chunk.
//   A[i][j] = beta_i * kk[i][j] * exp(gc_i - gc_j)   (i > j)       kk = K K^T of the chunk
//   X = (I + A)^-1    by forward substitution, thread c owning column c in registers
//   Tu = X diag(beta),  Tw = X diag(beta * exp(gc)),  qk[i][j] = scale * qkr[i][j] * exp(gc_i - gc_j)  (i >= j)
// The backward takes dA = -(X^T dX X^T) (two batched matmuls done by the caller) and folds it,
// together with dTu, dTw, dqk, into dkk, dqkr, d gc and d beta.
// ------------------------------------------------------------------------------------
constexpr int GC = 64;

__device__ __forceinline__ void load_row64(const bf16* p, float (&v)[GC]) {
#pragma unroll
  for (int j = 0; j < GC / 8; ++j) {
    float t[8];
    load8(p + 8 * j, t);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[8 * j + e] = t[e];
  }
}
__device__ __forceinline__ void store_row64(bf16* p, const float (&v)[GC]) {
#pragma unroll
  for (int j = 0; j < GC / 8; ++j) {
    float t[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) t[e] = v[8 * j + e];
    store8(p + 8 * j, t);
  }
}

__global__ void __launch_bounds__(64) gdn_tmat_fwd_kernel(const bf16* __restrict__ kk, const bf16* __restrict__ qkr,
                                                          const float* __restrict__ gc, const float* __restrict__ beta,
                                                          bf16* __restrict__ Tu, bf16* __restrict__ Tw, bf16* __restrict__ qk,
                                                          float* __restrict__ X, float scale) {
  __shared__ float As[GC][GC + 1];
  __shared__ float g_s[GC], b_s[GC];
  const long ch = blockIdx.x;
  const int i = threadIdx.x;
  const long mat = ch * GC * GC;
  g_s[i] = gc[ch * GC + i];
  b_s[i] = beta[ch * GC + i];
  __syncthreads();
  const float gi = g_s[i], bi = b_s[i];
  float row[GC];
  load_row64(kk + mat + i * GC, row);
#pragma unroll
  for (int j = 0; j < GC; ++j) As[i][j] = (j < i) ? bi * row[j] * __expf(gi - g_s[j]) : 0.f;
  // qk row while the A tile settles
  load_row64(qkr + mat + i * GC, row);
#pragma unroll
  for (int j = 0; j < GC; ++j) row[j] = (j <= i) ? scale * row[j] * __expf(gi - g_s[j]) : 0.f;
  store_row64(qk + mat + i * GC, row);
  __syncthreads();
  // column c = threadIdx.x of X: x[r] = [r == c] - sum_{j < r} A[r][j] x[j]
  const int c = i;
  float x[GC];
#pragma unroll
  for (int r = 0; r < GC; ++r) {
    float acc = (r == c) ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < r; ++j) acc = fmaf(-As[r][j], x[j], acc);
    x[r] = acc;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < GC; ++r) As[r][c] = x[r];          // reuse the tile for X
  __syncthreads();
  float tu[GC], tw[GC];
#pragma unroll
  for (int j = 0; j < GC; ++j) {
    const float xv = As[i][j];
    row[j] = xv;
    tu[j] = xv * b_s[j];
    tw[j] = tu[j] * __expf(g_s[j]);
  }
  float4* xo = reinterpret_cast<float4*>(X + mat + i * GC);
#pragma unroll
  for (int j = 0; j < GC / 4; ++j) xo[j] = make_float4(row[4 * j], row[4 * j + 1], row[4 * j + 2], row[4 * j + 3]);
  store_row64(Tu + mat + i * GC, tu);
  store_row64(Tw + mat + i * GC, tw);
}

// dX[i][c] = (dTu[i][c] + dTw[i][c] * exp(gc_c)) * beta_c   for c <= i, else 0
__global__ void __launch_bounds__(64) gdn_tmat_dx_kernel(const bf16* __restrict__ dTu, const bf16* __restrict__ dTw,
                                                         const float* __restrict__ gc, const float* __restrict__ beta,
                                                         float* __restrict__ dX) {
  __shared__ float g_s[GC], b_s[GC];
  const long ch = blockIdx.x;
  const int i = threadIdx.x;
  const long mat = ch * GC * GC;
  g_s[i] = __expf(gc[ch * GC + i]);
  b_s[i] = beta[ch * GC + i];
  __syncthreads();
  float a[GC], b[GC];
  load_row64(dTu + mat + i * GC, a);
  load_row64(dTw + mat + i * GC, b);
  float4* o = reinterpret_cast<float4*>(dX + mat + i * GC);
#pragma unroll
  for (int j = 0; j < GC; ++j) a[j] = (j <= i) ? (a[j] + b[j] * g_s[j]) * b_s[j] : 0.f;
#pragma unroll
  for (int j = 0; j < GC / 4; ++j) o[j] = make_float4(a[4 * j], a[4 * j + 1], a[4 * j + 2], a[4 * j + 3]);
}

__global__ void __launch_bounds__(64) gdn_tmat_bwd_kernel(const float* __restrict__ dA, const bf16* __restrict__ kk,
                                                          const bf16* __restrict__ qkr, const bf16* __restrict__ dqk,
                                                          const bf16* __restrict__ dTu, const bf16* __restrict__ dTw,
                                                          const float* __restrict__ X, const float* __restrict__ gc,
                                                          const float* __restrict__ beta, bf16* __restrict__ dkk,
                                                          bf16* __restrict__ dqkr, float* __restrict__ dgc,
                                                          float* __restrict__ dbeta, float scale) {
  __shared__ float Cg[GC][GC + 1];      // per element: contribution to d gc of its column index
  __shared__ float Cb[GC][GC + 1];      // per element: contribution to d beta of its column index
  __shared__ float g_s[GC], b_s[GC];
  const long ch = blockIdx.x;
  const int i = threadIdx.x;
  const long mat = ch * GC * GC;
  g_s[i] = gc[ch * GC + i];
  b_s[i] = beta[ch * GC + i];
  __syncthreads();
  const float gi = g_s[i], bi = b_s[i];
  float r1[GC], r2[GC], out[GC];
  float dg_row = 0.f, db_row = 0.f;
  // ---- A part: dA (fp32 row) with kk
  load_row64(kk + mat + i * GC, r1);
  const float4* da4 = reinterpret_cast<const float4*>(dA + mat + i * GC);
#pragma unroll
  for (int j = 0; j < GC / 4; ++j) {
    const float4 v = da4[j];
    r2[4 * j] = v.x; r2[4 * j + 1] = v.y; r2[4 * j + 2] = v.z; r2[4 * j + 3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < GC; ++j) {
    float cg = 0.f;
    out[j] = 0.f;
    if (j < i) {
      const float e = __expf(gi - g_s[j]);
      const float araw = r1[j] * e;
      const float d = r2[j];
      out[j] = d * bi * e;
      db_row += d * araw;
      const float t = d * bi * araw;
      dg_row += t;
      cg = -t;
    }
    Cg[i][j] = cg;
  }
  store_row64(dkk + mat + i * GC, out);
  // ---- qk part
  load_row64(qkr + mat + i * GC, r1);
  load_row64(dqk + mat + i * GC, r2);
#pragma unroll
  for (int j = 0; j < GC; ++j) {
    out[j] = 0.f;
    if (j <= i) {
      const float e = __expf(gi - g_s[j]);
      out[j] = r2[j] * scale * e;
      const float t = out[j] * r1[j];
      dg_row += t;
      Cg[i][j] -= t;
    }
  }
  store_row64(dqkr + mat + i * GC, out);
  // ---- Tu / Tw part (column-indexed scalings)
  load_row64(dTu + mat + i * GC, r1);
  load_row64(dTw + mat + i * GC, r2);
  const float4* x4 = reinterpret_cast<const float4*>(X + mat + i * GC);
#pragma unroll
  for (int j = 0; j < GC / 4; ++j) {
    const float4 v = x4[j];
    out[4 * j] = v.x; out[4 * j + 1] = v.y; out[4 * j + 2] = v.z; out[4 * j + 3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < GC; ++j) {
    float cb = 0.f;
    if (j <= i) {
      const float eg = __expf(g_s[j]);
      const float xv = out[j];
      cb = (r1[j] + r2[j] * eg) * xv;
      Cg[i][j] += r2[j] * xv * b_s[j] * eg;
    }
    Cb[i][j] = cb;
  }
  __syncthreads();
  float dg_col = 0.f, db_col = 0.f;
#pragma unroll 8
  for (int r = 0; r < GC; ++r) { dg_col += Cg[r][i]; db_col += Cb[r][i]; }
  dgc[ch * GC + i] = dg_row + dg_col;
  dbeta[ch * GC + i] = db_row + db_col;
}

// ------------------------------------------------------------------------------------
// Rotary embedding, halves layout.  x (tokens T per batch, H heads, D); cos/sin (T, D/2).
// sign = +1 forward, -1 backward (rotation by the opposite angle).  In-place safe.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rope_kernel(const bf16* __restrict__ x, const float* __restrict__ cs,
                                                   const float* __restrict__ sn, bf16* __restrict__ y, long n_items,
                                                   int T, int H, int D, float sign) {
  const int d2v = D / 16;   // 8-wide vectors per half
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_items; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % d2v);
    const long bh = i / d2v;            // (b*T + t)*H + h
    const long bt = bh / H;
    const int t = static_cast<int>(bt % T);
    const bf16* px = x + bh * D + v * 8;
    float a[8], b[8], o1[8], o2[8];
    load8(px, a);
    load8(px + D / 2, b);
    const float* pc = cs + static_cast<long>(t) * (D / 2) + v * 8;
    const float* ps = sn + static_cast<long>(t) * (D / 2) + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = pc[j], s = ps[j] * sign;
      o1[j] = a[j] * c - b[j] * s;
      o2[j] = b[j] * c + a[j] * s;
    }
    bf16* py = y + bh * D + v * 8;
    store8(py, o1);
    store8(py + D / 2, o2);
  }
}

// ------------------------------------------------------------------------------------
// Causal depthwise conv1d, width W <= 4, channel-last (B, T, C), optional bias and SiLU.
// A CTA owns CT_C channels and walks CT_SEG consecutive tiles of CT_T time steps.  The rows of a
// tile reach shared memory through cp.async, the next tile's rows while the current tile is
// computed, so global loads are always in flight and never on a thread's dependency chain; the
// taps read shared memory.  Thread (rg, c8): 8 channels c8*8.., rows rg, rg+16, ... of the tile.
// ------------------------------------------------------------------------------------
constexpr int CT_T = 64, CT_C = 128, CT_SEG = 8, CT_THREADS = 256, CT_RG = CT_THREADS / (CT_C / 8);
constexpr int CONV_TCHUNK = CT_T * CT_SEG;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {   // zero fill when !pred
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int W>
__global__ void __launch_bounds__(CT_THREADS) conv1d_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                const bf16* __restrict__ bias, bf16* __restrict__ y,
                                                                int T, int C, long ldx, int act) {
  constexpr int XR = CT_T + W - 1;
  __shared__ __align__(16) bf16 sx[2][XR * CT_C];                // x rows t0-(W-1) .. t0+CT_T-1 of a tile
  const int c8 = threadIdx.x % (CT_C / 8), rg = threadIdx.x / (CT_C / 8);
  const int c = blockIdx.x * CT_C + c8 * 8;
  const long b = blockIdx.z;
  const bool c_ok = c < C;
  const int seg0 = blockIdx.y * CT_SEG;
  const int n_tiles = min(CT_SEG, (T + CT_T - 1) / CT_T - seg0);
  auto load_tile = [&](int n, int buf) {
    const int t0 = (seg0 + n) * CT_T;
    for (int i = rg; i < XR; i += CT_RG) {
      const int t = t0 - (W - 1) + i;
      const bool ok = c_ok && t >= 0 && t < T;
      cp_async16(sx[buf] + i * CT_C + c8 * 8, ok ? x + (b * T + t) * ldx + c : x, ok);
    }
    cp_async_commit();
  };
  load_tile(0, 0);
  float wv[W][8], bv[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    bv[k] = (bias && c_ok) ? __bfloat162float(bias[c + k]) : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) wv[j][k] = c_ok ? __bfloat162float(w[(c + k) * W + j]) : 0.f;
  }
  for (int n = 0; n < n_tiles; ++n) {
    const int buf = n & 1;
    if (n + 1 < n_tiles) { load_tile(n + 1, buf ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int t0 = (seg0 + n) * CT_T;
    if (c_ok) {
      for (int i = rg; i < CT_T; i += CT_RG) {
        const int t = t0 + i;
        if (t >= T) break;
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = bv[k];
#pragma unroll
        for (int j = 0; j < W; ++j) {
          float xv[8];
          unpack8(*reinterpret_cast<const uint4*>(sx[buf] + (i + j) * CT_C + c8 * 8), xv);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += wv[j][k] * xv[k];
        }
        if (act) {
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] = silu_f(o[k]);
        }
        store8(y + (b * T + t) * C + c, o);
      }
    }
    __syncthreads();                                // the buffer is refilled two tiles on
  }
}

// Backward: dpre[t] = dy[t] (times SiLU'(pre[t]), pre recomputed from x), dx[s] = sum_j w[j] dpre[s + (W-1) - j],
// dw[j] = sum_t dpre[t] x[t - (W-1) + j], db = sum_t dpre[t].  A tile needs dpre on CT_T + W - 1
// rows, hence x on CT_T + 2 (W - 1) rows.  Weight and bias gradients stay in registers over the
// CTA's tiles and leave as one partial sum per (time segment, batch): partial layout
// [chunk][W + 1][C] (row W = bias gradient), chunk = blockIdx.z * gridDim.y + blockIdx.y; each time
// step is counted by one tile only, and every sum runs in a fixed order.
template <int W>
__global__ void __launch_bounds__(CT_THREADS) conv1d_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                const bf16* __restrict__ bias, const bf16* __restrict__ dy,
                                                                bf16* __restrict__ dx, float* __restrict__ partial,
                                                                int T, int C, long ldx, int act) {
  constexpr int XR = CT_T + 2 * (W - 1), DR = CT_T + W - 1;
  extern __shared__ __align__(16) uint8_t conv_smem[];
  bf16* sx0 = reinterpret_cast<bf16*>(conv_smem);                // [2][XR][CT_C]  x rows t0-(W-1) ..
  bf16* sdy0 = sx0 + 2 * XR * CT_C;                              // [2][DR][CT_C]  dy rows t0 ..
  float* sdp = reinterpret_cast<float*>(sdy0 + 2 * DR * CT_C);   // [DR][CT_C]     dpre rows t0 ..
  float* sred = reinterpret_cast<float*>(conv_smem);             // [warps][W + 1][CT_C], over the x tiles once they are dead
  const int c8 = threadIdx.x % (CT_C / 8), rg = threadIdx.x / (CT_C / 8);
  const int c = blockIdx.x * CT_C + c8 * 8;
  const long b = blockIdx.z;
  const bool c_ok = c < C;
  const int seg0 = blockIdx.y * CT_SEG;
  const int n_tiles = min(CT_SEG, (T + CT_T - 1) / CT_T - seg0);
  auto load_tile = [&](int n, int buf) {
    const int t0 = (seg0 + n) * CT_T;
    bf16* sx = sx0 + buf * XR * CT_C;
    bf16* sdy = sdy0 + buf * DR * CT_C;
    for (int i = rg; i < XR; i += CT_RG) {
      const int t = t0 - (W - 1) + i;
      const bool ok = c_ok && t >= 0 && t < T;
      cp_async16(sx + i * CT_C + c8 * 8, ok ? x + (b * T + t) * ldx + c : x, ok);
    }
    for (int i = rg; i < DR; i += CT_RG) {
      const int t = t0 + i;
      const bool ok = c_ok && t < T;
      cp_async16(sdy + i * CT_C + c8 * 8, ok ? dy + (b * T + t) * C + c : dy, ok);
    }
    cp_async_commit();
  };
  load_tile(0, 0);
  float wv[W][8], bv[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    bv[k] = (bias && c_ok) ? __bfloat162float(bias[c + k]) : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) wv[j][k] = c_ok ? __bfloat162float(w[(c + k) * W + j]) : 0.f;
  }
  float dwacc[W][8], dbacc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    dbacc[k] = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) dwacc[j][k] = 0.f;
  }
  for (int n = 0; n < n_tiles; ++n) {
    const int buf = n & 1;
    const bf16* sx = sx0 + buf * XR * CT_C;
    const bf16* sdy = sdy0 + buf * DR * CT_C;
    if (n + 1 < n_tiles) { load_tile(n + 1, buf ^ 1); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    const int t0 = (seg0 + n) * CT_T;
    // ---- dpre (rows past T hold dy = 0, so their dpre is 0)
    for (int i = rg; i < DR; i += CT_RG) {
      float dv[8], dp[8];
      unpack8(*reinterpret_cast<const uint4*>(sdy + i * CT_C + c8 * 8), dv);
      if (act) {
        float pre[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) pre[k] = bv[k];
#pragma unroll
        for (int j = 0; j < W; ++j) {
          float xv[8];
          unpack8(*reinterpret_cast<const uint4*>(sx + (i + j) * CT_C + c8 * 8), xv);
#pragma unroll
          for (int k = 0; k < 8; ++k) pre[k] += wv[j][k] * xv[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) dp[k] = dv[k] * dsilu_f(pre[k]);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) dp[k] = dv[k];
      }
      float4* d4 = reinterpret_cast<float4*>(sdp + i * CT_C + c8 * 8);
      d4[0] = make_float4(dp[0], dp[1], dp[2], dp[3]);
      d4[1] = make_float4(dp[4], dp[5], dp[6], dp[7]);
    }
    __syncthreads();
    // ---- dx, and this thread's share of dw / db (its rows only)
    for (int i = rg; i < CT_T; i += CT_RG) {
      const int t = t0 + i;
      if (t >= T) break;
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = 0.f;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float4* d4 = reinterpret_cast<const float4*>(sdp + (i + (W - 1) - j) * CT_C + c8 * 8);
        const float4 a = d4[0], e = d4[1];
        const float dq[8] = {a.x, a.y, a.z, a.w, e.x, e.y, e.z, e.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] += wv[j][k] * dq[k];
      }
      if (c_ok) store8(dx + (b * T + t) * C + c, o);
      const float4* p4 = reinterpret_cast<const float4*>(sdp + i * CT_C + c8 * 8);
      const float4 a = p4[0], e = p4[1];
      const float dp[8] = {a.x, a.y, a.z, a.w, e.x, e.y, e.z, e.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) dbacc[k] += dp[k];
#pragma unroll
      for (int j = 0; j < W; ++j) {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4*>(sx + (i + j) * CT_C + c8 * 8), xv);
#pragma unroll
        for (int k = 0; k < 8; ++k) dwacc[j][k] += dp[k] * xv[k];
      }
    }
    __syncthreads();                                // sdp and this buffer are rewritten next
  }
  // ---- the two row groups of a warp meet by shuffle, the warps through shared memory, in a fixed order
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    dbacc[k] += __shfl_xor_sync(0xffffffffu, dbacc[k], 16);
#pragma unroll
    for (int j = 0; j < W; ++j) dwacc[j][k] += __shfl_xor_sync(0xffffffffu, dwacc[j][k], 16);
  }
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) < 16) {
#pragma unroll
    for (int j = 0; j <= W; ++j) {
      float4* d4 = reinterpret_cast<float4*>(sred + (warp * (W + 1) + j) * CT_C + c8 * 8);
      if (j < W) {
        d4[0] = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
        d4[1] = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
      } else {
        d4[0] = make_float4(dbacc[0], dbacc[1], dbacc[2], dbacc[3]);
        d4[1] = make_float4(dbacc[4], dbacc[5], dbacc[6], dbacc[7]);
      }
    }
  }
  __syncthreads();
  const long chunk = static_cast<long>(blockIdx.z) * gridDim.y + blockIdx.y;
  float* pp = partial + chunk * (W + 1) * C;
  for (int e = threadIdx.x; e < (W + 1) * CT_C; e += CT_THREADS) {
    const int j = e / CT_C, cc = e - j * CT_C;
    const int cg = blockIdx.x * CT_C + cc;
    if (cg >= C) continue;
    float acc = 0.f;
#pragma unroll
    for (int wi = 0; wi < CT_THREADS / 32; ++wi) acc += sred[(wi * (W + 1) + j) * CT_C + cc];
    pp[static_cast<long>(j) * C + cg] = acc;
  }
}

// ------------------------------------------------------------------------------------
// Embedding
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const long* __restrict__ ids, const bf16* __restrict__ w,
                                                            bf16* __restrict__ y, long n, int d, long vocab,
                                                            KernelStatus* status) {
  const int d8 = d / 8;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n * d8; i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long tok = i / d8;
    const int v = static_cast<int>(i - tok * d8);
    long id = ids[tok];
    if (v == 0) NSA_CHECK_INDEX(id >= 0 && id < vocab, status, id);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    *reinterpret_cast<uint4*>(y + tok * d + v * 8) = *reinterpret_cast<const uint4*>(w + id * d + v * 8);
  }
}
// ids sorted ascending with `perm` giving the original token position of each sorted entry.
// One CTA column per run start: sums the run's gradient rows in sorted order (deterministic).
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const long* __restrict__ sorted_ids,
                                                            const long* __restrict__ perm, const bf16* __restrict__ dy,
                                                            float* __restrict__ dw, long n, int d) {
  const long i = blockIdx.x;
  const long id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;   // not a run start
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (long j = i; j < n && sorted_ids[j] == id; ++j) {
      float v[8];
      load8(dy + perm[j] * d + c, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) dw[id * d + c + k] += acc[k];
  }
}

inline int grid_for(long n, int block, int per_sm = 8) {
  long g = (n + block - 1) / block;
  long cap = static_cast<long>(nsa::sm_count()) * per_sm;
  return static_cast<int>(g < cap ? (g < 1 ? 1 : g) : cap);
}

template <int MODE>
int launch_rms_fwd(const void* x, const void* g, const void* w, void* y, float* rstd, long rows, int d, float eps, cudaStream_t st,
                   long ldg = 0) {
  if (ldg == 0) ldg = d;
  if (ldg % 8 || (reinterpret_cast<uintptr_t>(g) & 15)) return nsa::fail(NSA_ERR_ALIGNMENT, "rmsnorm: gate rows must be 16-byte aligned");
  const bf16 *X = (const bf16*)x, *G = (const bf16*)g, *Wt = (const bf16*)w;
  bf16* Y = (bf16*)y;
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width must be a multiple of 8");
  if (d <= 256) rmsnorm_fwd_kernel<32, 1, MODE><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(X, G, Wt, Y, rstd, rows, d, eps, ldg);
  else if (d <= 512) rmsnorm_fwd_kernel<32, 2, MODE><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(X, G, Wt, Y, rstd, rows, d, eps, ldg);
  else if (d <= 2048) rmsnorm_fwd_kernel<256, 1, MODE><<<(unsigned)rows, 256, 0, st>>>(X, G, Wt, Y, rstd, rows, d, eps, ldg);
  else if (d <= 4096) rmsnorm_fwd_kernel<256, 2, MODE><<<(unsigned)rows, 256, 0, st>>>(X, G, Wt, Y, rstd, rows, d, eps, ldg);
  else if (d <= 8192) rmsnorm_fwd_kernel<256, 4, MODE><<<(unsigned)rows, 256, 0, st>>>(X, G, Wt, Y, rstd, rows, d, eps, ldg);
  else return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width above 8192 is not supported");
  nsa::count_launch();
  return 0;
}

template <int MODE>
int launch_rms_bwd(const void* x, const void* g, const void* w, const void* dy, const float* rstd, void* dx, void* dg,
                   float* partial, int grid, long rows, int d, cudaStream_t st, const void* dres = nullptr, long ldg = 0) {
  const bf16 *X = (const bf16*)x, *G = (const bf16*)g, *Wt = (const bf16*)w, *DY = (const bf16*)dy, *DR = (const bf16*)dres;
  bf16 *DX = (bf16*)dx, *DG = (bf16*)dg;
  if (d <= 256) rmsnorm_bwd_kernel<32, 1, MODE><<<grid, 256, 0, st>>>(X, G, Wt, DY, rstd, DX, DG, partial, rows, d, DR, ldg);
  else if (d <= 512) rmsnorm_bwd_kernel<32, 2, MODE><<<grid, 256, 0, st>>>(X, G, Wt, DY, rstd, DX, DG, partial, rows, d, DR, ldg);
  else if (d <= 2048) rmsnorm_bwd_kernel<256, 1, MODE><<<grid, 256, 0, st>>>(X, G, Wt, DY, rstd, DX, DG, partial, rows, d, DR, ldg);
  else if (d <= 4096) rmsnorm_bwd_kernel<256, 2, MODE><<<grid, 256, 0, st>>>(X, G, Wt, DY, rstd, DX, DG, partial, rows, d, DR, ldg);
  else if (d <= 8192) rmsnorm_bwd_kernel<256, 4, MODE><<<grid, 256, 0, st>>>(X, G, Wt, DY, rstd, DX, DG, partial, rows, d, DR, ldg);
  else return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width above 8192 is not supported");
  nsa::count_launch();
  return 0;
}

int launch_rms_add_fwd(const void* x, const void* r, const void* w, void* h, void* y, float* rstd, long rows, int d, float eps,
                       cudaStream_t st) {
  const bf16 *X = (const bf16*)x, *R = (const bf16*)r, *Wt = (const bf16*)w;
  bf16 *H = (bf16*)h, *Y = (bf16*)y;
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width must be a multiple of 8");
  if (d <= 256) rmsnorm_add_fwd_kernel<32, 1><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(X, R, Wt, H, Y, rstd, rows, d, eps);
  else if (d <= 512) rmsnorm_add_fwd_kernel<32, 2><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(X, R, Wt, H, Y, rstd, rows, d, eps);
  else if (d <= 2048) rmsnorm_add_fwd_kernel<256, 1><<<(unsigned)rows, 256, 0, st>>>(X, R, Wt, H, Y, rstd, rows, d, eps);
  else if (d <= 4096) rmsnorm_add_fwd_kernel<256, 2><<<(unsigned)rows, 256, 0, st>>>(X, R, Wt, H, Y, rstd, rows, d, eps);
  else if (d <= 8192) rmsnorm_add_fwd_kernel<256, 4><<<(unsigned)rows, 256, 0, st>>>(X, R, Wt, H, Y, rstd, rows, d, eps);
  else return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width above 8192 is not supported");
  nsa::count_launch();
  return 0;
}

}  // namespace

// mode: 0 plain, 1 norm-then-gate, 2 gate-then-norm.  rstd (rows) fp32 is written for backward.
extern "C" int nsa_rmsnorm_fwd(const void* x, const void* gate, const void* w, void* y, float* rstd, long rows, int d,
                               float eps, int mode, cudaStream_t st) {
  if (mode == 0) return launch_rms_fwd<0>(x, gate, w, y, rstd, rows, d, eps, st);
  if (mode == 1) return launch_rms_fwd<1>(x, gate, w, y, rstd, rows, d, eps, st);
  return launch_rms_fwd<2>(x, gate, w, y, rstd, rows, d, eps, st);
}

// Number of per-CTA partial rows the backward needs in `partial` (fp32 [parts, d]).
extern "C" int nsa_rmsnorm_bwd_parts(long rows, int d) {
  const int rows_per_cta = d <= 512 ? 8 : 1;
  long want = (rows + rows_per_cta - 1) / rows_per_cta;
  long cap = static_cast<long>(nsa::sm_count()) * 4;
  return static_cast<int>(want < cap ? want : cap);
}

// dw_bf16 / dw_f32: either may be null.  `partial` is caller-provided scratch of
// nsa_rmsnorm_bwd_parts(rows, d) * d floats.
extern "C" int nsa_rmsnorm_bwd(const void* x, const void* gate, const void* w, const void* dy, const float* rstd,
                               void* dx, void* dgate, void* dw_bf16, float* dw_f32, float* partial, long rows, int d,
                               int mode, cudaStream_t st) {
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width must be a multiple of 8");
  const int parts = nsa_rmsnorm_bwd_parts(rows, d);
  int rc;
  if (mode == 0) rc = launch_rms_bwd<0>(x, gate, w, dy, rstd, dx, dgate, partial, parts, rows, d, st);
  else if (mode == 1) rc = launch_rms_bwd<1>(x, gate, w, dy, rstd, dx, dgate, partial, parts, rows, d, st);
  else rc = launch_rms_bwd<2>(x, gate, w, dy, rstd, dx, dgate, partial, parts, rows, d, st);
  if (rc) return rc;
  reduce_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(partial, parts, d, (bf16*)dw_bf16, dw_f32);
  nsa::count_launch();
  return 0;
}

// Gated modes with the gate given as a column slice of a wider row-major matrix: `ldg` is the
// gate's row pitch in elements (a multiple of 8; the slice must start 16-byte aligned).  x, y, dx
// and dgate stay contiguous [rows, d].
extern "C" int nsa_rmsnorm_fwd_ldg(const void* x, const void* gate, long ldg, const void* w, void* y, float* rstd, long rows,
                                   int d, float eps, int mode, cudaStream_t st) {
  if (mode == 1) return launch_rms_fwd<1>(x, gate, w, y, rstd, rows, d, eps, st, ldg);
  if (mode == 2) return launch_rms_fwd<2>(x, gate, w, y, rstd, rows, d, eps, st, ldg);
  return nsa::fail(NSA_ERR_SHAPE, "nsa_rmsnorm_fwd_ldg: gated modes only");
}
extern "C" int nsa_rmsnorm_bwd_ldg(const void* x, const void* gate, long ldg, const void* w, const void* dy, const float* rstd,
                                   void* dx, void* dgate, void* dw_bf16, float* dw_f32, float* partial, long rows, int d,
                                   int mode, cudaStream_t st) {
  if (d % 8 || ldg % 8 || (reinterpret_cast<uintptr_t>(gate) & 15))
    return nsa::fail(NSA_ERR_ALIGNMENT, "rmsnorm: widths multiples of 8 and 16-byte aligned gate rows required");
  const int parts = nsa_rmsnorm_bwd_parts(rows, d);
  int rc;
  if (mode == 1) rc = launch_rms_bwd<1>(x, gate, w, dy, rstd, dx, dgate, partial, parts, rows, d, st, nullptr, ldg);
  else if (mode == 2) rc = launch_rms_bwd<2>(x, gate, w, dy, rstd, dx, dgate, partial, parts, rows, d, st, nullptr, ldg);
  else return nsa::fail(NSA_ERR_SHAPE, "nsa_rmsnorm_bwd_ldg: gated modes only");
  if (rc) return rc;
  reduce_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(partial, parts, d, (bf16*)dw_bf16, dw_f32);
  nsa::count_launch();
  return 0;
}

// h = x + r and y = rmsnorm(h) * w in one pass (plain mode).  x, r, h, y: [rows, d] bf16 contiguous.
extern "C" int nsa_rmsnorm_add_fwd(const void* x, const void* r, const void* w, void* h, void* y, float* rstd, long rows,
                                   int d, float eps, cudaStream_t st) {
  return launch_rms_add_fwd(x, r, w, h, y, rstd, rows, d, eps, st);
}

// Plain-mode backward that also adds `dres` (the gradient arriving at the norm's input through the
// residual stream, [rows, d] bf16) into dx.  `partial` as for nsa_rmsnorm_bwd.
extern "C" int nsa_rmsnorm_bwd_res(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                                   void* dx, void* dw_bf16, float* dw_f32, float* partial, long rows, int d,
                                   cudaStream_t st) {
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "rmsnorm: width must be a multiple of 8");
  const int parts = nsa_rmsnorm_bwd_parts(rows, d);
  const int rc = launch_rms_bwd<0>(x, nullptr, w, dy, rstd, dx, nullptr, partial, parts, rows, d, st, dres);
  if (rc) return rc;
  reduce_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(partial, parts, d, (bf16*)dw_bf16, dw_f32);
  nsa::count_launch();
  return 0;
}

// ------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc (or anything that may call it) at the
// point where they need a backward pass: an embedding runtime whose device-memory budget is
// fixed when the library is loaded, a worker thread that is forbidden to take the allocator
// lock, a latency-critical loop that cannot afford the implicit device synchronisation an
// allocation may cause.  nsa_rmsnorm_bwd needs a scratch buffer for the per-CTA partial
// sums of the weight gradient; this variant keeps that scratch in the library itself.
//
// The scratch is one file-scope device array of NSA_NOALLOC_SCRATCH_FLOATS floats
// (592 * 4096 floats = 9.25 MiB).  Every GPU that loads the library holds that much from load
// until process exit, whether or not this entry point is ever called.
// ------------------------------------------------------------------------------------
#define NSA_NOALLOC_SCRATCH_FLOATS (592 * 4096)
static __device__ __align__(256) float g_noalloc_scratch[NSA_NOALLOC_SCRATCH_FLOATS];

// Device address of g_noalloc_scratch per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use, so the address is looked up once
// per device with that device current.  The cache is filled without a lock: host threads that
// race on a device's first call all store the same value.
static float* g_noalloc_scratch_addr[64] = {nullptr};

static int noalloc_scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return nsa::fail_cuda(e, "nsa_rmsnorm_bwd_noalloc: cudaGetDevice");
  if (dev < 0 || dev >= 64) return nsa::fail(NSA_ERR_LIMIT, "nsa_rmsnorm_bwd_noalloc: device index above 63");
  if (g_noalloc_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess) return nsa::fail_cuda(e, "nsa_rmsnorm_bwd_noalloc: cudaGetSymbolAddress");
    g_noalloc_scratch_addr[dev] = ptr;
  }
  *out = g_noalloc_scratch_addr[dev];
  return 0;
}

// Same arguments and results as nsa_rmsnorm_bwd, minus `partial`.
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
//  * The first call on each device looks up the scratch address (a synchronous runtime
//    query); make that first call before any stream capture begins on that device.
//  * Limit: nsa_rmsnorm_bwd_parts(rows, d) * d must not exceed NSA_NOALLOC_SCRATCH_FLOATS
//    (true whenever sm_count * 4 * d <= 592 * 4096, e.g. d <= 4096 on a 148-SM part); larger
//    problems are rejected with NSA_ERR_LIMIT and
//    nothing is launched.
//  * All calls on a device share the one scratch array, which keeps whatever the previous
//    call left in it.  Nothing in it has to start at zero: the backward kernel overwrites
//    every (part, column) entry that the reduction then reads.  Two calls whose kernels can
//    overlap on the GPU (different streams, or concurrent host threads) race on the array;
//    serialise them on one stream.
extern "C" int nsa_rmsnorm_bwd_noalloc(const void* x, const void* gate, const void* w, const void* dy,
                                       const float* rstd, void* dx, void* dgate, void* dw_bf16, float* dw_f32,
                                       long rows, int d, int mode, cudaStream_t st) {
  if (rows <= 0 || d <= 0) return nsa::fail(NSA_ERR_SHAPE, "nsa_rmsnorm_bwd_noalloc: empty problem");
  const long need = static_cast<long>(nsa_rmsnorm_bwd_parts(rows, d)) * d;
  if (need > static_cast<long>(NSA_NOALLOC_SCRATCH_FLOATS))
    return nsa::fail(NSA_ERR_LIMIT,
                     "nsa_rmsnorm_bwd_noalloc: problem needs more than the 592*4096-float built-in scratch "
                     "(use nsa_rmsnorm_bwd with caller-provided scratch)");
  float* scratch = nullptr;
  const int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc) return rc;
  return nsa_rmsnorm_bwd(x, gate, w, dy, rstd, dx, dgate, dw_bf16, dw_f32, scratch, rows, d, mode, st);
}

extern "C" int nsa_l2norm_fwd(const void* x, void* y, float* rinv, long rows, int d, float eps, cudaStream_t st) {
  if (d % 8 || d > 512) return nsa::fail(NSA_ERR_SHAPE, "l2norm: width must be a multiple of 8, at most 512");
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (d <= 256) l2norm_fwd_kernel<1><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)y, rinv, rows, d, eps);
  else l2norm_fwd_kernel<2><<<grid, 256, 0, st>>>((const bf16*)x, (bf16*)y, rinv, rows, d, eps);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_l2norm_bwd(const void* y, const void* dy, const float* rinv, void* dx, long rows, int d, cudaStream_t st) {
  if (d % 8 || d > 512) return nsa::fail(NSA_ERR_SHAPE, "l2norm: width must be a multiple of 8, at most 512");
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (d <= 256) l2norm_bwd_kernel<1><<<grid, 256, 0, st>>>((const bf16*)y, (const bf16*)dy, rinv, (bf16*)dx, rows, d);
  else l2norm_bwd_kernel<2><<<grid, 256, 0, st>>>((const bf16*)y, (const bf16*)dy, rinv, (bf16*)dx, rows, d);
  nsa::count_launch();
  return 0;
}

// gate / up: [rows, cols] with row pitches ldg / ldu (elements, multiples of 8); y contiguous.
extern "C" int nsa_swiglu_fwd(const void* g, const void* u, void* y, long rows, int cols, long ldg, long ldu, cudaStream_t st) {
  if ((cols % 8) || (ldg % 8) || (ldu % 8)) return nsa::fail(NSA_ERR_SHAPE, "swiglu: sizes must be multiples of 8");
  const long n8 = rows * (cols / 8);
  swiglu_fwd_kernel<<<grid_for(n8, 256), 256, 0, st>>>((const bf16*)g, (const bf16*)u, (bf16*)y, n8, cols / 8, ldg / 8, ldu / 8);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, long rows, int cols,
                              long ldg, long ldu, long ldo, cudaStream_t st) {
  if ((cols % 8) || (ldg % 8) || (ldu % 8) || (ldo % 8)) return nsa::fail(NSA_ERR_SHAPE, "swiglu: sizes must be multiples of 8");
  const long n8 = rows * (cols / 8);
  swiglu_bwd_kernel<<<grid_for(n8, 256), 256, 0, st>>>((const bf16*)g, (const bf16*)u, (const bf16*)dy, (bf16*)dg, (bf16*)du,
                                                        n8, cols / 8, ldg / 8, ldu / 8, ldo / 8);
  nsa::count_launch();
  return 0;
}

// o, o1..o3: [rows, D] bf16 contiguous; g1..g3: [rows] bf16.  D in {64, 128, 256}.
extern "C" int nsa_gate_combine_fwd(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2,
                                    const void* g3, void* o, long rows, int D, cudaStream_t st) {
  if (D != 64 && D != 128 && D != 256) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: head_dim must be 64, 128 or 256");
  const long n8 = rows * (D / 8);
  const int grid = grid_for(n8, 256);
#define NSA_GC_FWD(L) gate_combine_fwd_kernel<L><<<grid, 256, 0, st>>>((const bf16*)o1, (const bf16*)o2, (const bf16*)o3, \
    (const bf16*)g1, (const bf16*)g2, (const bf16*)g3, (bf16*)o, n8, 1, 1L, 0)
  if (D == 64) NSA_GC_FWD(8); else if (D == 128) NSA_GC_FWD(16); else NSA_GC_FWD(32);
#undef NSA_GC_FWD
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_gate_combine_bwd(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2,
                                    const void* g3, const void* d_o, void* do1, void* do2, void* do3, void* dg1,
                                    void* dg2, void* dg3, long rows, int D, cudaStream_t st) {
  if (D != 64 && D != 128 && D != 256) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: head_dim must be 64, 128 or 256");
  const long n8 = rows * (D / 8);
  const long blocks = (n8 + 255) / 256;
  if (blocks > 2147483647L) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: problem too large for one launch");
#define NSA_GC_BWD(L) gate_combine_bwd_kernel<L><<<(unsigned)blocks, 256, 0, st>>>((const bf16*)o1, (const bf16*)o2, \
    (const bf16*)o3, (const bf16*)g1, (const bf16*)g2, (const bf16*)g3, (const bf16*)d_o, (bf16*)do1, (bf16*)do2, (bf16*)do3, \
    (bf16*)dg1, (bf16*)dg2, (bf16*)dg3, n8, 1, 1L, 0)
  if (D == 64) NSA_GC_BWD(8); else if (D == 128) NSA_GC_BWD(16); else NSA_GC_BWD(32);
#undef NSA_GC_BWD
  nsa::count_launch();
  return 0;
}

// The same with the three gates as columns of one [tokens, >= 3*Hq] bf16 matrix (row pitch ldg, the
// gate projection's output as it stands) and, with sig != 0, given as logits: the sigmoid and its
// derivative are applied here.  rows = tokens * Hq.  dg1..dg3 use the same pitch.
extern "C" int nsa_gate_combine_fwd_ex(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2,
                                       const void* g3, long ldg, int Hq, int sig, void* o, long rows, int D, cudaStream_t st) {
  if (D != 64 && D != 128 && D != 256) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: head_dim must be 64, 128 or 256");
  if (Hq <= 0 || rows % Hq) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: rows must be tokens * heads");
  const long n8 = rows * (D / 8);
  const int grid = grid_for(n8, 256);
#define NSA_GC_FWD(L) gate_combine_fwd_kernel<L><<<grid, 256, 0, st>>>((const bf16*)o1, (const bf16*)o2, (const bf16*)o3, \
    (const bf16*)g1, (const bf16*)g2, (const bf16*)g3, (bf16*)o, n8, Hq, ldg, sig)
  if (D == 64) NSA_GC_FWD(8); else if (D == 128) NSA_GC_FWD(16); else NSA_GC_FWD(32);
#undef NSA_GC_FWD
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_gate_combine_bwd_ex(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2,
                                       const void* g3, long ldg, int Hq, int sig, const void* d_o, void* do1, void* do2,
                                       void* do3, void* dg1, void* dg2, void* dg3, long rows, int D, cudaStream_t st) {
  if (D != 64 && D != 128 && D != 256) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: head_dim must be 64, 128 or 256");
  if (Hq <= 0 || rows % Hq) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: rows must be tokens * heads");
  const long n8 = rows * (D / 8);
  const long blocks = (n8 + 255) / 256;
  if (blocks > 2147483647L) return nsa::fail(NSA_ERR_SHAPE, "gate_combine: problem too large for one launch");
#define NSA_GC_BWD(L) gate_combine_bwd_kernel<L><<<(unsigned)blocks, 256, 0, st>>>((const bf16*)o1, (const bf16*)o2, \
    (const bf16*)o3, (const bf16*)g1, (const bf16*)g2, (const bf16*)g3, (const bf16*)d_o, (bf16*)do1, (bf16*)do2, (bf16*)do3, \
    (bf16*)dg1, (bf16*)dg2, (bf16*)dg3, n8, Hq, ldg, sig)
  if (D == 64) NSA_GC_BWD(8); else if (D == 128) NSA_GC_BWD(16); else NSA_GC_BWD(32);
#undef NSA_GC_BWD
  nsa::count_launch();
  return 0;
}

// Block mean pooling (see nsa_pool_fwd_kernel).  x: [B, T, width] bf16 with row pitch ldx; y: [B, nC, width]
// contiguous, nC = (T - block) / stride + 1.  dx is contiguous [B, T, width].
extern "C" int nsa_pool_fwd(const void* x, void* y, int B, int T, int width, long ldx, int block, int stride, cudaStream_t st) {
  if (width % 8 || ldx % 8 || T < block || block <= 0 || stride <= 0)
    return nsa::fail(NSA_ERR_SHAPE, "nsa_pool: width and pitch multiples of 8, T >= block required");
  const int nC = (T - block) / stride + 1;
  const long n = static_cast<long>(B) * nC * (width / 8);
  nsa_pool_fwd_kernel<<<grid_for(n, 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, T, nC, width / 8, ldx, block, stride, n);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_pool_bwd(const void* dy, void* dx, int B, int T, int width, int block, int stride, cudaStream_t st) {
  if (width % 8 || T < block || block <= 0 || stride <= 0)
    return nsa::fail(NSA_ERR_SHAPE, "nsa_pool: width multiple of 8, T >= block required");
  const int nC = (T - block) / stride + 1;
  const long n = static_cast<long>(B) * T * (width / 8);
  nsa_pool_bwd_kernel<<<grid_for(n, 256), 256, 0, st>>>((const bf16*)dy, (bf16*)dx, T, nC, width / 8, block, stride, n);
  nsa::count_launch();
  return 0;
}

// q, k: [B, T, H, 128]; v: [B, T, H, V] (V multiple of 8); sq, sk: [B*H, Tp] fp32;
// outputs [B*H, Tp, 128 or V] bf16.
extern "C" int nsa_gdn_pack_fwd(const void* q, const void* k, const void* v, const float* sq, const float* sk, void* qh,
                                void* kh, void* vh, void* qd, void* kt, int B, int T, int Tp, int H, int K, int V,
                                cudaStream_t st) {
  if (K != 128 || V % 8 || Tp < T) return nsa::fail(NSA_ERR_SHAPE, "gdn_pack: key width 128 and value width multiple of 8 required");
  const long rows = static_cast<long>(B) * H * Tp;
  gdn_pack_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, sq, sk, (bf16*)qh,
                                                                  (bf16*)kh, (bf16*)vh, (bf16*)qd, (bf16*)kt, B, T, Tp, H, V);
  nsa::count_launch();
  return 0;
}
// dqh, dkh, dvh, dqd, dkt may be null (treated as zero).  dq, dk, dv: token-major outputs; dsq, dsk: [B*H, Tp] fp32.
extern "C" int nsa_gdn_pack_bwd(const void* q, const void* k, const float* sq, const float* sk, const void* dqh,
                                const void* dkh, const void* dvh, const void* dqd, const void* dkt, void* dq, void* dk,
                                void* dv, float* dsq, float* dsk, int B, int T, int Tp, int H, int K, int V, cudaStream_t st) {
  if (K != 128 || V % 8 || Tp < T) return nsa::fail(NSA_ERR_SHAPE, "gdn_pack: key width 128 and value width multiple of 8 required");
  const long rows = static_cast<long>(B) * H * Tp;
  gdn_pack_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const bf16*)q, (const bf16*)k, sq, sk, (const bf16*)dqh,
                                                                  (const bf16*)dkh, (const bf16*)dvh, (const bf16*)dqd, (const bf16*)dkt,
                                                                  (bf16*)dq, (bf16*)dk, (bf16*)dv, dsq, dsk, B, T, Tp, H, V);
  nsa::count_launch();
  return 0;
}

// Per-chunk matrices of the gated delta rule; n_chunks = B*H*NC, every matrix 64 x 64 row-major.
extern "C" int nsa_gdn_tmat_fwd(const void* kk, const void* qkr, const float* gc, const float* beta, void* Tu, void* Tw,
                                void* qk, float* X, long n_chunks, float scale, cudaStream_t st) {
  if (n_chunks <= 0 || n_chunks > 2147483647L) return nsa::fail(NSA_ERR_SHAPE, "gdn_tmat: bad chunk count");
  gdn_tmat_fwd_kernel<<<(unsigned)n_chunks, 64, 0, st>>>((const bf16*)kk, (const bf16*)qkr, gc, beta, (bf16*)Tu, (bf16*)Tw,
                                                        (bf16*)qk, X, scale);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_gdn_tmat_dx(const void* dTu, const void* dTw, const float* gc, const float* beta, float* dX,
                               long n_chunks, cudaStream_t st) {
  if (n_chunks <= 0 || n_chunks > 2147483647L) return nsa::fail(NSA_ERR_SHAPE, "gdn_tmat: bad chunk count");
  gdn_tmat_dx_kernel<<<(unsigned)n_chunks, 64, 0, st>>>((const bf16*)dTu, (const bf16*)dTw, gc, beta, dX);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_gdn_tmat_bwd(const float* dA, const void* kk, const void* qkr, const void* dqk, const void* dTu,
                                const void* dTw, const float* X, const float* gc, const float* beta, void* dkk, void* dqkr,
                                float* dgc, float* dbeta, long n_chunks, float scale, cudaStream_t st) {
  if (n_chunks <= 0 || n_chunks > 2147483647L) return nsa::fail(NSA_ERR_SHAPE, "gdn_tmat: bad chunk count");
  gdn_tmat_bwd_kernel<<<(unsigned)n_chunks, 64, 0, st>>>(dA, (const bf16*)kk, (const bf16*)qkr, (const bf16*)dqk, (const bf16*)dTu,
                                                        (const bf16*)dTw, X, gc, beta, (bf16*)dkk, (bf16*)dqkr, dgc, dbeta, scale);
  nsa::count_launch();
  return 0;
}

// Head-major (B, H, Th, D) <-> token-major (B, Tt, H, D) copy of bf16 rows (D a multiple of 8); see the kernel.
extern "C" int nsa_permute_rows(const void* src, void* dst, int B, int H, int Th, int Tt, int D, int to_token, cudaStream_t st) {
  if (D % 8) return nsa::fail(NSA_ERR_SHAPE, "permute_rows: width must be a multiple of 8");
  const long rows = static_cast<long>(B) * H * (to_token ? Tt : Th);
  if (rows <= 0) return 0;
  permute_rows_kernel<<<grid_for(rows, 8, 16), 256, 0, st>>>((const bf16*)src, (bf16*)dst, B, H, Th, Tt, D, to_token);
  nsa::count_launch();
  return 0;
}

// in: [outer][parts][n] bf16 contiguous -> out: [outer][n] bf16 (n a multiple of 8).
extern "C" int nsa_sum_parts_bf16(const void* in, void* out, long outer, int parts, long n, cudaStream_t st) {
  if (n % 8 || parts <= 0) return nsa::fail(NSA_ERR_SHAPE, "sum_parts: width must be a multiple of 8");
  const long total = outer * (n / 8);
  sum_parts_bf16_kernel<<<grid_for(total, 256), 256, 0, st>>>((const bf16*)in, (bf16*)out, parts, n / 8, outer);
  nsa::count_launch();
  return 0;
}

extern "C" int nsa_rope(const void* x, const float* cos_t, const float* sin_t, void* y, long batch, int T, int H, int D,
                        int backward, cudaStream_t st) {
  if (D % 16) return nsa::fail(NSA_ERR_SHAPE, "rope: head_dim must be a multiple of 16");
  const long n = batch * T * H * (D / 16);
  rope_kernel<<<grid_for(n, 256), 256, 0, st>>>((const bf16*)x, cos_t, sin_t, (bf16*)y, n, T, H, D, backward ? -1.f : 1.f);
  nsa::count_launch();
  return 0;
}

extern "C" int nsa_conv1d_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int C, long ldx,
                              int width, int act, cudaStream_t st) {
  if (C % 8 || ldx % 8 || width != 4) return nsa::fail(NSA_ERR_SHAPE, "conv1d: channels multiple of 8 and width 4 required");
  dim3 grid((C + CT_C - 1) / CT_C, (T + CONV_TCHUNK - 1) / CONV_TCHUNK, B);
  conv1d_fwd_kernel<4><<<grid, CT_THREADS, 0, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)y, T, C, ldx, act);
  nsa::count_launch();
  return 0;
}
extern "C" long nsa_conv1d_bwd_parts(int B, int T) { return static_cast<long>(B) * ((T + CONV_TCHUNK - 1) / CONV_TCHUNK); }
// partial: scratch of parts * 5 * C floats.  dw_f32: [4*C] laid out [j][c]; db_f32: [C].
extern "C" int nsa_conv1d_bwd(const void* x, const void* w, const void* bias, const void* dy, void* dx, float* partial,
                              float* dwdb_f32, int B, int T, int C, long ldx, int width, int act, cudaStream_t st) {
  if (C % 8 || ldx % 8 || width != 4) return nsa::fail(NSA_ERR_SHAPE, "conv1d: channels multiple of 8 and width 4 required");
  dim3 grid((C + CT_C - 1) / CT_C, (T + CONV_TCHUNK - 1) / CONV_TCHUNK, B);
  constexpr int smem = 2 * (CT_T + 6) * CT_C * 2 + 2 * (CT_T + 3) * CT_C * 2 + (CT_T + 3) * CT_C * 4;
  static_assert((CT_THREADS / 32) * 5 * CT_C * 4 <= 2 * (CT_T + 6) * CT_C * 2, "conv1d: reduction scratch");
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(conv1d_bwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return nsa::fail_cuda(e, "conv1d_bwd: shared memory attribute");
    cfg = true;
  }
  conv1d_bwd_kernel<4><<<grid, CT_THREADS, smem, st>>>((const bf16*)x, (const bf16*)w, (const bf16*)bias, (const bf16*)dy, (bf16*)dx,
                                                       partial, T, C, ldx, act);
  const int parts = static_cast<int>(nsa_conv1d_bwd_parts(B, T));
  reduce_partials_kernel<<<(5 * C + 255) / 256, 256, 0, st>>>(partial, parts, 5 * C, nullptr, dwdb_f32);
  nsa::count_launch(2);
  return 0;
}

extern "C" int nsa_embedding_fwd(const long* ids, const void* w, void* y, long n, int d, long vocab, cudaStream_t st) {
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "embedding: width must be a multiple of 8");
  embedding_fwd_kernel<<<grid_for(n * (d / 8), 256), 256, 0, st>>>(ids, (const bf16*)w, (bf16*)y, n, d, vocab, nsa::status_ptr());
  nsa::count_launch();
  return 0;
}
// dw (fp32 [vocab, d]) must be zero-initialised by the caller; rows of absent ids stay zero.
extern "C" int nsa_embedding_bwd(const long* sorted_ids, const long* perm, const void* dy, float* dw, long n, int d, cudaStream_t st) {
  if (d % 8) return nsa::fail(NSA_ERR_SHAPE, "embedding: width must be a multiple of 8");
  embedding_bwd_kernel<<<(unsigned)n, 256, 0, st>>>(sorted_ids, perm, (const bf16*)dy, dw, n, d);
  nsa::count_launch();
  return 0;
}
