// Sequential scan of the experimental complex-state SSM block ("Mamba-3"), forward only, as in
// the reference (models/mamba.py:204-345: a Triton kernel on a (batch, heads) grid that walks
// the sequence).  One CTA per (batch, head); thread n keeps the complex state h[n] in registers.
//   z = A dt / 2;  Abar = (1 + z) / (1 - z);  Bbar = B dt / (1 - z)
//   h <- Abar h + Bbar u_t          (u_t = sum over the head's channels of x_t)
//   g_t = Re sum_n C_t[n] h[n] + D  (the caller multiplies x_t by g_t)
// The next step's operands are fetched before the current step's arithmetic, so the only serial
// cost per step is the state update and one CTA-wide reduction.
#include "host.cuh"

namespace {
__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
__device__ __forceinline__ float2 cdiv(float2 a, float2 b) {
  const float inv = 1.f / (b.x * b.x + b.y * b.y);
  return make_float2((a.x * b.x + a.y * b.y) * inv, (a.y * b.x - a.x * b.y) * inv);
}

// u, dt: [B, L, H]; A: [H, N] complex; Bc, Cc: [B, L, H, N] complex; D: [H]; gate out: [B, L, H]
__global__ void __launch_bounds__(256) mamba3_scan_kernel(const float* __restrict__ u, const float* __restrict__ dt,
                                                          const float2* __restrict__ A, const float2* __restrict__ Bc,
                                                          const float2* __restrict__ Cc, const float* __restrict__ D,
                                                          float* __restrict__ gate, int L, int H, int N) {
  __shared__ float red[2][8];
  const int b = blockIdx.y, h = blockIdx.x, n = threadIdx.x;
  const bool live = n < N;
  const float2 a = live ? A[h * N + n] : make_float2(0.f, 0.f);
  const float dh = D[h];
  float2 st = make_float2(0.f, 0.f);
  const long bl0 = static_cast<long>(b) * L;
  long row = bl0 * H + h;
  float u_n = u[row], dt_n = dt[row];
  float2 b_n = live ? Bc[row * N + n] : make_float2(0.f, 0.f);
  float2 c_n = live ? Cc[row * N + n] : make_float2(0.f, 0.f);
  const int warps = (blockDim.x + 31) >> 5;
  for (int t = 0; t < L; ++t) {
    const float ut = u_n, dtt = dt_n;
    const float2 bt = b_n, ct = c_n;
    const long cur = row;
    if (t + 1 < L) {
      row += H;
      u_n = u[row]; dt_n = dt[row];
      if (live) { b_n = Bc[row * N + n]; c_n = Cc[row * N + n]; }
    }
    const float2 z = make_float2(a.x * dtt * 0.5f, a.y * dtt * 0.5f);
    const float2 den = make_float2(1.f - z.x, -z.y);
    const float2 abar = cdiv(make_float2(1.f + z.x, z.y), den);
    const float2 bbar = cdiv(make_float2(bt.x * dtt, bt.y * dtt), den);
    const float2 ah = cmul(abar, st);
    st = make_float2(ah.x + bbar.x * ut, ah.y + bbar.y * ut);
    float yr = live ? ct.x * st.x - ct.y * st.y : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) yr += __shfl_xor_sync(0xffffffffu, yr, o);
    float* r = red[t & 1];                    // two buffers: one barrier per step is enough
    if ((n & 31) == 0) r[n >> 5] = yr;
    __syncthreads();
    if (n == 0) {
      float s = dh;
      for (int wv = 0; wv < warps; ++wv) s += r[wv];
      gate[cur] = s;
    }
  }
}
}  // namespace

extern "C" int nsa_mamba3_scan(const float* u, const float* dt, const float* A, const float* Bc, const float* Cc,
                               const float* D, float* gate, int B, int L, int H, int N, cudaStream_t st) {
  if (N <= 0 || N > 256) return nsa::fail(NSA_ERR_SHAPE, "mamba3_scan: d_state must be in 1..256");
  if (B <= 0 || L <= 0 || H <= 0) return nsa::fail(NSA_ERR_SHAPE, "mamba3_scan: empty problem");
  const int threads = ((N + 31) / 32) * 32;
  mamba3_scan_kernel<<<dim3(H, B), threads, 0, st>>>(u, dt, (const float2*)A, (const float2*)Bc, (const float2*)Cc, D, gate, L, H, N);
  nsa::count_launch();
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_mamba3_scan launch");
}
