// Mamba-2 SSD: inter-chunk state passing.  The chunk-local end states S_c (fp32) and the chunk
// decays gamma_c are produced by the batched per-chunk pass; this kernel runs the recurrence
//     Hprev_0 = 0,   Hprev_{c+1} = gamma_c * Hprev_c + S_c
// for every (batch, head, state element) in one launch, and its reverse for the backward:
//     g_c = dHprev_c + gamma_c * g_{c+1}   (g_{nc} = 0),   dS_c = g_{c+1}.
// Layout: S, Hprev, dHprev, dS are [B, nc, H, E] (E = headdim * d_state), gamma is [B, nc, H].
// One thread per (b, h, e); consecutive threads touch consecutive e, so every access is
// coalesced and each element is read and written exactly once.
#include "host.cuh"

namespace {
__global__ void __launch_bounds__(256) ssd_state_fwd_kernel(const float* __restrict__ S, const float* __restrict__ gamma,
                                                            float* __restrict__ Hprev, float* __restrict__ Hlast,
                                                            int nc, int H, long E) {
  const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int h = blockIdx.y, b = blockIdx.z;
  float st = 0.f;
  for (int c = 0; c < nc; ++c) {
    const long bch = (static_cast<long>(b) * nc + c) * H + h;
    Hprev[bch * E + e] = st;
    st = gamma[bch] * st + S[bch * E + e];
  }
  if (Hlast) Hlast[(static_cast<long>(b) * H + h) * E + e] = st;
}
__global__ void __launch_bounds__(256) ssd_state_bwd_kernel(const float* __restrict__ dHprev, const float* __restrict__ gamma,
                                                            float* __restrict__ dS, int nc, int H, long E) {
  const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const int h = blockIdx.y, b = blockIdx.z;
  float g = 0.f;
  for (int c = nc - 1; c >= 0; --c) {
    const long bch = (static_cast<long>(b) * nc + c) * H + h;
    dS[bch * E + e] = g;
    g = dHprev[bch * E + e] + gamma[bch] * g;
  }
}
}  // namespace

extern "C" int nsa_ssd_state_fwd(const float* S, const float* gamma, float* Hprev, float* Hlast, int B, int nc, int H,
                                 long E, cudaStream_t st) {
  dim3 grid((unsigned)((E + 255) / 256), H, B);
  ssd_state_fwd_kernel<<<grid, 256, 0, st>>>(S, gamma, Hprev, Hlast, nc, H, E);
  nsa::count_launch();
  return 0;
}
extern "C" int nsa_ssd_state_bwd(const float* dHprev, const float* gamma, float* dS, int B, int nc, int H, long E,
                                 cudaStream_t st) {
  dim3 grid((unsigned)((E + 255) / 256), H, B);
  ssd_state_bwd_kernel<<<grid, 256, 0, st>>>(dHprev, gamma, dS, nc, H, E);
  nsa::count_launch();
  return 0;
}
