/* Public C interface of libnsa_b200.so (sm_100a).  Every function takes device pointers,
 * sizes and a CUDA stream, launches asynchronously on that stream and returns 0 on success
 * or an NSA_ERR_* code (text from nsa_last_error()).  Unless a function says otherwise, it
 * allocates nothing: outputs and scratch buffers are provided by the caller.
 * bf16 tensors are row-major; "ld" arguments are row pitches in elements. */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* nsa_last_error(void);
long long nsa_launch_count(void);
void nsa_launch_count_reset(void);
int nsa_status_read(int* out4, int reset);   /* {code, block, info, count}; see status.cuh */
int nsa_sm_count(void);

/* C[M,N] = op(A) op(B), fp32 accumulate on tcgen05 tensor cores.  a_mn/b_mn select the
 * storage of each operand (0: reduction dimension contiguous, 1: M resp. N contiguous). */
int nsa_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                  int a_mn, int b_mn, int out_fp32, int accumulate, int max_ctas, cudaStream_t stream);

/* mode 0: y = rmsnorm(x) w; 1: rmsnorm(x) w silu(gate); 2: rmsnorm(x silu(gate)) w. */
int nsa_rmsnorm_fwd(const void* x, const void* gate, const void* w, void* y, float* rstd, long rows, int d,
                    float eps, int mode, cudaStream_t st);
int nsa_rmsnorm_bwd_parts(long rows, int d);
/* partial: scratch of nsa_rmsnorm_bwd_parts(rows, d) * d floats. */
int nsa_rmsnorm_bwd(const void* x, const void* gate, const void* w, const void* dy, const float* rstd, void* dx,
                    void* dgate, void* dw_bf16, float* dw_f32, float* partial, long rows, int d, int mode,
                    cudaStream_t st);
/* RMSNorm backward that allocates nothing and takes no scratch argument: the partial-sum
 * scratch is a 9.25 MiB array built into the library (held by every GPU that loads it).
 * For hosts that may not call cudaMalloc where they run the backward pass.  Rejects
 * problems with nsa_rmsnorm_bwd_parts(rows, d) * d > 592 * 4096 (NSA_ERR_LIMIT).  First call
 * per device does a one-time address lookup: make it before any stream capture.  Calls
 * share the scratch: do not let two of them overlap on the GPU.
 * This entry point has no counterpart in the reference project. */
int nsa_rmsnorm_bwd_noalloc(const void* x, const void* gate, const void* w, const void* dy, const float* rstd,
                            void* dx, void* dgate, void* dw_bf16, float* dw_f32, long rows, int d, int mode,
                            cudaStream_t st);
int nsa_l2norm_fwd(const void* x, void* y, float* rinv, long rows, int d, float eps, cudaStream_t st);
int nsa_l2norm_bwd(const void* y, const void* dy, const float* rinv, void* dx, long rows, int d, cudaStream_t st);
int nsa_swiglu_fwd(const void* g, const void* u, void* y, long rows, int cols, long ldg, long ldu, cudaStream_t st);
int nsa_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, long rows, int cols, long ldg,
                   long ldu, long ldo, cudaStream_t st);
int nsa_rope(const void* x, const float* cos_t, const float* sin_t, void* y, long batch, int T, int H, int D,
             int backward, cudaStream_t st);
int nsa_conv1d_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int C, long ldx, int width,
                   int act, cudaStream_t st);
long nsa_conv1d_bwd_parts(int B, int T);
int nsa_conv1d_bwd(const void* x, const void* w, const void* bias, const void* dy, void* dx, float* partial,
                   float* dwdb_f32, int B, int T, int C, long ldx, int width, int act, cudaStream_t st);
int nsa_embedding_fwd(const long* ids, const void* w, void* y, long n, int d, long vocab, cudaStream_t st);
int nsa_embedding_bwd(const long* sorted_ids, const long* perm, const void* dy, float* dw, long n, int d, cudaStream_t st);

int nsa_adamw_step(void* p, const void* g, float* m, float* v, float* master, const float* grad_scale, long n,
                   int p_fp32, int g_fp32, int step, float lr, float b1, float b2, float eps, float wd, cudaStream_t st);
int nsa_adamw8bit_step(void* p, const void* g, uint8_t* mq, float* mabs, uint8_t* vq, float* vabs,
                       const float* cb_signed, const float* cb_unsigned, const float* grad_scale, long n, int p_fp32,
                       int g_fp32, int step, float lr, float b1, float b2, float eps, float wd, cudaStream_t st);
int nsa_sumsq_parts(void);
int nsa_sumsq(const void* g, long n, int g_fp32, float* partial, float* out, int accumulate, cudaStream_t st);
int nsa_cross_entropy(void* logits, const long* labels, float* loss_rows, const float* inv_count, long rows, int V,
                      long ld, long ignore_index, int write_grad, cudaStream_t st);

#ifdef __cplusplus
}
#endif
