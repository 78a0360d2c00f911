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
// bf16 rows between head-major (B, H, Th, D) and token-major (B, Tt, H, D); to_token 1: head -> token (t < Th copied),
// 0: token -> head (rows t >= Tt zeroed).
int nsa_permute_rows(const void* src, void* dst, int B, int H, int Th, int Tt, int D, int to_token, cudaStream_t st);
// out[o][i] = sum over p of in[o][p][i]; bf16 in and out, fp32 sums in ascending p; n a multiple of 8.
int nsa_sum_parts_bf16(const void* in, void* out, long outer, int parts, long n, cudaStream_t st);
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

/* ---- attention family: (B, T, H, D) bf16 tensors, L = log2-sum-exp per row (csrc/attention.cu) ---- */
int nsa_attn_fwd(const void* q, const void* k, const void* v, void* o, float* L, int B, int T, int S, int Hq, int
    Hkv, int D, float scale, int causal, int window, int kp_stride, int kp_off, const int* tile_blocks, const unsigned
    long long* tile_masks, const int* tile_counts, int max_u, cudaStream_t st);
int nsa_attn_importance(const void* q, const void* k_cmp, const float* L_in, float* imp, int B, int T, int S, int Hq,
    int Hkv, int D, float scale, int kp_stride, int kp_off, int nS, cudaStream_t st);
int nsa_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* L, float*
    delta, void* dq, float* dk, float* dv, int B, int T, int S, int Hq, int Hkv, int D, float scale, int causal, int
    window, int kp_stride, int kp_off, const int* tile_blocks, const unsigned long long* tile_masks, const int*
    tile_counts, int max_u, cudaStream_t st);
int nsa_attn_bwd_split(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* L,
    float* delta, void* dq, float* dk, float* dv, int B, int T, int S, int Hq, int Hkv, int D, float scale, int causal,
    int window, int kp_stride, int kp_off, const int* tile_blocks, const unsigned long long* tile_masks, const int*
    tile_counts, int max_u, const int* tok_list, const int* list_start, const int* item_start, int nS, int item_bound,
    int visits_per_cta, cudaStream_t st);
int nsa_union_blocks(const int* idx, int* tile_blocks, unsigned long long* tile_masks, int* tile_counts, int B, int
    T, int Hkv, int G, int top_n, int nS, int max_u, cudaStream_t st);

/* ---- peer-memory collectives and the IPC arena (csrc/comm.cu) ---- */
int nsa_enable_peer_access(int peer_device);
int nsa_comm_signal(unsigned* const* flag_rows, int W, int slot, unsigned epoch, cudaStream_t st);
int nsa_comm_wait(const unsigned* flags, int n, unsigned epoch, long long max_cycles, cudaStream_t st);
int nsa_comm_allgather(const void* const* shards, void* out, long shard_bytes, int W, int rank, const unsigned*
    flags, unsigned epoch, long long max_cycles, int ctas_per_peer, cudaStream_t st);
int nsa_comm_reduce_scatter_parts(void);
int nsa_comm_reduce_scatter(const float* const* grads, float* grad_shard, long S, int W, int rank, float scale, int
    accumulate, float* sumsq_partial, const unsigned* flags, unsigned epoch, long long max_cycles, cudaStream_t st);
int nsa_comm_rs_adamw8bit(const float* const* grads, void* p_shard, int p_fp32, uint8_t* mq, float* mabs, uint8_t*
    vq, float* vabs, const float* cb_signed, const float* cb_unsigned, const uint8_t* wd_mask, long S, int W, int rank,
    float scale, int step, float lr, float b1, float b2, float eps, float wd, const unsigned* flags, unsigned epoch, long
    long max_cycles, cudaStream_t st);
int nsa_ipc_alloc(long nbytes, void** out_ptr, unsigned char* handle64);
int nsa_ipc_open(const unsigned char* handle64, void** out_ptr);
int nsa_ipc_close(void* p);
int nsa_ipc_free(void* p);

/* ---- more element-wise kernels (csrc/elementwise.cu) ---- */
int nsa_gate_combine_fwd(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2, const void*
    g3, void* o, long rows, int D, cudaStream_t st);
int nsa_gate_combine_bwd(const void* o1, const void* o2, const void* o3, const void* g1, const void* g2, const void*
    g3, const void* d_o, void* do1, void* do2, void* do3, void* dg1, void* dg2, void* dg3, long rows, int D, cudaStream_t
    st);

/* ---- Gated DeltaNet state recurrence (csrc/gdn.cu) ---- */
int nsa_gdn_seq_fwd(const void* w, const void* qd, const void* kt, const void* u, const float* gamma, void* v_new,
    void* o_inter, void* S_all, int BH, int NC, int K, int V, cudaStream_t st);   /* o_inter: bf16 */
int nsa_gdn_seq_bwd(const void* w, const void* qd, const void* kt, const void* S_all, const void* v_new, const void*
    dv_new, const void* d_o, const float* gamma, void* du, void* dw_part, void* dqd_part, void* dkt_part, float*
    dgamma_part, int BH, int NC, int K, int V, cudaStream_t st);

/* ---- GEMM (csrc/gemm.cu) ---- */
int nsa_gemm_bf16_ag(const void* A, void* C, int M, int N, int K, int lda, int ldc, const void* const* shards, void*
    full, long shard_elems, long b_elem_offset, int W, int rank, unsigned* chunk_flags, int chunks_per_shard, const
    unsigned* peer_flags, unsigned epoch, long long max_cycles, int copy_ctas, cudaStream_t stream);

/* ---- forward-only scan of the complex-state block (csrc/mamba3.cu) ---- */
int nsa_mamba3_scan(const float* u, const float* dt, const float* A, const float* Bc, const float* Cc, const float*
    D, float* gate, int B, int L, int H, int N, cudaStream_t st);

/* ---- Mamba-2 SSD chunk kernels (csrc/ssd.cu) ---- */
int nsa_ssd_state_fwd(const float* S, const float* gamma, float* Hprev, void* Hprev_bf16, float* Hlast, int B, int
    nc, int H, long E, cudaStream_t st);
int nsa_ssd_state_bwd(const float* dHprev, const float* gamma, float* dS, void* dS_bf16, int B, int nc, int H, long
    E, cudaStream_t st);
int nsa_ssd_chunk_state(int mode, const void* bc, long ld_bc, const void* v, long ld_v, const float* dt, const float*
    A, float* S_out, float* gamma_out, int B, int T, int H, int N, int P, cudaStream_t st);
int nsa_ssd_chunk_out(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x, const void*
    Hprev_bf16, const float* dt, const float* A, const float* Dskip, void* y, int B, int T, int H, int N, int P,
    cudaStream_t st);
int nsa_ssd_chunk_grad(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x, const void*
    dy, const void* y, const void* Hprev_bf16, const void* dHn_bf16, const float* dt, const float* A, const float* Dskip,
    void* dx, float* dB_acc, float* dC_acc, float* q_out, float* k_out, int B, int T, int H, int N, int P, cudaStream_t
    st);

/* ---- further entry points of attention.cu ---- */
int nsa_select_blocks(const float* imp, int* idx, long rows, int T, int nS, int sel_block, int top_n, cudaStream_t
    st);

/* ---- further entry points of elementwise.cu ---- */
int nsa_gdn_pack_fwd(const void* q, const void* k, const void* v, const float* sq, const float* sk, void* qh, void*
    kh, void* vh, void* qd, void* kt, int B, int T, int Tp, int H, int K, int V, cudaStream_t st);
int nsa_gdn_pack_bwd(const void* q, const void* k, const float* sq, const float* sk, const void* dqh, const void*
    dkh, const void* dvh, const void* dqd, const void* dkt, void* dq, void* dk, void* dv, float* dsq, float* dsk, int B,
    int T, int Tp, int H, int K, int V, cudaStream_t st);
int nsa_gdn_tmat_fwd(const void* kk, const void* qkr, const float* gc, const float* beta, void* Tu, void* Tw, void*
    qk, float* X, long n_chunks, float scale, cudaStream_t st);
int nsa_gdn_tmat_dx(const void* dTu, const void* dTw, const float* gc, const float* beta, float* dX, long n_chunks,
    cudaStream_t st);
int nsa_gdn_tmat_bwd(const float* dA, const void* kk, const void* qkr, const void* dqk, const void* dTu, const void*
    dTw, const float* X, const float* gc, const float* beta, void* dkk, void* dqkr, float* dgc, float* dbeta, long
    n_chunks, float scale, cudaStream_t st);

/* ---- further entry points of optim.cu ---- */
int nsa_affine_quant(const float* t, uint8_t* q, float* scale, float* zero, long rows, int cols, int q_block, int
    bits, cudaStream_t st);
int nsa_affine_dequant(const uint8_t* q, const float* scale, const float* zero, float* out, long rows, int cols, int
    q_block, cudaStream_t st);

/* ---- further entry points of runtime.cu ---- */
int nsa_copy2d(void* dst, long dst_pitch_bytes, const void* src, long src_pitch_bytes, long width_bytes, long rows,
    cudaStream_t st);

/* ---- further entry points of ssd.cu ---- */
int nsa_ssd_chunk_grad_heads(const void* Cm, long ld_c, const void* Bm, long ld_b, const void* x, long ld_x, const
    void* dy, const void* y, const void* Hprev_bf16, const void* dHn_bf16, const float* dt, const float* A, const float*
    Dskip, void* dx, void* dB_heads, void* dC_heads, float* q_out, float* k_out, float* r_out, int B, int T, int H, int
    N, int P, cudaStream_t st);

#ifdef __cplusplus
}
#endif
