// C ABI of the sm_100a kernel library (libpfeife_b200_kernels.so).  Every entry point takes raw
// device pointers plus a CUDA stream handle (as void*), launches asynchronously on that stream
// and returns 0, a positive cudaError_t, or a negative argument error:
//   -1 unsupported dtype, -2 misaligned pointer / pitch, -3 size beyond a kernel limit,
//   -100/-101 tensor-map encoding failed.
// dtype codes: 0 = fp32, 1 = fp16, 2 = bf16.
#pragma once
#ifdef __cplusplus
#define PF_DECL extern "C"
#else
#define PF_DECL
#endif

// ---- device.cu
PF_DECL int pf_bind_device(int device);
PF_DECL int pf_device_count();

// ---- gemm_sm100.cu : C[M,N] = epi(alpha * A . B^T), tcgen05 / TMEM / TMA
PF_DECL int pf_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn, int b_mn, int in_dtype, int out_dtype,
                    const void* bias, int bias_dtype, const void* residual, long long ldr,
                    void* aux, long long ldaux, int epilogue, int accumulate, float alpha,
                    int* status, int sm_count, int tile_n, void* stream);

// ---- elementwise.cu
PF_DECL int pf_elementwise(const void* a, const void* b, void* out, long long n, int op, int dtype,
                           int sm_count, void* stream);
PF_DECL int pf_glu_fwd(const void* gu, void* out, long long rows, int H, int gelu, int dtype,
                       int sm_count, void* stream);
PF_DECL int pf_glu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int H,
                       int gelu, int dtype, int sm_count, void* stream);
PF_DECL int pf_axpy_f32(void* dst, const void* src, long long n, float scale, int accumulate,
                        int src_dtype, int sm_count, void* stream);
PF_DECL int pf_cast(const void* src, void* dst, long long n, int src_dtype, int dst_dtype,
                    int sm_count, void* stream);
PF_DECL int pf_colsum(const void* x, void* out_f32, long long rows, int cols, long long ld,
                      int dtype, int sm_count, void* stream);
PF_DECL int pf_transpose16(const void* src, void* dst, int rows, int cols, long long ld_src,
                           long long ld_dst, void* stream);

// ---- norm.cu
PF_DECL int pf_norm_fwd(const void* x, const void* res, const void* gamma, const void* beta,
                        void* y, void* h_out, void* mean, void* rstd, long long rows, int N,
                        float eps, int rms, int dtype, void* stream);
PF_DECL int pf_norm_bwd_ctas(long long rows, int sm_count);
PF_DECL int pf_norm_bwd(const void* dy, const void* h, const void* gamma, const void* mean,
                        const void* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                        void* scratch, long long rows, int N, int rms, int accumulate, int dtype,
                        int sm_count, void* stream);

// ---- optim.cu
PF_DECL int pf_nonfinite(const void* g, long long n, void* found_inf, int sm_count, void* stream);
PF_DECL int pf_adamw(void* p, void* g, void* m, void* v, void* lp, long long n,
                     const void* found_inf, const void* loss_scale, float lr, float beta1,
                     float beta2, float eps, float weight_decay, int step,
                     const void* applied_steps, float grad_scale, int adamw, int zero_grad,
                     int lp_dtype, int sm_count, void* stream);
PF_DECL int pf_step_advance(void* applied_steps, const void* found_inf, void* stream);
PF_DECL int pf_sgd(void* p, void* g, void* mom, void* lp, long long n, const void* found_inf,
                   const void* loss_scale, float lr, float momentum, float dampening,
                   float weight_decay, int nesterov, int first_step, float grad_scale,
                   int zero_grad, int lp_dtype, int sm_count, void* stream);
PF_DECL int pf_loss_scale_update(void* state, void* found_inf, float growth, float backoff,
                                 int interval, void* stream);

// ---- loss_embed.cu
PF_DECL int pf_ce_fwd(const void* logits, const void* target, void* loss, void* lse,
                      long long rows, int V, long long ld, long long ignore_index, int dtype,
                      void* stream);
PF_DECL int pf_ce_bwd(const void* logits, const void* target, const void* lse, const void* gscale,
                      void* dlogits, long long rows, int V, long long ld, long long ignore_index,
                      int dtype, void* stream);
PF_DECL int pf_mse_fwd(const void* a, const void* b, void* out_f32, long long n, int dtype,
                       int sm_count, void* stream);
PF_DECL int pf_mse_bwd(const void* a, const void* b, const void* gout_f32, void* da, long long n,
                       int dtype, int sm_count, void* stream);
PF_DECL int pf_embed_fwd(const void* table, const void* ids, void* out, long long tokens, int D,
                         long long vocab, int table_dtype, int out_dtype, void* stream);
PF_DECL int pf_embed_bwd(const void* dout, const void* ids, void* dtable_f32, long long tokens,
                         int D, long long vocab, int dtype, void* stream);
PF_DECL int pf_rope(const void* x, void* out, const void* cos_t, const void* sin_t, long long B,
                    int S, int H, int D, long long stride_b, long long stride_s,
                    long long stride_h, int inverse, int dtype, int sm_count, void* stream);

// ---- attn_sm100.cu : flash attention on tcgen05 (strides in elements: batch, seq, head)
PF_DECL int pf_attn_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int B,
                        int H, int Sq, int Sk, int D, const long long* sq, const long long* sk,
                        const long long* sv, int causal, float scale, int dtype, int* status,
                        void* stream);
PF_DECL int pf_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                        const void* out, const void* lse, void* delta, void* dq_accum, void* dq,
                        void* dk, void* dv, int B, int H, int Sq, int Sk, int D,
                        const long long* sq, const long long* sk, const long long* sv,
                        const long long* sdq, const long long* sdkv, int causal, float scale,
                        int dtype, int* status, int sm_count, void* stream);

// ---- dp_fused.cu : reduce-scatter + AdamW + all-gather over NVLink peer memory, IPC plumbing
PF_DECL int pf_dp_fused_step(int rank, int world, void* const* grad, void* const* master,
                             void* const* lp, void* const* flags, void* m, void* v,
                             void* local_sync, long long shard_lo, long long shard_hi,
                             long long total, int ngroups, const long long* groups,
                             const float* hyper, const void* applied_steps, int host_step,
                             float grad_scale, int lp_dtype, int check_inf, int found_given,
                             const void* loss_scale, void* found_inf, int epoch,
                             int arrivals_before, int* barriers_out, int* grid_out, int* status,
                             void* trace, int sm_count, void* stream);
PF_DECL int pf_gather_rows(void* dst, void* const* copies, const int* row_end, int world, int rank,
                           int rows, long long row_bytes, int sm_count, void* stream);
PF_DECL int pf_ipc_get_handle(void* ptr, void* handle_out_64);
PF_DECL int pf_ipc_open(const void* handle_64, void** ptr_out);
PF_DECL int pf_ipc_close(void* ptr);
PF_DECL int pf_get_base(void* ptr, void** base_out, long long* size_out);
PF_DECL int pf_peek_u32(const void* dev_ptr, unsigned int* out);

// ---- conv_gn.cu : NHWC im2col / col2im, GroupNorm(+SiLU), nearest 2x upsample
PF_DECL int pf_im2col(const void* x, void* cols, int B, int H, int W, int C, int KH, int KW,
                      int Ho, int Wo, int stride, int pad, long long ldc, int dtype, int sm_count,
                      void* stream);
PF_DECL int pf_col2im(const void* dcols, void* dx, int B, int H, int W, int C, int KH, int KW,
                      int Ho, int Wo, int stride, int pad, long long ldc, int dtype, int sm_count,
                      void* stream);
PF_DECL int pf_groupnorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                             void* mean, void* rstd, int B, int HW, int C, int G, float eps,
                             int act_silu, int dtype, int sm_count, void* stream);
PF_DECL int pf_groupnorm_bwd(const void* dy, const void* x, const void* mean, const void* rstd,
                             const void* gamma, const void* beta, void* dx, void* dgamma,
                             void* dbeta, void* sums, int B, int HW, int C, int G, int act_silu,
                             int dtype, int sm_count, void* stream);
PF_DECL int pf_upsample2x(const void* x, void* y, int B, int H, int W, int C, int backward,
                          int dtype, int sm_count, void* stream);

// ---- gemm_sm100.cu : convolution as an implicit GEMM over an NHWC activation
PF_DECL int pf_conv_gemm(const void* x, const void* w2, void* y, int B, int H, int W, int C,
                         int Cout, int KH, int KW, int stride, int pad, long long ldw,
                         long long ldy, int in_dtype, int out_dtype, const void* bias,
                         int bias_dtype, const void* residual, long long ldr, int epilogue,
                         int* status, int sm_count, void* stream);

PF_DECL int pf_conv_wgrad(const void* dy, const void* x, void* dw2, int B, int H, int W, int C,
                          int Cout, int KH, int KW, int stride, int pad, int in_dtype,
                          int accumulate, int* status, int sm_count, void* stream);

// ---- gemm_sm100.cu : GEMM with the all-gather of a row-sharded weight fused in
PF_DECL int pf_gemm_allgather(const void* A, void* w_full, void* const* copies, int world,
                              int rank, const int* row_end, void* ready, void* C, int M, int N,
                              int K, long long lda, long long ldb, long long ldc, int in_dtype,
                              int out_dtype, const void* bias, int bias_dtype,
                              const void* residual, long long ldr, void* aux, long long ldaux,
                              int epilogue, float alpha, int* status, int sm_count, void* stream);
