// C ABI of the elfa_b200 native library (libelfa_b200.so). Every function returns an ELFA_* code
// (0 = ok); elfa_last_error() gives the message of the last failure on the calling thread.
// All device pointers are raw CUDA pointers; `stream` is a cudaStream_t passed as void*.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogue flags (bitmask).
#define ELFA_EPI_BIAS 1u          // + bias[N] (bf16)
#define ELFA_EPI_GELU 2u          // tanh-GELU after bias
#define ELFA_EPI_DGELU_AUX 4u     // multiply by GELU'(aux[M,N])
#define ELFA_EPI_ADD_AUX 8u       // + aux[M,N] (residual)
#define ELFA_EPI_ACCUM 16u        // C += result
#define ELFA_EPI_OUT_F32 32u      // C is fp32 (default bf16)
#define ELFA_EPI_STORE_PREACT 64u // also store the value before GELU to `preact`
#define ELFA_EPI_STAGED 128u      // bf16 output through shared memory and TMA stores (the epilogue of the fused reduce-scatter form)

const char* elfa_last_error(void);
int elfa_version(void);
int elfa_set_deterministic(int on);
// SHA-256 (hex) over the sources this library was built from; the Python side compares it with the sources it finds
const char* elfa_source_hash(void);
long long elfa_launch_count(int reset);
int elfa_status(unsigned int* out);
// Checked variant of the library (built with -DELFA_BOUNDS): kernels test the tile coordinates, ring-slot offsets and push
// ranges they compute, record a violation in the status word (bit 4) and skip the access.
int elfa_bounds_enabled();
int elfa_bounds_selftest(void* stream);
int elfa_device_info(int device, long long* out6);
int elfa_is_blackwell(int device);
int elfa_enable_peer_access(int* n_enabled);
int elfa_pinned_alloc(void** out, size_t bytes);
int elfa_pinned_free(void* p);

// C[M,N] = epilogue(alpha * op(A) * op(B)); see gemm_bf16.cu for operand conventions.
int elfa_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                   long long ldc, int a_mn_major, int b_mn_major, const void* bias, const void* aux, long long ldaux,
                   void* preact, long long ldpre, float alpha, unsigned flags, int force_bn, int max_ctas, void* stream);

// ---- norm.cu -----------------------------------------------------------------------------------
int elfa_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out, float* mean_out,
                  float* rstd_out, int rows, int D, float eps, int kind, void* stream);
int elfa_norm_bwd_partials(int rows, int D);
int elfa_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* dres, void* dx,
                  void* dw, void* db, float* scratch, int rows, int D, int kind, int grads_f32, int accumulate, void* stream);

// ---- elementwise.cu ----------------------------------------------------------------------------
int elfa_elementwise(int op, const void* a, const void* b, void* out, long long n, float alpha, void* stream);
int elfa_embedding_fwd(const long long* ids, const void* tok, const void* pos, void* out, int tokens, int D, int seq, int pos_div, int pos0,
                       int vocab_lo, int vocab_hi, int vocab_total, void* stream);
int elfa_embedding_bwd(const long long* ids, const void* dy, void* dtok, void* dpos, int tokens, int D, int seq, int pos_div, int pos0,
                       int vocab_lo, int vocab_hi, int grads_f32, void* stream);
int elfa_cast(const void* src, int src_type, void* dst, int dst_type, long long n, float scale, void* stream);

// ---- xent.cu -----------------------------------------------------------------------------------
int elfa_xent_stats(const void* logits, long long ld, const long long* targets, float* stats, int rows, int V, int vocab_lo,
                    int vocab_total, void* stream);
int elfa_xent_stats_push(const void* logits, long long ld, const long long* targets, const unsigned long long* peer_tables,
                         int slice, int world, int rows, int V, int vocab_lo, int vocab_total, void* stream);
int elfa_xent_grad(void* logits, long long ld, void* dlogits, long long ldd, const long long* targets, const float* stats,
                   int nslices, float* loss_out, int rows, int V, int vocab_lo, int vocab_total, float smoothing,
                   const float* grad_scale_ptr, float grad_scale, void* stream);

// ---- optim.cu ----------------------------------------------------------------------------------
int elfa_sumsq(const void* grad, int grad_type, long long n, float* part, void* scalars, int accumulate, void* stream);
int elfa_clip_coef(void* scalars, float max_norm, float inv_loss_scale, void* stream);
int elfa_adamw(void* param, int param_type, float* master, float* m, float* v, const void* grad, int grad_type, long long n,
               float lr, float beta1, float beta2, float eps, float wd, int step, const void* scalars, void* stream);
int elfa_lion(void* param, int param_type, float* master, float* m, const void* grad, int grad_type, long long n, float lr,
              float beta1, float beta2, float wd, const void* scalars, void* stream);
int elfa_muon_momentum(float* m, const void* grad, int grad_type, void* y, long long n, float beta, const void* scalars,
                       float* part, float* norm_out, void* stream);
int elfa_three_i_minus(void* g, int d, void* stream);
int elfa_muon_apply(void* param, int param_type, float* master, const void* y, long long n, float lr, const void* scalars,
                    void* stream);

// ---- attention_fwd.cu --------------------------------------------------------------------------
int elfa_attention_fwd(const void* qkv, long long stride_s, long long stride_b, void* out, long long o_stride_s,
                       long long o_stride_b, float* lse, int S, int B, int H, int hd, float scale, int causal, void* stream);

int elfa_attention_fwd_ex(const void* qkv, long long stride_s, long long stride_b, void* out, long long o_stride_s,
                          long long o_stride_b, float* lse, int S, int B, int H, int Hkv, int hd, float scale, int causal,
                          const int* doc_start, void* stream);
// ---- attention_bwd.cu --------------------------------------------------------------------------
int elfa_attention_bwd(const void* qkv, long long stride_s, long long stride_b, const void* out, const void* dout,
                       long long o_stride_s, long long o_stride_b, const float* lse, float* delta, void* dqkv,
                       long long d_stride_s, long long d_stride_b, int S, int B, int H, int hd, float scale, int causal,
                       void* stream);

int elfa_attention_bwd_ex(const void* qkv, long long stride_s, long long stride_b, const void* out, const void* dout,
                          long long o_stride_s, long long o_stride_b, const float* lse, float* delta, void* dqkv,
                          long long d_stride_s, long long d_stride_b, int S, int B, int H, int Hkv, int hd, float scale, int causal,
                          const int* doc_start, void* stream);
// ---- gemm_mxfp8.cu ------------------------------------------------------------------------------
// Block-scaled MXFP8 tensor-core GEMM (e4m3 payloads, ue8m0 scales per 32 K-elements in 512-byte atoms)
long long elfa_mxfp8_sf_bytes(int rows, int cols, int b_operand);
int elfa_mxfp8_quantize_gemm(const void* x, long long ldx, void* payload, void* sf, void* deq, int rows, int cols, int b_operand,
                             void* stream);
int elfa_mxfp8_dequantize(const void* payload, const void* sf, void* out, int rows, int cols, int b_operand, void* stream);
int elfa_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long long ldc,
                    const void* bias, void* preact, long long ldpre, unsigned flags, int force_bn, void* stream);

// Block-scaled NVFP4 tensor-core GEMM (e2m1 payloads two per byte, ue4m3 scales per 16 K-elements, fp32 tensor scale)
long long elfa_nvfp4_sf_bytes(int rows, int cols, int b_operand);
int elfa_nvfp4_quantize_gemm(const void* x, long long ldx, void* payload, void* sf, void* deq, int rows, int cols, int b_operand,
                             const float* tensor_amax, void* stream);
int elfa_gemm_nvfp4(const void* A, const void* sfa, const float* amax_a, const void* B, const void* sfb, const float* amax_b, void* C,
                    int M, int N, int K, long long ldc, const void* bias, void* preact, long long ldpre, unsigned flags, int force_bn,
                    void* stream);

// ---- quant.cu ----------------------------------------------------------------------------------
int elfa_mxfp8_fake_quant(const void* x, void* out, int rows, int cols, int axis, void* stream);
int elfa_mxfp8_quantize(const void* x, void* payload, void* scales, int rows, int cols, void* stream);
int elfa_nvfp4_fake_quant(const void* x, void* out, int rows, int cols, int axis, const float* tensor_amax, void* stream);
int elfa_amax(const void* x, long long n, float* out, void* stream);
int elfa_fp8_tensor_fake_quant(const void* x, void* out, long long n, const float* scale, int fmt, void* stream);
int elfa_int_affine_fake_quant(const void* x, void* out, long long n, int bits, float* minmax, float* part, void* stream);
int elfa_qat_surrogate_bwd(const void* x, const void* g, void* out, long long n, int mode, float p0, float p1, void* stream);

// ---- fused GEMM + collective (gemm_bf16.cu) ----------------------------------------------------------
int elfa_gemm_ag(const void* x_local, long long ldx, const unsigned long long* peer_xfull, const unsigned long long* peer_flags,
                 const void* my_flags, unsigned int* arrivals_io, const void* B, void* C, int M, int N, int K, long long ldb,
                 long long ldc, int b_mn_major, void* preact, long long ldpre, unsigned flags, int rank, int world, int wait_ms,
                 void* stream);
int elfa_gemm_ag_mxfp8(const unsigned long long* peer_buf, const unsigned long long* peer_flags, const void* my_flags,
                       unsigned int* arrivals_io, const void* B, const void* sfb, void* C, int M, int N, int K, long long ldc,
                       void* preact, long long ldpre, unsigned flags, int rank, int world, int wait_ms, void* stream);
// ZeRO stage 3: the parameter all-gather inside the consuming GEMM. B [K, N] row-major is bytes [w_off, w_off + K*N*2) of a
// bucket sharded over `world` ranks (`shard_bytes` each, rank r's shard at shard_src[r], peer addressable); the kernel copies it
// into the local bucket `bucket_dst` (B = bucket_dst + w_off) while it multiplies. `flags_dev`: `world` zeroed u32 counters.
int elfa_gemm_gb(const void* A, long long lda, void* C, long long ldc, int M, int N, int K, void* preact, long long ldpre,
                 unsigned flags, const unsigned long long* shard_src, void* bucket_dst, long long w_off, long long shard_bytes,
                 void* flags_dev, int rank, int world, int wait_ms, void* stream);
int elfa_gemm_rs(const void* A, long long lda, const void* B, long long ldb, int b_mn_major, int M, int N, int K,
                 const unsigned long long* peer_recv, const unsigned long long* peer_flags, const void* my_flags,
                 unsigned int* arrivals_io, void* out, long long ld_out, int rank, int world, int wait_ms, int max_ctas, void* stream);

int elfa_gemm_rs_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, int M, int N, int K,
                       const unsigned long long* peer_recv, const unsigned long long* peer_flags, const void* my_flags,
                       unsigned int* arrivals_io, void* out, long long ld_out, int rank, int world, int wait_ms, int max_ctas, void* stream);
int elfa_gemm_rs_slot_cols(int N);

// ---- multimem.cu (NVLS: reductions inside the NVSwitch through the arena's multicast mapping) ------------------
int elfa_multimem_collective(unsigned long long mc, const void* local, void* out, long long off_bytes, long long n, int dtype,
                             int rank, int world, float scale, int mode, void* stream);

// ---- zero.cu -----------------------------------------------------------------------------------
int elfa_symm_barrier(const unsigned long long* peer_flags, const void* my_flags, int rank, int world, unsigned int epoch,
                      int wait_ms, void* stream);
int elfa_zero_reduce(const unsigned long long* peer_grads, int rank, int world, long long lo, long long n, float* reduced,
                     float scale, float* part, void* scalars, void* stream);
int elfa_zero_adamw_allgather(const unsigned long long* peer_params, int rank, int world, long long lo, long long n, float* master,
                              float* m, float* v, const float* reduced, float lr, float beta1, float beta2, float eps, float wd,
                              int step, const void* scalars, long long wd_lo, long long wd_hi, void* stream);

int elfa_zero_pack_bf16(const float* src, void* dst, long long n, void* stream);
int elfa_zero3_reduce_acc_bf16(const unsigned long long* peer_staged, int world, long long lo, long long n, float* acc, float scale,
                               void* stream);
int elfa_zero3_gather_window(const unsigned long long* peer_shards, int world, long long src_off_bytes, long long shard_bytes,
                             long long lo_bytes, long long hi_bytes, void* dst, void* stream);
int elfa_zero3_gather(const unsigned long long* peer_shards, int world, long long src_off_bytes, long long shard_bytes, void* dst,
                      void* stream);
int elfa_zero3_reduce_acc(const unsigned long long* peer_grads, int world, long long lo, long long n, float* acc, float scale,
                          void* stream);

int elfa_softmax_rows(const void* x, void* out, long long rows, int cols, long long ldx, long long ldo, float scale, void* stream);

// ---- p2p.cu ------------------------------------------------------------------------------------
int elfa_p2p_send(const void* src, unsigned long long peer_dst, long long bytes, unsigned long long peer_counter, int* blocks_out,
                  void* stream);
int elfa_p2p_wait(const void* counter, unsigned int target, int wait_ms, void* stream);
// Link probe: copy `bytes` to `dst` (a peer address) with per-thread 16-byte stores (mode 0) or a bulk-copy pipeline through
// shared memory (mode 1: `warps` lanes per CTA, `depth` buffers of `piece` bytes each).
int elfa_p2p_probe(const void* src, unsigned long long dst, long long bytes, int mode, int ctas, int warps, int piece, int depth,
                   void* stream);

// ---- prism.cu ----------------------------------------------------------------------------------
int elfa_prism_fwd(const void* u, const void* v, const unsigned long long* p, void* y, long long tokens, int G, int d, int L,
                   void* stream);
int elfa_prism_bwd(const void* u, const void* v, const unsigned long long* p, const void* dy, void* du, void* dv,
                   const unsigned long long* dp, long long tokens, int G, int d, int L, void* stream);

// ---- efla.cu -----------------------------------------------------------------------------------
int elfa_efla_scan_fwd(const void* k, const void* v, const float* beta, const float* state0, void* o, float* state_out,
                       float* ckpt, int B, int T, int H, int d, int chunk, void* stream);
int elfa_efla_scan_bwd(const void* k, const void* v, const float* beta, const float* ckpt, const void* dout,
                       const float* dstate_out, void* dk, void* dv, float* dbeta_tok, float* dstate0, float* work,
                       float* dk_part, float* dc_part, int B, int T, int H, int d, int chunk, void* stream);
int elfa_shortconv_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int C, int W, void* stream);
int elfa_shortconv_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, float* db, int B, int T, int C, int W,
                       void* stream);

#ifdef __cplusplus
}
#endif
