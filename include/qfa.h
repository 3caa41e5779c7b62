/*
 * qfa.h -- C ABI of libqfa_sm100a.so: per-token asymmetric INT8 quantizer and
 * INT8 flash attention (forward, backward) for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes raw DEVICE pointers, sizes and element strides; the
 * library allocates no user-visible memory, launches on the stream it is given
 * and returns without synchronising.  Return value: 0 = launched; negative =
 * argument rejected before any launch (see qfa_strerror).  Kernels that wait on
 * hardware barriers use bounded waits; when a wait runs out they store a positive
 * code into the caller's `status` word (device memory, may be NULL) and return.
 *
 * "Reference" in the comments is the Triton project this library is a drop-in
 * for on this path; citations are file:line in that project.
 */
#ifndef QFA_H_
#define QFA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* qfa_stream_t;

#if defined(__GNUC__)
#define QFA_API __attribute__((visibility("default")))
#else
#define QFA_API
#endif

/* dtype codes for 16-bit floating tensors */
#define QFA_F16 0
#define QFA_BF16 1

/* numeric mode of the attention kernels */
#define QFA_MODE_REF 0  /* Q stays 16-bit, logits from a 16-bit MMA on dequantized K (the reference's math) */
#define QFA_MODE_INT8 1 /* Q and K int8, logits from an int8 x int8 -> int32 MMA plus zero-point corrections */

/* error codes (negative: rejected on the host; positive: reported by a kernel) */
#define QFA_OK 0
#define QFA_ERR_NULL -1        /* a required pointer is NULL */
#define QFA_ERR_DTYPE -2       /* dtype code is not QFA_F16 / QFA_BF16 */
#define QFA_ERR_SHAPE -3       /* a size is <= 0 or too large for the kernel */
#define QFA_ERR_HEAD_DIM -4    /* head dimension not supported by this entry point */
#define QFA_ERR_STRIDE -5      /* innermost stride must be 1 / row stride not supported */
#define QFA_ERR_ALIGN -6       /* pointer or stride not aligned for vector / TMA access */
#define QFA_ERR_MODE -7        /* unknown mode, or operands missing for the mode */
#define QFA_ERR_CUDA -8        /* a CUDA runtime / driver call failed (see qfa_last_cuda_error) */
#define QFA_ERR_TOO_LARGE -9   /* size exceeds the fixed capacity of a no-allocation entry point */
#define QFA_STATUS_WAIT_TIMEOUT 1 /* a bounded mbarrier wait inside a kernel ran out */

/* ---------------------------------------------------------------------------------------------
 * Quantizer.  Replaces the launch in asymmetric_quant_per_token (asymmetric_quant.py:109-149) and
 * the kernel _asymmetric_quant_kernel (asymmetric_quant.py:32-106).
 *
 *   x        (Z,H,M,D) fp16/bf16, element strides sx_z, sx_h, sx_m, sx_k (any values)
 *   codes    int8, written with the SAME strides as x (asymmetric_quant.py:64,127)
 *   scale    fp16 bits, contiguous (Z*H*M)          (asymmetric_quant.py:93)
 *   zp       int8, contiguous (Z*H*M)               (asymmetric_quant.py:94)
 *   rowsum   int32 sum of each row's codes, contiguous (Z*H*M); may be NULL.  Not in the
 *            reference; the int8 attention path needs it.
 * Results are bit-identical to the reference kernel's.
 */
QFA_API int qfa_quant_per_token(const void* x, int8_t* codes, uint16_t* scale_f16, int8_t* zp,
                        int32_t* rowsum_or_null,
                        int64_t Z, int64_t H, int64_t M, int64_t D,
                        int64_t sx_z, int64_t sx_h, int64_t sx_m, int64_t sx_k,
                        int dtype, qfa_stream_t stream);

/* Same quantizer; additionally writes the dequantized row (code - zp) * fp16(scale), rounded to
 * `dtype`, i.e. the operand the reference builds in registers at quant_flash_attn.py:65-66.
 * `dequant` is contiguous (Z,H,M,D) and may be NULL. */
QFA_API int qfa_quant_dequant_per_token(const void* x, int8_t* codes, uint16_t* scale_f16, int8_t* zp,
                                int32_t* rowsum_or_null, void* dequant_or_null,
                                int64_t Z, int64_t H, int64_t M, int64_t D,
                                int64_t sx_z, int64_t sx_h, int64_t sx_m, int64_t sx_k,
                                int dtype, qfa_stream_t stream);

/* Several tensors in one call.  Replaces the back-to-back asymmetric_quant_per_token calls a caller of the
 * attention path makes for its operands (the reference quantizes outside the attention operator,
 * test_accuracy.py:88; the int8 operator needs Q, K and V).  Each job has the arguments of
 * qfa_quant_dequant_per_token.  At most 4 jobs; when all of them have the same head dimension, inner stride 1
 * and 16-byte aligned rows they run as ONE kernel launch (block ranges of one grid), otherwise one launch per
 * job; results are bit-identical to separate calls either way. */
typedef struct {
  const void* x;
  int8_t* codes;
  uint16_t* scale_f16;
  int8_t* zp;
  int32_t* rowsum_or_null;
  void* dequant_or_null;
  int64_t Z, H, M, D;
  int64_t sx_z, sx_h, sx_m, sx_k;
  void* centered_or_null; /* code - zero_point as fp16, contiguous (Z, H, M, D), 16-byte aligned: QfaFwdArgs.k_ctr */
} QfaQuantJob;
QFA_API int qfa_quant_batch_per_token(const QfaQuantJob* jobs, int n_jobs, int dtype, qfa_stream_t stream);

/* Dequantize: out[token][:] = (code - zp) * fp16(scale) rounded to `dtype`, the operand the reference
 * builds at quant_flash_attn.py:65-66 / :150-151.  codes (Z,H,M,D) with element strides s_z, s_h, s_m (inner
 * stride 1, D a multiple of 16); scale / zp contiguous over tokens; out contiguous (Z,H,M,D). */
QFA_API int qfa_dequant_per_token(const int8_t* codes, const uint16_t* scale_f16, const int8_t* zp, void* out,
                                  int64_t Z, int64_t H, int64_t M, int64_t D,
                                  int64_t s_z, int64_t s_h, int64_t s_m, int dtype, qfa_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * One quantized operand of the attention kernels: codes (B,H,S,D) with element strides (inner
 * stride 1), and per-token scale / zero-point / code-sum arrays contiguous over (B*H*S).
 */
/* code - zero_point as fp16 (exact), contiguous (Z, H, M, D) output; codes with strides s_z, s_h, s_m (multiples of
 * 16), D a multiple of 16, pointers 16-byte aligned.  No counterpart in the reference: it feeds QfaFwdArgs.k_ctr. */
QFA_API int qfa_center_per_token(const int8_t* codes, const int8_t* zp, void* out_f16,
                                 int64_t Z, int64_t H, int64_t M, int64_t D,
                                 int64_t s_z, int64_t s_h, int64_t s_m, qfa_stream_t stream);
typedef struct {
  const int8_t* codes;
  int64_t stride[3];     /* batch, head, token strides of codes, in elements */
  const uint16_t* scale; /* fp16 bits */
  const int8_t* zp;
  const int32_t* rowsum; /* needed for Q and K in QFA_MODE_INT8, else may be NULL */
} QfaQuantTensor;

/* Forward.  Replaces QuantFlashAttention.forward's launch (quant_flash_attn.py:179-204) and the
 * kernel _attn_fwd_kernel_quantized (quant_flash_attn.py:27-83); `causal` follows
 * flash_attn_triton.py:441,50 (row >= column, top-left aligned).
 *
 * QFA_MODE_REF : q (16-bit) is read, `qq` is ignored.  k and v may be the same tensor.
 * QFA_MODE_INT8: qq, k (codes + scale + zp + rowsum) feed the int8 MMA; q is ignored.
 * v_hat (optional, 16-bit, contiguous (B,H,Skv,D)): dequantized V as written by
 * qfa_quant_dequant_per_token; when NULL the kernel dequantizes v's codes itself.  It selects the tcgen05 kernels:
 * QFA_MODE_INT8 always needs it for them; QFA_MODE_REF (k and v the same tensor, non-causal) needs it with more than
 * 128 query rows only -- with 17 to 128 rows the tcgen05 kernel dequantizes the codes itself and ignores v_hat.
 * o: 16-bit (B,H,Sq,D) with strides; lse: fp32, row b*H+h starts at lse + (b*H+h)*lse_stride.
 */
typedef struct {
  int32_t mode, dtype, causal;
  float sm_scale;
  int64_t B, H, Sq, Skv, D;
  const void* q;
  int64_t q_stride[3];
  QfaQuantTensor qq, k, v;
  const void* v_hat;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride;
  int32_t* status; /* device int32 or NULL */
  /* Grouped K/V heads (no counterpart in the reference, which has one K/V tensor per query head): number of
   * heads of k, v (and v_hat); 0 means H.  Must divide H; query head h reads K/V head h / (H / Hkv).  Served
   * by the tcgen05 forward (QFA_MODE_INT8 with v_hat, head dim 64 or 128); any other combination with
   * Hkv != H returns QFA_ERR_SHAPE. */
  int64_t Hkv;
  /* Optional (QFA_MODE_INT8 with v_hat): the centered K codes, code - zero_point as fp16, contiguous
   * (B, Hkv, Skv, D), 16-byte aligned (qfa_center_per_token, or the `centered_or_null` output of the batched
   * quantizer).  When given, the tcgen05 forward forms the same integer dot products sum((q - z_q)(k - z_k)) with
   * a 16-bit MMA over centered operands (exact in fp32 for D <= 128) instead of the int8 MMA plus zero-point
   * corrections; the results agree to fp32 rounding and the kernel is faster.  NULL selects the int8 MMA. */
  const void* k_ctr;
} QfaFwdArgs;

QFA_API int qfa_attn_fwd(const QfaFwdArgs* args, qfa_stream_t stream);

/* Backward pre-pass, delta[row] = sum_d O*dO.  Replaces _bwd_preprocess_kernel
 * (quant_flash_attn.py:88-101).  o and d_o are 16-bit (B,H,Sq,D) with their own strides. */
QFA_API int qfa_attn_bwd_delta(const void* o, const int64_t o_stride[3], const void* d_o,
                       const int64_t do_stride[3], float* delta, int64_t delta_stride,
                       int64_t B, int64_t H, int64_t Sq, int64_t D, int dtype, qfa_stream_t stream);

/* Backward.  Replaces QuantFlashAttention.backward's main launch (quant_flash_attn.py:225-235) and
 * _bwd_kernel_quantized (quant_flash_attn.py:109-166).
 *
 * Forward operands as in QfaFwdArgs, plus lse and delta (same row stride), d_o, and outputs:
 *   dq            16-bit (B,H,Sq,D)
 *   dk, dv        16-bit (B,H,Skv,D).  If `dkv_fused` is non-zero only `dk` is written and holds
 *                 dV + sm_scale*dK as the reference does (quant_flash_attn.py:161); requires k == v.
 * dq_accum: fp32 scratch, contiguous (B,H,Sq,D), owned by the caller; the mma.sync kernel zero-fills it,
 * accumulates dQ into it with atomics and converts it into dq (the short-query and tcgen05 kernels do not
 * touch it).
 * Gradients: dq = sm_scale * dS.K^, dk = sm_scale * dS^T.Q, dv = P^T.dO.
 */
typedef struct {
  int32_t mode, dtype, causal, dkv_fused;
  float sm_scale;
  int64_t B, H, Sq, Skv, D;
  const void* q;
  int64_t q_stride[3];
  QfaQuantTensor qq, k, v;
  const void* d_o;
  int64_t do_stride[3];
  const float* lse;
  const float* delta;
  int64_t lse_stride;
  void* dq;
  int64_t dq_stride[3];
  void* dk;
  int64_t dk_stride[3];
  void* dv;
  int64_t dv_stride[3];
  float* dq_accum;
  int32_t* status;
  /* Optional (QFA_MODE_INT8): dequantized Q, K, V as 16-bit contiguous (B,H,S,D) tensors
   * (qfa_dequant_per_token / qfa_quant_dequant_per_token).  When all three are given and the head
   * dimension is 64 or 128 the tcgen05 backward kernels run and dq_accum is not used. */
  const void* q_hat;
  const void* k_hat;
  const void* v_hat;
} QfaBwdArgs;

QFA_API int qfa_attn_bwd(const QfaBwdArgs* args, qfa_stream_t stream);

/* Backward without allocation.  No counterpart in the reference (its backward allocates its
 * buffers with torch, quant_flash_attn.py:213-216); added for hosts that cannot obtain device
 * memory at call time, e.g. an inference-engine plugin whose enqueue hook must not allocate, or a
 * process that gave the whole device to a memory pool at start-up.
 *
 * Same validation, arithmetic and outputs as qfa_attn_bwd, with two differences.  (1) `dq_accum` in `args` is
 * ignored: the fp32 dQ accumulator is a fixed array inside the library (qfa_static_scratch_capacity() floats
 * = 16 MiB, resident on every GPU that loads the library until the process exits).  (2) `q_hat`, `k_hat` and
 * `v_hat` are ignored too, so the call always runs the general (mma.sync) backward kernels, the ones that
 * accumulate dQ in scratch memory; these are slower than the tcgen05 kernels qfa_attn_bwd picks when the
 * dequantized operands are supplied.  The call itself requests no memory: it makes no cudaMalloc / cudaFree
 * and calls no allocating library routine.
 *   - B*H*Sq*D must not exceed qfa_static_scratch_capacity(); larger problems return
 *     QFA_ERR_TOO_LARGE before anything is launched.
 *   - The FIRST call on each device does one-time set-up with that device current: it looks up the array's
 *     device address, which makes the CUDA runtime load the module that holds the 16 MiB array, and the first
 *     launch loads the kernels.  That set-up does take device memory from the driver.  A host that is about
 *     to hand the whole device to its own pool must therefore make one (small) call first, at start-up, and
 *     outside any stream capture; later calls find everything in place.
 *   - All calls share the one array; the used part is zero-filled on the caller's stream at the start of
 *     each call and holds the previous call's data otherwise.  Two calls whose kernels overlap on the GPU
 *     (different streams) race on it: serialize them. */
QFA_API int qfa_attn_bwd_static_scratch(const QfaBwdArgs* args, qfa_stream_t stream);
/* Capacity, in floats, of the accumulator used by qfa_attn_bwd_static_scratch. */
QFA_API int64_t qfa_static_scratch_capacity(void);

/* Self-test of the bounded waits.  No counterpart in the reference (its kernels have no device-side waits).
 * Launches one tiny kernel whose only thread waits, for at most `budget_ns` nanoseconds (1 .. 100 000 000), on a
 * barrier that nothing completes.  The wait gives up, the kernel stores QFA_STATUS_WAIT_TIMEOUT into `status`
 * (device-accessible int32, required) and returns normally: nothing traps, the context stays usable and later
 * launches of every entry point are unaffected.  Lets a deployment check the time-out reporting path end to
 * end without provoking a fault. */
QFA_API int qfa_selftest_wait_timeout(uint64_t budget_ns, int32_t* status, qfa_stream_t stream);

/* Tensor-pipe rate probe.  No counterpart in the reference.  One CTA per SM of the current device issues
 * `iters` (2 .. 20000) rounds of four K-steps of 128 x n x K tcgen05 MMAs on operand tiles resident in shared
 * memory (no loads, no epilogue), so that ops / time is the peak rate of that MMA form on this GPU: the
 * denominator the attention kernels' int8 roofline needs and no library GEMM reports.
 *   form 0: kind::i8, A and B from shared memory (K = 32)      form 1: kind::f16 (bf16), A and B from shared memory
 *   form 2: kind::f16 (bf16), A from tensor memory             (K = 16);   n = 128 or 256.
 * *ops_out (host pointer, may be NULL) receives 2 * 128 * n * K * 4 * iters * SMs; time the launch with events on
 * `stream`.  `status` as for the attention kernels (may be NULL). */
QFA_API int qfa_probe_mma_rate(int form, int n, int iters, double* ops_out, int32_t* status, qfa_stream_t stream);

/* Text for a return / status code. */
QFA_API const char* qfa_strerror(int code);
/* Last CUDA error string seen by this library on the calling thread ("" if none). */
QFA_API const char* qfa_last_cuda_error(void);
/* ABI version of this header. */
QFA_API int qfa_version(void);
/* Number of kernel launches issued by this library since load (all threads). */
QFA_API int64_t qfa_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* QFA_H_ */
