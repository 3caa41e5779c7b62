// C ABI of libqfa_sm100a.so: argument validation, dispatch, error text.  See include/qfa.h.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "qfa_common.cuh"

namespace qfa {

static std::atomic<int64_t> g_launches{0};
static thread_local char g_cuda_err[256] = "";

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

unsigned int next_launch_epoch() {
  static std::atomic<unsigned int> counter{0};
  unsigned int e = counter.fetch_add(1, std::memory_order_relaxed) + 1;
  if (e == 0) e = counter.fetch_add(1, std::memory_order_relaxed) + 1;   // 0 means "no launch ever timed out"
  return e;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return QFA_ERR_CUDA;
}

int quant_entry(const void* x, int8_t* codes, uint16_t* scale, int8_t* zp, int32_t* rowsum, void* dequant, int64_t Z,
                int64_t H, int64_t M, int64_t D, int64_t sz, int64_t sh, int64_t sm, int64_t sk, int dtype,
                cudaStream_t stream);
int quant_batch_entry(const QfaQuantJob* jobs, int n, int dtype, cudaStream_t stream);
int dequant_entry(const int8_t* codes, const uint16_t* scale, const int8_t* zp, void* out, int64_t Z, int64_t H, int64_t M,
                  int64_t D, int64_t sz, int64_t sh, int64_t sm, int dtype, cudaStream_t stream);
int attn_bwd_tc_supported(const QfaBwdArgs& a);
int attn_bwd_tc_entry(const QfaBwdArgs& a, cudaStream_t stream);
int center_entry(const int8_t* codes, const int8_t* zp, void* out, int64_t Z, int64_t H, int64_t M, int64_t D, int64_t sz,
                 int64_t sh, int64_t sm, cudaStream_t stream);
int attn_fwd_mma_entry(const QfaFwdArgs& a, cudaStream_t stream);
int attn_fwd_tc_supported(const QfaFwdArgs& a);
int attn_fwd_tc_entry(const QfaFwdArgs& a, cudaStream_t stream);
int attn_bwd_mma_entry(const QfaBwdArgs& a, float* dq_accum, cudaStream_t stream);
int mma_probe_entry(int form, int n, int iters, double* ops_out, int32_t* status, cudaStream_t stream);
int wait_timeout_selftest_entry(uint64_t budget_ns, int32_t* status, cudaStream_t stream);
int attn_fwd_shortq_supported(const QfaFwdArgs& a);
int attn_fwd_shortq_entry(const QfaFwdArgs& a, cudaStream_t stream);
int attn_bwd_shortq_supported(const QfaBwdArgs& a);
int attn_bwd_shortq_entry(const QfaBwdArgs& a, cudaStream_t stream);
int attn_bwd_delta_entry(const void* o, const int64_t* so, const void* d_o, const int64_t* sd, float* delta,
                         int64_t delta_stride, int64_t B, int64_t H, int64_t Sq, int64_t D, int dtype,
                         cudaStream_t stream);

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool strides_mult(const int64_t* s, int64_t m) { return s[0] % m == 0 && s[1] % m == 0 && s[2] % m == 0; }

static int check_quant_tensor(const QfaQuantTensor& t, bool need_sum) {
  if (!t.codes || !t.scale || !t.zp) return QFA_ERR_NULL;
  if (need_sum && !t.rowsum) return QFA_ERR_MODE;
  if (!aligned16(t.codes) || !strides_mult(t.stride, 16)) return QFA_ERR_ALIGN;
  return QFA_OK;
}

static int check_common(int mode, int dtype, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D) {
  if (mode != QFA_MODE_REF && mode != QFA_MODE_INT8) return QFA_ERR_MODE;
  if (dtype != QFA_F16 && dtype != QFA_BF16) return QFA_ERR_DTYPE;
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0) return QFA_ERR_SHAPE;
  if (B * H > 0x7fffffffLL / 2 || Sq > (1 << 30) || Skv > (1 << 30)) return QFA_ERR_SHAPE;
  if (D != 64 && D != 128) return QFA_ERR_HEAD_DIM;
  return QFA_OK;
}

}  // namespace qfa

using namespace qfa;

extern "C" {

QFA_API int qfa_quant_per_token(const void* x, int8_t* codes, uint16_t* scale_f16, int8_t* zp, int32_t* rowsum_or_null,
                        int64_t Z, int64_t H, int64_t M, int64_t D, int64_t sx_z, int64_t sx_h, int64_t sx_m,
                        int64_t sx_k, int dtype, qfa_stream_t stream) {
  return quant_entry(x, codes, scale_f16, zp, rowsum_or_null, nullptr, Z, H, M, D, sx_z, sx_h, sx_m, sx_k, dtype,
                     reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_quant_dequant_per_token(const void* x, int8_t* codes, uint16_t* scale_f16, int8_t* zp, int32_t* rowsum_or_null,
                                void* dequant_or_null, int64_t Z, int64_t H, int64_t M, int64_t D, int64_t sx_z,
                                int64_t sx_h, int64_t sx_m, int64_t sx_k, int dtype, qfa_stream_t stream) {
  return quant_entry(x, codes, scale_f16, zp, rowsum_or_null, dequant_or_null, Z, H, M, D, sx_z, sx_h, sx_m, sx_k,
                     dtype, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_quant_batch_per_token(const QfaQuantJob* jobs, int n_jobs, int dtype, qfa_stream_t stream) {
  return quant_batch_entry(jobs, n_jobs, dtype, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_dequant_per_token(const int8_t* codes, const uint16_t* scale_f16, const int8_t* zp, void* out, int64_t Z,
                                  int64_t H, int64_t M, int64_t D, int64_t s_z, int64_t s_h, int64_t s_m, int dtype,
                                  qfa_stream_t stream) {
  return dequant_entry(codes, scale_f16, zp, out, Z, H, M, D, s_z, s_h, s_m, dtype, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_center_per_token(const int8_t* codes, const int8_t* zp, void* out_f16, int64_t Z, int64_t H, int64_t M,
                                 int64_t D, int64_t s_z, int64_t s_h, int64_t s_m, qfa_stream_t stream) {
  return center_entry(codes, zp, out_f16, Z, H, M, D, s_z, s_h, s_m, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_attn_fwd(const QfaFwdArgs* a, qfa_stream_t stream) {
  if (!a) return QFA_ERR_NULL;
  int rc = check_common(a->mode, a->dtype, a->B, a->H, a->Sq, a->Skv, a->D);
  if (rc) return rc;
  if (!a->o || !a->lse) return QFA_ERR_NULL;
  if (!aligned16(a->o) || !strides_mult(a->o_stride, 8)) return QFA_ERR_ALIGN;
  if (a->lse_stride < a->Sq) return QFA_ERR_STRIDE;
  if (a->mode == QFA_MODE_REF) {
    if (!a->q) return QFA_ERR_NULL;
    if (!aligned16(a->q) || !strides_mult(a->q_stride, 8)) return QFA_ERR_ALIGN;
  } else {
    if ((rc = check_quant_tensor(a->qq, true))) return rc;
  }
  if ((rc = check_quant_tensor(a->k, a->mode == QFA_MODE_INT8))) return rc;
  if ((rc = check_quant_tensor(a->v, false))) return rc;
  if (a->k_ctr && !aligned16(a->k_ctr)) return QFA_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool grouped = a->Hkv != 0 && a->Hkv != a->H;
  if (grouped && (a->Hkv < 0 || a->H % a->Hkv != 0)) return QFA_ERR_SHAPE;
  if (attn_fwd_tc_supported(*a)) return attn_fwd_tc_entry(*a, s);
  if (grouped) return QFA_ERR_SHAPE;                 // only the tcgen05 forward reads grouped K/V heads
  if (attn_fwd_shortq_supported(*a)) return attn_fwd_shortq_entry(*a, s);
  return attn_fwd_mma_entry(*a, s);
}

QFA_API int qfa_attn_bwd_delta(const void* o, const int64_t o_stride[3], const void* d_o, const int64_t do_stride[3],
                       float* delta, int64_t delta_stride, int64_t B, int64_t H, int64_t Sq, int64_t D, int dtype,
                       qfa_stream_t stream) {
  if (!o || !d_o || !delta || !o_stride || !do_stride) return QFA_ERR_NULL;
  if (dtype != QFA_F16 && dtype != QFA_BF16) return QFA_ERR_DTYPE;
  if (B <= 0 || H <= 0 || Sq <= 0) return QFA_ERR_SHAPE;
  if (D <= 0 || D % 8 != 0) return QFA_ERR_HEAD_DIM;
  if (delta_stride < Sq) return QFA_ERR_STRIDE;
  if (!aligned16(o) || !aligned16(d_o) || !strides_mult(o_stride, 8) || !strides_mult(do_stride, 8))
    return QFA_ERR_ALIGN;
  return attn_bwd_delta_entry(o, o_stride, d_o, do_stride, delta, delta_stride, B, H, Sq, D, dtype,
                              reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_attn_bwd(const QfaBwdArgs* a, qfa_stream_t stream) {
  if (!a) return QFA_ERR_NULL;
  int rc = check_common(a->mode, a->dtype, a->B, a->H, a->Sq, a->Skv, a->D);
  if (rc) return rc;
  if (!a->d_o || !a->lse || !a->delta || !a->dq || !a->dk) return QFA_ERR_NULL;
  if (!a->dkv_fused && !a->dv) return QFA_ERR_NULL;
  if (a->lse_stride < a->Sq) return QFA_ERR_STRIDE;
  if (!aligned16(a->d_o) || !strides_mult(a->do_stride, 8) || !aligned16(a->dq) || !strides_mult(a->dq_stride, 8) ||
      !aligned16(a->dk) || !strides_mult(a->dk_stride, 8))
    return QFA_ERR_ALIGN;
  if (!a->dkv_fused && (!aligned16(a->dv) || !strides_mult(a->dv_stride, 8))) return QFA_ERR_ALIGN;
  if (a->mode == QFA_MODE_REF) {
    if (!a->q) return QFA_ERR_NULL;
    if (!aligned16(a->q) || !strides_mult(a->q_stride, 8)) return QFA_ERR_ALIGN;
  } else {
    if ((rc = check_quant_tensor(a->qq, true))) return rc;
  }
  if ((rc = check_quant_tensor(a->k, a->mode == QFA_MODE_INT8))) return rc;
  if ((rc = check_quant_tensor(a->v, false))) return rc;
  if (a->dkv_fused && (a->k.codes != a->v.codes || a->k.scale != a->v.scale || a->k.zp != a->v.zp)) return QFA_ERR_MODE;
  if (attn_bwd_shortq_supported(*a)) return attn_bwd_shortq_entry(*a, reinterpret_cast<cudaStream_t>(stream));
  if (attn_bwd_tc_supported(*a)) return attn_bwd_tc_entry(*a, reinterpret_cast<cudaStream_t>(stream));
  if (!a->dq_accum) return QFA_ERR_NULL;
  if (!aligned16(a->dq_accum)) return QFA_ERR_ALIGN;
  return attn_bwd_mma_entry(*a, a->dq_accum, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_selftest_wait_timeout(uint64_t budget_ns, int32_t* status, qfa_stream_t stream) {
  return wait_timeout_selftest_entry(budget_ns, status, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API int qfa_probe_mma_rate(int form, int n, int iters, double* ops_out, int32_t* status, qfa_stream_t stream) {
  return mma_probe_entry(form, n, iters, ops_out, status, reinterpret_cast<cudaStream_t>(stream));
}

QFA_API const char* qfa_strerror(int code) {
  switch (code) {
    case QFA_OK: return "ok";
    case QFA_ERR_NULL: return "a required pointer is NULL";
    case QFA_ERR_DTYPE: return "unsupported dtype (expected fp16 or bf16)";
    case QFA_ERR_SHAPE: return "a size is not positive or exceeds the kernel's range";
    case QFA_ERR_HEAD_DIM: return "unsupported head dimension (attention supports 64 and 128)";
    case QFA_ERR_STRIDE: return "unsupported stride";
    case QFA_ERR_ALIGN: return "pointer or stride not aligned (16-byte rows required)";
    case QFA_ERR_MODE: return "unknown mode, or operands missing / inconsistent for the mode";
    case QFA_ERR_CUDA: return "a CUDA call failed (see qfa_last_cuda_error)";
    case QFA_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
    case QFA_STATUS_WAIT_TIMEOUT: return "a bounded barrier wait inside a kernel ran out";
    default: return "unknown qfa code";
  }
}

QFA_API const char* qfa_last_cuda_error(void) { return g_cuda_err; }
QFA_API int qfa_version(void) { return 5; }
QFA_API int64_t qfa_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
