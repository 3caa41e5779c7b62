// qfa_attn_bwd_static_scratch: the attention backward without any caller- or library-side
// allocation of its fp32 dQ accumulator.
//
// Some hosts of this library cannot obtain device memory at call time: an inference-engine plugin
// whose enqueue hook is forbidden to allocate, or a process that handed the whole device to a
// memory pool at start-up, so that a cudaMalloc would fail or stall every stream.  For them the
// accumulator lives in a fixed array inside the library image.  The price: the array occupies
// device memory on every GPU that loads the library until the process exits, problems larger
// than the array are rejected, and all calls share the one array.
#include <mutex>

#include "qfa_common.cuh"

namespace qfa {

int attn_bwd_mma_entry(const QfaBwdArgs& a, float* dq_accum, cudaStream_t stream);

// B*H*Sq*D of the largest problem this entry point takes (4 Mi floats = 16 MiB per GPU).
constexpr int64_t kStaticScratchFloats = int64_t(4) << 20;
static __device__ __align__(256) float g_bwd_dq_scratch[kStaticScratchFloats];

static float* g_scratch_ptr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of the array on the CURRENT device.  In host code the name g_bwd_dq_scratch is
// only a handle for the runtime, not a device pointer; the address must be asked for, once per
// device, with that device current.
static int scratch_for_current_device(float** out) {
  int dev = 0;
  QFA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return QFA_ERR_SHAPE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    float* ptr = nullptr;
    QFA_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_bwd_dq_scratch));
    if (!ptr) return QFA_ERR_CUDA;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return QFA_OK;
}

}  // namespace qfa

using namespace qfa;

extern "C" QFA_API int64_t qfa_static_scratch_capacity(void) { return kStaticScratchFloats; }

extern "C" QFA_API int qfa_attn_bwd_static_scratch(const QfaBwdArgs* a, qfa_stream_t stream) {
  if (!a) return QFA_ERR_NULL;
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->D <= 0) return QFA_ERR_SHAPE;
  // reject before anything is launched; the products cannot overflow: each factor is checked first
  if (a->B > kStaticScratchFloats || a->H > kStaticScratchFloats || a->Sq > kStaticScratchFloats ||
      a->D > kStaticScratchFloats)
    return QFA_ERR_TOO_LARGE;
  if (a->B * a->H > kStaticScratchFloats || a->B * a->H * a->Sq > kStaticScratchFloats ||
      a->B * a->H * a->Sq * a->D > kStaticScratchFloats)
    return QFA_ERR_TOO_LARGE;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != QFA_OK) return rc;
  // Same validation as qfa_attn_bwd, with the static array as accumulator.  The launcher of the
  // general backward zero-fills the part of the array the call uses with a memset on the caller's
  // stream before its kernels run (the array keeps the previous call's contents otherwise).
  QfaBwdArgs b = *a;
  b.dq_accum = scratch;
  b.q_hat = b.k_hat = b.v_hat = nullptr;   // always the kernel that accumulates dQ in scratch memory
  return qfa_attn_bwd(&b, stream);
}
