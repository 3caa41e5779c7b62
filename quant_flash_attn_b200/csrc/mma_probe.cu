// Tensor-pipe rate probe: how fast can ONE thread per SM feed tcgen05.mma when nothing else happens?
//
// The attention kernels are judged against a tensor-core roofline, and the int8 (kind::i8) peak of the part is
// not something a library GEMM reports.  This kernel puts one CTA on every SM, keeps two operand tiles resident
// in shared memory (contents are irrelevant for the rate and are zeroed), and lets one thread issue `iters`
// rounds of four K-steps of 128 x N x K MMAs into two alternating accumulators in tensor memory, with a single
// commit at the end.  No loads, no epilogue: the time is the issue/execute rate of the MMA form itself.
//   form 0: kind::i8  A, B from shared memory (K = 32 per step)       form 1: kind::f16 (bf16) A, B from shared
//   form 2: kind::f16 (bf16) A from tensor memory, B from shared      (K = 16 per step)
// N is 128 or 256.  The wait for the final commit is bounded like every wait of this library.
#include "qfa_common.cuh"
#include "sm100_ptx.cuh"

namespace qfa {

using namespace sm100;

constexpr int kProbeSmem = 16384 + 32768 + 1024;      // A 128 x 128 B, B 256 x 128 B, alignment slack

template <int FORM, int N>
__global__ void __launch_bounds__(128, 1) mma_probe_kernel(int iters, unsigned int epoch, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (16384 + 32768) / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  // generic-proxy writes of the operand tiles must be visible to the tensor core's (async proxy) reads
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const uint32_t sa = smem_u32(smem), sb = sa + 16384;
    const uint64_t da = make_smem_desc(sa, 16, 1024, kSwizzle128B);
    const uint64_t db = make_smem_desc(sb, 16, 1024, kSwizzle128B);
    constexpr uint32_t idesc = (FORM == 0) ? make_idesc(2, 1, 1, 0, 0, 128, N) : make_idesc(1, 1, 1, 0, 0, 128, N);
    // accumulators: [0, N) and [N, 2N) for N = 128; one accumulator [0, 256) for N = 256 when A sits in tensor memory
    const uint32_t acc1 = (FORM == 2 && N == 256) ? 0u : static_cast<uint32_t>(N);
    const uint32_t a_tmem = tmem + 448;                       // 4 steps x 8 columns of 16-bit A, past the accumulators
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem + ((it & 1) ? acc1 : 0u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t acc = (it > 1 || k > 0) ? 1u : 0u;
        if (FORM == 0) mma_i8_ss(d, desc_advance(da, k * 32), desc_advance(db, k * 32), idesc, acc);
        else if (FORM == 1) mma_f16_ss(d, desc_advance(da, k * 32), desc_advance(db, k * 32), idesc, acc);
        else mma_f16_ts(d, a_tmem + k * 8, desc_advance(db, k * 32), idesc, acc);
      }
    }
    mma_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, abort_flag, epoch);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && *abort_flag && status) *status = QFA_STATUS_WAIT_TIMEOUT;
}

template <int FORM, int N>
static int launch_probe(int iters, int n_ctas, int32_t* status, cudaStream_t stream) {
  auto kern = mma_probe_kernel<FORM, N>;
  static DeviceOnce done;
  int rc = once_per_device(done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem));
    return QFA_OK;
  });
  if (rc != QFA_OK) return rc;
  kern<<<n_ctas, 128, kProbeSmem, stream>>>(iters, next_launch_epoch(), status);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

// Launches the probe on every SM of the current device; *ops_out = integer multiply-adds x 2 (or flops) the launch
// performs, so that rate = *ops_out / measured time.
int mma_probe_entry(int form, int n, int iters, double* ops_out, int32_t* status, cudaStream_t stream) {
  if (form < 0 || form > 2 || (n != 128 && n != 256)) return QFA_ERR_MODE;
  if (iters < 2 || iters > 20000) return QFA_ERR_SHAPE;          // at most ~10 ms of tensor work per SM
  int dev = 0, sms = 0;
  QFA_CUDA_TRY(cudaGetDevice(&dev));
  QFA_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int k = form == 0 ? 32 : 16;
  if (ops_out) *ops_out = 2.0 * 128.0 * n * k * 4.0 * iters * sms;
#define QFA_PROBE(F, NN) if (form == F && n == NN) return launch_probe<F, NN>(iters, sms, status, stream)
  QFA_PROBE(0, 128); QFA_PROBE(0, 256); QFA_PROBE(1, 128); QFA_PROBE(1, 256); QFA_PROBE(2, 128); QFA_PROBE(2, 256);
#undef QFA_PROBE
  return QFA_ERR_MODE;
}

}  // namespace qfa
