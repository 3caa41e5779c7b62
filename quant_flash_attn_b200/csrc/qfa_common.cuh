// Shared device helpers for the qfa kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/qfa.h"

namespace qfa {

// Bumps the library-wide launch counter (reported by qfa_launch_count).
void note_launch(int n = 1);
// Records a failed CUDA call for qfa_last_cuda_error and returns QFA_ERR_CUDA.
int cuda_fail(cudaError_t e, const char* what);

#define QFA_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::qfa::cuda_fail(_e, #expr); \
  } while (0)

// Launch epoch for the kernels with bounded barrier waits: ONE process-wide counter for every launcher, never 0,
// so the epoch a timed-out launch leaves in the device-side abort word is never handed out again.
unsigned int next_launch_epoch();

// One-time set-up of a kernel on the current device (opt-in shared memory size, register checks), usable from
// several host threads at once: `setup` is idempotent, so two threads that race both run it and both succeed.
// Devices beyond kMaxDevices are rejected instead of being launched on without the set-up.
constexpr int kMaxDevices = 64;
struct DeviceOnce {
  std::atomic<bool> done[kMaxDevices];
};
template <typename F>
inline int once_per_device(DeviceOnce& flags, F&& setup) {
  int dev = 0;
  QFA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return cuda_fail(cudaErrorInvalidDevice, "device ordinals above 63 are not supported");
  if (flags.done[dev].load(std::memory_order_acquire)) return QFA_OK;
  const int rc = setup();
  if (rc != QFA_OK) return rc;
  flags.done[dev].store(true, std::memory_order_release);
  return QFA_OK;
}

// ------------------------------------------------------------------ 16-bit type traits
template <typename T>
struct Half16;

template <>
struct Half16<__half> {
  using T = __half;
  using T2 = __half2;
  static __device__ __forceinline__ float to_f32(T v) { return __half2float(v); }
  static __device__ __forceinline__ T from_f32(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
  }
};

template <>
struct Half16<__nv_bfloat16> {
  using T = __nv_bfloat16;
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f32(T v) { return __bfloat162float(v); }
  static __device__ __forceinline__ T from_f32(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
  }
};

// ------------------------------------------------------------------ warp-level MMA (legacy tensor path)
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8,f32) += A(16x16) * B(16x8), 16-bit operands
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D(16x8,s32) += A(16x32,s8) * B(32x8,s8)
__device__ __forceinline__ void mma_16832_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// dequantize 4 packed int8 codes: (c - zp) * scale
__device__ __forceinline__ void dequant4(uint32_t packed, float zp, float scale, float (&out)[4]) {
  out[0] = (static_cast<float>(static_cast<int8_t>(packed & 0xff)) - zp) * scale;
  out[1] = (static_cast<float>(static_cast<int8_t>((packed >> 8) & 0xff)) - zp) * scale;
  out[2] = (static_cast<float>(static_cast<int8_t>((packed >> 16) & 0xff)) - zp) * scale;
  out[3] = (static_cast<float>(static_cast<int8_t>(packed >> 24)) - zp) * scale;
}

// Four int8 codes (one 32-bit word, lowest byte first) minus a zero point, as two packed fp16 pairs.  Exact:
// byte ^ 0x80 is code + 128 as an unsigned byte, 0x6400 | byte is the fp16 number 1024 + byte, 1152 + zp <= 1279 is
// an fp16 integer, and the difference lies in [-255, 255].
__device__ __forceinline__ void center4(uint32_t w, int zp, uint32_t& o01, uint32_t& o23) {
  const __half2 off = __half2half2(__int2half_rn(1152 + zp));
  const uint32_t u = w ^ 0x80808080u;
  const uint32_t a0 = __byte_perm(u, 0x64646464u, 0x4140), a1 = __byte_perm(u, 0x64646464u, 0x4342);
  const __half2 h0 = __hsub2(*reinterpret_cast<const __half2*>(&a0), off);
  const __half2 h1 = __hsub2(*reinterpret_cast<const __half2*>(&a1), off);
  o01 = *reinterpret_cast<const uint32_t*>(&h0);
  o23 = *reinterpret_cast<const uint32_t*>(&h1);
}

__device__ __forceinline__ float half_bits_to_f32(uint16_t bits) {
  return __half2float(__ushort_as_half(bits));
}

}  // namespace qfa
