// Flash-attention forward over quantized K/V using warp-level MMA (mma.sync).
//
// Covers both numeric modes of qfa_attn_fwd for any Sq/Skv (ragged tails included):
//   REF  : logits = (q*sm_scale -> 16 bit) . K^   with K^ = (code-zp)*scale rounded to 16 bit,
//          i.e. what _attn_fwd_kernel_quantized computes (quant_flash_attn.py:50-83)
//   INT8 : logits = s_q s_k (q.k - z_k*sum(q) - z_q*sum(k) + D z_q z_k) * sm_scale from an
//          int8 x int8 -> int32 MMA on the codes
// P.V runs on 16-bit MMAs with V dequantized and rounded to 16 bit while it is staged into
// shared memory (quant_flash_attn.py:65-66,75).  One CTA = 64 query rows of one (batch, head);
// 4 warps x 16 rows; K/V tiles of 64 tokens are prefetched into registers while the previous
// tile is being consumed.  This is the general-shape kernel (short-Q reference shapes, ragged
// lengths); the tcgen05 kernel in attn_fwd_tc.cu takes over for tile-aligned int8 problems.
#include "qfa_common.cuh"

namespace qfa {

struct FwdDev {
  const void* q;
  int64_t q_stride[3];
  QfaQuantTensor qq, k, v;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride;
  int H, Sq, Skv;
  float sm_scale;
  int causal;
  int kv_shared;  // REF mode and k, v are the same tensor: stage it once
};

template <int D, bool INT8>
struct FwdCfg {
  static constexpr int BM = 64, BN = 64, WARPS = 4, THREADS = 128;
  static constexpr int QK_ROW_BYTES = INT8 ? D : 2 * D;      // bytes of one Q / K row as MMA operand
  static constexpr int QK_STRIDE = QK_ROW_BYTES + 16;        // padded: conflict-free ldmatrix
  static constexpr int V_STRIDE = 2 * D + 16;
  static constexpr int KSTEPS = QK_ROW_BYTES / 32;           // 32 operand bytes per MMA k-step
  static constexpr int CHUNKS = BN * D / 16 / THREADS;       // 16-code chunks per thread per tile
  static constexpr int CHUNKS_PER_ROW = D / 16;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + BM * QK_STRIDE;
  static constexpr int V_OFF = K_OFF + BN * QK_STRIDE;
  static constexpr int META_OFF = V_OFF + BN * V_STRIDE;     // float ks[BN]; int kz[BN]; int ksum[BN]
  static constexpr int SMEM = META_OFF + 3 * BN * 4;
};

template <typename T>
__device__ __forceinline__ void store_dequant16(uint8_t* dst, const uint4& codes, float zp, float scale) {
  using H16 = Half16<T>;
  float f[4];
  uint4 lo, hi;
  dequant4(codes.x, zp, scale, f); lo.x = H16::pack(f[0], f[1]); lo.y = H16::pack(f[2], f[3]);
  dequant4(codes.y, zp, scale, f); lo.z = H16::pack(f[0], f[1]); lo.w = H16::pack(f[2], f[3]);
  dequant4(codes.z, zp, scale, f); hi.x = H16::pack(f[0], f[1]); hi.y = H16::pack(f[2], f[3]);
  dequant4(codes.w, zp, scale, f); hi.z = H16::pack(f[0], f[1]); hi.w = H16::pack(f[2], f[3]);
  *reinterpret_cast<uint4*>(dst) = lo;
  *reinterpret_cast<uint4*>(dst + 16) = hi;
}

template <typename T, int D, bool INT8>
__global__ void __launch_bounds__(128) attn_fwd_mma_kernel(FwdDev p) {
  using C = FwdCfg<D, INT8>;
  using H16 = Half16<T>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sQ = smem + C::Q_OFF;
  uint8_t* sK = smem + C::K_OFF;
  uint8_t* sV = smem + C::V_OFF;
  float* sKs = reinterpret_cast<float*>(smem + C::META_OFF);
  int* sKz = reinterpret_cast<int*>(smem + C::META_OFF + C::BN * 4);
  int* sKsum = reinterpret_cast<int*>(smem + C::META_OFF + 2 * C::BN * 4);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m_blocks = (p.Sq + C::BM - 1) / C::BM;
  const int bh = blockIdx.x / m_blocks;
  const int b = bh / p.H, h = bh % p.H;
  const int m0 = (blockIdx.x % m_blocks) * C::BM;
  const int64_t tok_q0 = static_cast<int64_t>(bh) * p.Sq;    // flat token index of row 0 of this head
  const int64_t tok_k0 = static_cast<int64_t>(bh) * p.Skv;

  const int8_t* kc = p.k.codes + b * p.k.stride[0] + h * p.k.stride[1];
  const int8_t* vc = p.v.codes + b * p.v.stride[0] + h * p.v.stride[1];

  // ---------------- stage Q
  if (INT8) {
    const int8_t* qc = p.qq.codes + b * p.qq.stride[0] + h * p.qq.stride[1];
    for (int c = tid; c < C::BM * C::CHUNKS_PER_ROW; c += C::THREADS) {
      int r = c / C::CHUNKS_PER_ROW, cc = c % C::CHUNKS_PER_ROW;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m0 + r < p.Sq) v = *reinterpret_cast<const uint4*>(qc + (m0 + r) * p.qq.stride[2] + cc * 16);
      *reinterpret_cast<uint4*>(sQ + r * C::QK_STRIDE + cc * 16) = v;
    }
  } else {
    const T* q = static_cast<const T*>(p.q) + b * p.q_stride[0] + h * p.q_stride[1];
    for (int c = tid; c < C::BM * (D / 8); c += C::THREADS) {
      int r = c / (D / 8), cc = c % (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m0 + r < p.Sq) v = *reinterpret_cast<const uint4*>(q + (m0 + r) * p.q_stride[2] + cc * 8);
      // q = (q * sm_scale).to(q_dtype)  (quant_flash_attn.py:52)
      float2 f;
      f = H16::unpack(v.x); v.x = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.y); v.y = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.z); v.z = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.w); v.w = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      *reinterpret_cast<uint4*>(sQ + r * C::QK_STRIDE + cc * 16) = v;
    }
  }

  // per-row constants of the two rows this thread owns (INT8)
  const int row_l[2] = {warp * 16 + g, warp * 16 + g + 8};
  int q_z[2] = {0, 0}, q_a[2] = {0, 0};
  float q_f[2] = {0.f, 0.f};
  if (INT8) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int row = m0 + row_l[r];
      if (row < p.Sq) {
        int64_t tk = tok_q0 + row;
        q_z[r] = p.qq.zp[tk];
        q_a[r] = D * q_z[r] - p.qq.rowsum[tk];
        q_f[r] = half_bits_to_f32(p.qq.scale[tk]) * p.sm_scale * kLog2e;
      }
    }
  }

  int kv_end = p.Skv;
  if (p.causal) kv_end = min(p.Skv, m0 + C::BM);
  const int n_tiles = (kv_end + C::BN - 1) / C::BN;

  // register prefetch buffers
  uint4 kreg[C::CHUNKS], vreg[C::CHUNKS];
  float ksc[C::CHUNKS], kzp[C::CHUNKS], vsc[C::CHUNKS], vzp[C::CHUNKS];
  float meta_s = 0.f;
  int meta_z = 0, meta_sum = 0;

  auto prefetch = [&](int tile) {
    const int n0 = tile * C::BN;
#pragma unroll
    for (int i = 0; i < C::CHUNKS; ++i) {
      int c = tid + i * C::THREADS;
      int r = c / C::CHUNKS_PER_ROW, cc = c % C::CHUNKS_PER_ROW;
      int n = n0 + r;
      bool ok = n < p.Skv;
      kreg[i] = make_uint4(0, 0, 0, 0);
      vreg[i] = make_uint4(0, 0, 0, 0);
      ksc[i] = 0.f; kzp[i] = 0.f; vsc[i] = 0.f; vzp[i] = 0.f;
      if (ok) {
        if (INT8 || !p.kv_shared) {
          kreg[i] = __ldg(reinterpret_cast<const uint4*>(kc + n * p.k.stride[2] + cc * 16));
          if (!INT8) {
            ksc[i] = half_bits_to_f32(p.k.scale[tok_k0 + n]);
            kzp[i] = static_cast<float>(p.k.zp[tok_k0 + n]);
          }
        }
        vreg[i] = __ldg(reinterpret_cast<const uint4*>(vc + n * p.v.stride[2] + cc * 16));
        vsc[i] = half_bits_to_f32(p.v.scale[tok_k0 + n]);
        vzp[i] = static_cast<float>(p.v.zp[tok_k0 + n]);
      }
    }
    if (INT8 && tid < C::BN) {
      int n = n0 + tid;
      meta_s = 0.f; meta_z = 0; meta_sum = 0;
      if (n < p.Skv) {
        meta_s = half_bits_to_f32(p.k.scale[tok_k0 + n]);
        meta_z = p.k.zp[tok_k0 + n];
        meta_sum = p.k.rowsum[tok_k0 + n];
      }
    }
  };

  auto commit = [&]() {
#pragma unroll
    for (int i = 0; i < C::CHUNKS; ++i) {
      int c = tid + i * C::THREADS;
      int r = c / C::CHUNKS_PER_ROW, cc = c % C::CHUNKS_PER_ROW;
      if (INT8) {
        *reinterpret_cast<uint4*>(sK + r * C::QK_STRIDE + cc * 16) = kreg[i];
      } else if (!p.kv_shared) {
        store_dequant16<T>(sK + r * C::QK_STRIDE + cc * 32, kreg[i], kzp[i], ksc[i]);
      }
      store_dequant16<T>(sV + r * C::V_STRIDE + cc * 32, vreg[i], vzp[i], vsc[i]);
    }
    if (INT8 && tid < C::BN) {
      sKs[tid] = meta_s;
      sKz[tid] = meta_z;
      sKsum[tid] = meta_sum;
    }
  };

  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  const uint8_t* sKop = (!INT8 && p.kv_shared) ? sV : sK;
  const int k_stride = (!INT8 && p.kv_shared) ? C::V_STRIDE : C::QK_STRIDE;

  if (n_tiles > 0) prefetch(0);
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int n0 = tile * C::BN;
    __syncthreads();
    commit();
    __syncthreads();
    if (tile + 1 < n_tiles) prefetch(tile + 1);

    // ---------------- S = Q K^T for this warp's 16 rows
    float s[8][4];
    {
      int acc_i[8][4];
      float acc_f[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc_i[i][e] = 0; acc_f[i][e] = 0.f; }
      const uint32_t a_base = smem_u32(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::QK_STRIDE +
                                       ((lane >> 4) & 1) * 16);
      const uint32_t b_base = smem_u32(sKop + ((lane & 7) + ((lane >> 4) & 1) * 8) * k_stride + ((lane >> 3) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < C::KSTEPS; ++kk) {
        uint32_t a[4];
        ldsm_x4(a_base + kk * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b_base + np * 16 * k_stride + kk * 32, b0, b1, b2, b3);
          if (INT8) {
            mma_16832_s8(acc_i[2 * np], a, b0, b1);
            mma_16832_s8(acc_i[2 * np + 1], a, b2, b3);
          } else {
            mma_16816<T>(acc_f[2 * np], a, b0, b1);
            mma_16816<T>(acc_f[2 * np + 1], a, b2, b3);
          }
        }
      }
      if (INT8) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            int col = nt * 8 + 2 * t + e;
            int kz = sKz[col], ksum = sKsum[col];
            float ks = sKs[col];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              int v = acc_i[nt][r * 2 + e] + kz * q_a[r] - q_z[r] * ksum;
              s[nt][r * 2 + e] = static_cast<float>(v) * (q_f[r] * ks);
            }
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[nt][e] = acc_f[nt][e] * kLog2e;
      }
    }

    // ---------------- masks (ragged KV tail, causal diagonal)
    const bool need_mask = (n0 + C::BN > p.Skv) || (p.causal && n0 + C::BN - 1 > m0);
    if (need_mask) {
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = n0 + nt * 8 + 2 * t + (e & 1);
          int row = m0 + row_l[e >> 1];
          if (col >= p.Skv || (p.causal && col > row)) s[nt][e] = -INFINITY;
        }
    }

    // ---------------- online softmax (base-2 domain)
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      float m_new = fmaxf(m_run[r], mx);
      float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = fast_exp2(m_run[r] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][2 * r] = fast_exp2(s[nt][2 * r] - m_use);
        s[nt][2 * r + 1] = fast_exp2(s[nt][2 * r + 1] - m_use);
        sum += s[nt][2 * r] + s[nt][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha[r] + sum;
      m_run[r] = m_new;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
    }

    // ---------------- O += P V  (P rounded to 16 bit, quant_flash_attn.py:75)
    const uint32_t v_base = smem_u32(sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::V_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = H16::pack(s[2 * kk][0], s[2 * kk][1]);
      a[1] = H16::pack(s[2 * kk][2], s[2 * kk][3]);
      a[2] = H16::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = H16::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_base + kk * 16 * C::V_STRIDE + dp * 32, b0, b1, b2, b3);
        mma_16816<T>(o_acc[2 * dp], a, b0, b1);
        mma_16816<T>(o_acc[2 * dp + 1], a, b2, b3);
      }
    }
  }

  // ---------------- epilogue: normalise, store O and LSE = m + log(l)  (quant_flash_attn.py:77-83)
  T* o = static_cast<T*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int row = m0 + row_l[r];
    if (row < p.Sq) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        uint32_t packed = H16::pack(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
        *reinterpret_cast<uint32_t*>(o + row * p.o_stride[2] + i * 8 + 2 * t) = packed;
      }
      if (t == 0) p.lse[static_cast<int64_t>(bh) * p.lse_stride + row] = (m_run[r] + log2f(l)) * kLn2;
    }
  }
}

template <typename T, int D, bool INT8>
static int launch_fwd(const FwdDev& dev, int B, cudaStream_t stream) {
  using C = FwdCfg<D, INT8>;
  auto kern = attn_fwd_mma_kernel<T, D, INT8>;
  static DeviceOnce attr_done;
  int rc = once_per_device(attr_done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    return QFA_OK;
  });
  if (rc != QFA_OK) return rc;
  const int64_t n_ctas = static_cast<int64_t>((dev.Sq + C::BM - 1) / C::BM) * B * dev.H;
  if (n_ctas > 0x7fffffffLL) return QFA_ERR_SHAPE;
  kern<<<static_cast<unsigned>(n_ctas), C::THREADS, C::SMEM, stream>>>(dev);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

int attn_fwd_mma_entry(const QfaFwdArgs& a, cudaStream_t stream) {
  FwdDev d;
  d.q = a.q;
  for (int i = 0; i < 3; ++i) { d.q_stride[i] = a.q_stride[i]; d.o_stride[i] = a.o_stride[i]; }
  d.qq = a.qq; d.k = a.k; d.v = a.v;
  d.o = a.o; d.lse = a.lse; d.lse_stride = a.lse_stride;
  d.H = static_cast<int>(a.H); d.Sq = static_cast<int>(a.Sq); d.Skv = static_cast<int>(a.Skv);
  d.sm_scale = a.sm_scale; d.causal = a.causal;
  d.kv_shared = (a.mode == QFA_MODE_REF && a.k.codes == a.v.codes && a.k.scale == a.v.scale && a.k.zp == a.v.zp &&
                 a.k.stride[0] == a.v.stride[0] && a.k.stride[1] == a.v.stride[1] && a.k.stride[2] == a.v.stride[2]);
  const int B = static_cast<int>(a.B);
  const bool i8 = a.mode == QFA_MODE_INT8;
  const bool bf = a.dtype == QFA_BF16;
  if (a.D == 64) {
    if (i8) return bf ? launch_fwd<__nv_bfloat16, 64, true>(d, B, stream) : launch_fwd<__half, 64, true>(d, B, stream);
    return bf ? launch_fwd<__nv_bfloat16, 64, false>(d, B, stream) : launch_fwd<__half, 64, false>(d, B, stream);
  }
  if (a.D == 128) {
    if (i8) return bf ? launch_fwd<__nv_bfloat16, 128, true>(d, B, stream) : launch_fwd<__half, 128, true>(d, B, stream);
    return bf ? launch_fwd<__nv_bfloat16, 128, false>(d, B, stream) : launch_fwd<__half, 128, false>(d, B, stream);
  }
  return QFA_ERR_HEAD_DIM;
}

}  // namespace qfa
