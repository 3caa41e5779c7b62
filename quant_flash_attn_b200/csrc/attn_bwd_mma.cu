// Flash-attention backward over quantized K/V using warp-level MMA (mma.sync).
//
//   delta pre-pass  : delta[row] = sum_d O*dO                       (quant_flash_attn.py:88-101)
//   main kernel     : P = exp(S - LSE) recomputed per tile pair     (quant_flash_attn.py:153-155)
//                     dV += P^T dO, dP = dO V^^T, dS = P*(dP-delta) (quant_flash_attn.py:156-158)
//                     dQ += dS K^, dK += dS^T Q                     (quant_flash_attn.py:159-160)
//   finalize        : dq = sm_scale * dq_accum -> 16 bit            (quant_flash_attn.py:164-166)
//
// Work decomposition: one CTA owns 64 K/V tokens of one (batch, head) and walks over the query
// tiles (the reference walks KV blocks inside one CTA per head, quant_flash_attn.py:141).  dK and
// dV stay in registers for the whole walk; dQ tiles are added into an fp32 scratch tensor with
// vector atomics because several KV tiles contribute to the same query rows.  Everything is
// computed transposed (S^T = K Q^T), so P^T and dS^T come out of the MMA already in the register
// layout the dV / dK products need as their left operand.
//
// REF mode follows the reference formulas literally (16-bit q, one tensor as K and V, fused
// dKV = dV + sm_scale*dK, quant_flash_attn.py:161).  INT8 mode recomputes S through the same
// int8 x int8 MMA + zero-point correction as the forward, uses the dequantized Q^/K^/V^ for the
// four 16-bit products and returns dK, dV separately.
#include "qfa_common.cuh"

namespace qfa {

struct BwdDev {
  const void* q;
  int64_t q_stride[3];
  QfaQuantTensor qq, k, v;
  const void* d_o;
  int64_t do_stride[3];
  const float* lse;
  const float* delta;
  int64_t lse_stride;
  void* dk;
  int64_t dk_stride[3];
  void* dv;
  int64_t dv_stride[3];
  float* dq_accum;  // (B,H,Sq,D) fp32 contiguous
  int H, Sq, Skv;
  float sm_scale;
  int causal, dkv_fused, kv_shared;
};

template <int D, bool INT8>
struct BwdCfg {
  static constexpr int BN = 64;                        // K/V tokens per CTA
  static constexpr int BM = (D == 128) ? 32 : 64;      // query rows per step
  static constexpr int THREADS = 128;
  static constexpr int C_STRIDE = D + 16;              // int8 rows
  static constexpr int T_STRIDE = 2 * D + 16;          // 16-bit rows
  static constexpr int DS_STRIDE = 2 * BM + 16;
  static constexpr int KC_OFF = 0;                                     // int8 K codes      (INT8)
  static constexpr int KS_OFF = KC_OFF + (INT8 ? BN * C_STRIDE : 0);   // K^ 16 bit
  static constexpr int VS_OFF = KS_OFF + BN * T_STRIDE;                // V^ 16 bit
  static constexpr int QC_OFF = VS_OFF + BN * T_STRIDE;                // int8 Q codes      (INT8)
  static constexpr int QS_OFF = QC_OFF + (INT8 ? BM * C_STRIDE : 0);   // Q / Q^ 16 bit
  static constexpr int DO_OFF = QS_OFF + BM * T_STRIDE;                // dO 16 bit
  static constexpr int DS_OFF = DO_OFF + BM * T_STRIDE;                // dS^T 16 bit [kv][q]
  static constexpr int ROW_OFF = DS_OFF + BN * DS_STRIDE;              // lse2[BM], delta[BM], qf[BM], qz[BM], qsum[BM]
  static constexpr int SMEM = ROW_OFF + 5 * BM * 4;
};

template <typename T>
__device__ __forceinline__ void store_dequant16_b(uint8_t* dst, const uint4& codes, float zp, float scale) {
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
__global__ void __launch_bounds__(128) attn_bwd_mma_kernel(BwdDev p) {
  using C = BwdCfg<D, INT8>;
  using H16 = Half16<T>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sKc = smem + C::KC_OFF;
  uint8_t* sKs = smem + C::KS_OFF;
  uint8_t* sVs = smem + C::VS_OFF;
  uint8_t* sQc = smem + C::QC_OFF;
  uint8_t* sQs = smem + C::QS_OFF;
  uint8_t* sDO = smem + C::DO_OFF;
  uint8_t* sDS = smem + C::DS_OFF;
  float* sLse2 = reinterpret_cast<float*>(smem + C::ROW_OFF);
  float* sDelta = sLse2 + C::BM;
  float* sQf = sDelta + C::BM;
  int* sQz = reinterpret_cast<int*>(sQf + C::BM);
  int* sQsum = sQz + C::BM;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_blocks = (p.Skv + C::BN - 1) / C::BN;
  const int bh = blockIdx.x / n_blocks;
  const int b = bh / p.H, h = bh % p.H;
  const int n0 = (blockIdx.x % n_blocks) * C::BN;
  const int64_t tok_q0 = static_cast<int64_t>(bh) * p.Sq;
  const int64_t tok_k0 = static_cast<int64_t>(bh) * p.Skv;
  constexpr int CPR = D / 16;  // 16-code chunks per row

  // ---------------- stage K codes / K^ / V^ once
  {
    const int8_t* kc = p.k.codes + b * p.k.stride[0] + h * p.k.stride[1];
    const int8_t* vc = p.v.codes + b * p.v.stride[0] + h * p.v.stride[1];
    for (int c = tid; c < C::BN * CPR; c += C::THREADS) {
      int r = c / CPR, cc = c % CPR;
      int n = n0 + r;
      uint4 kq = make_uint4(0, 0, 0, 0), vq = make_uint4(0, 0, 0, 0);
      float ks = 0.f, kz = 0.f, vs = 0.f, vz = 0.f;
      if (n < p.Skv) {
        kq = *reinterpret_cast<const uint4*>(kc + n * p.k.stride[2] + cc * 16);
        ks = half_bits_to_f32(p.k.scale[tok_k0 + n]);
        kz = static_cast<float>(p.k.zp[tok_k0 + n]);
        if (!p.kv_shared) {
          vq = *reinterpret_cast<const uint4*>(vc + n * p.v.stride[2] + cc * 16);
          vs = half_bits_to_f32(p.v.scale[tok_k0 + n]);
          vz = static_cast<float>(p.v.zp[tok_k0 + n]);
        }
      }
      if (INT8) *reinterpret_cast<uint4*>(sKc + r * C::C_STRIDE + cc * 16) = kq;
      store_dequant16_b<T>(sKs + r * C::T_STRIDE + cc * 32, kq, kz, ks);
      if (!p.kv_shared) store_dequant16_b<T>(sVs + r * C::T_STRIDE + cc * 32, vq, vz, vs);
    }
  }
  const uint8_t* sVop = p.kv_shared ? sKs : sVs;

  // per-row (kv) constants of the two rows this thread owns
  const int row_l[2] = {warp * 16 + g, warp * 16 + g + 8};
  int k_z[2] = {0, 0}, k_b[2] = {0, 0};
  float k_s[2] = {0.f, 0.f};
  if (INT8) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int n = n0 + row_l[r];
      if (n < p.Skv) {
        k_z[r] = p.k.zp[tok_k0 + n];
        k_b[r] = D * k_z[r] - p.k.rowsum[tok_k0 + n];
        k_s[r] = half_bits_to_f32(p.k.scale[tok_k0 + n]);
      }
    }
  }

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) { dk_acc[i][e] = 0.f; dv_acc[i][e] = 0.f; }

  const T* qg = INT8 ? nullptr : static_cast<const T*>(p.q) + b * p.q_stride[0] + h * p.q_stride[1];
  const int8_t* qcg = INT8 ? p.qq.codes + b * p.qq.stride[0] + h * p.qq.stride[1] : nullptr;
  const T* dog = static_cast<const T*>(p.d_o) + b * p.do_stride[0] + h * p.do_stride[1];
  float* dqa = p.dq_accum + tok_q0 * D;

  const int m_tiles = (p.Sq + C::BM - 1) / C::BM;
  const int m_first = p.causal ? (n0 / C::BM) : 0;   // first query tile with a row >= n0

  for (int mt = m_first; mt < m_tiles; ++mt) {
    const int m0 = mt * C::BM;
    __syncthreads();  // previous step's readers are done (also orders the K/V staging above)
    // ---------------- stage Q (codes + 16-bit), dO, LSE, delta
    if (INT8) {
      for (int c = tid; c < C::BM * CPR; c += C::THREADS) {
        int r = c / CPR, cc = c % CPR;
        int m = m0 + r;
        uint4 qq = make_uint4(0, 0, 0, 0);
        float qs = 0.f, qz = 0.f;
        if (m < p.Sq) {
          qq = *reinterpret_cast<const uint4*>(qcg + m * p.qq.stride[2] + cc * 16);
          qs = half_bits_to_f32(p.qq.scale[tok_q0 + m]);
          qz = static_cast<float>(p.qq.zp[tok_q0 + m]);
        }
        *reinterpret_cast<uint4*>(sQc + r * C::C_STRIDE + cc * 16) = qq;
        store_dequant16_b<T>(sQs + r * C::T_STRIDE + cc * 32, qq, qz, qs);
      }
    } else {
      for (int c = tid; c < C::BM * (D / 8); c += C::THREADS) {
        int r = c / (D / 8), cc = c % (D / 8);
        int m = m0 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < p.Sq) v = *reinterpret_cast<const uint4*>(qg + m * p.q_stride[2] + cc * 8);
        *reinterpret_cast<uint4*>(sQs + r * C::T_STRIDE + cc * 16) = v;
      }
    }
    for (int c = tid; c < C::BM * (D / 8); c += C::THREADS) {
      int r = c / (D / 8), cc = c % (D / 8);
      int m = m0 + r;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < p.Sq) v = *reinterpret_cast<const uint4*>(dog + m * p.do_stride[2] + cc * 8);
      *reinterpret_cast<uint4*>(sDO + r * C::T_STRIDE + cc * 16) = v;
    }
    if (tid < C::BM) {
      int m = m0 + tid;
      bool ok = m < p.Sq;
      // +inf LSE makes P exactly 0 for rows past the end
      sLse2[tid] = ok ? p.lse[static_cast<int64_t>(bh) * p.lse_stride + m] * kLog2e : INFINITY;
      sDelta[tid] = ok ? p.delta[static_cast<int64_t>(bh) * p.lse_stride + m] : 0.f;
      if (INT8) {
        sQf[tid] = ok ? half_bits_to_f32(p.qq.scale[tok_q0 + m]) * p.sm_scale * kLog2e : 0.f;
        sQz[tid] = ok ? static_cast<int>(p.qq.zp[tok_q0 + m]) : 0;
        sQsum[tid] = ok ? p.qq.rowsum[tok_q0 + m] : 0;
      }
    }
    __syncthreads();

    // ---------------- S^T = K Q^T (16 kv rows x BM query columns per warp)
    constexpr int NT = C::BM / 8;
    float pt[NT][4];
    {
      int acc_i[NT][4];
      float acc_f[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc_i[i][e] = 0; acc_f[i][e] = 0.f; }
      const uint8_t* aop = INT8 ? sKc : sKs;
      const uint8_t* bop = INT8 ? sQc : sQs;
      constexpr int STRIDE = INT8 ? C::C_STRIDE : C::T_STRIDE;
      constexpr int KSTEPS = (INT8 ? D : 2 * D) / 32;
      const uint32_t a_base =
          smem_u32(aop + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + ((lane >> 4) & 1) * 16);
      const uint32_t b_base = smem_u32(bop + ((lane & 7) + ((lane >> 4) & 1) * 8) * STRIDE + ((lane >> 3) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t a[4];
        ldsm_x4(a_base + kk * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b_base + np * 16 * STRIDE + kk * 32, b0, b1, b2, b3);
          if (INT8) {
            mma_16832_s8(acc_i[2 * np], a, b0, b1);
            mma_16832_s8(acc_i[2 * np + 1], a, b2, b3);
          } else {
            mma_16816<T>(acc_f[2 * np], a, b0, b1);
            mma_16816<T>(acc_f[2 * np + 1], a, b2, b3);
          }
        }
      }
      // P^T = exp2(S^T*log2e - LSE*log2e), masked
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = nt * 8 + 2 * t + (e & 1);   // query index inside the tile
          const int r = e >> 1;
          float s2;
          if (INT8) {
            int v = acc_i[nt][e] + sQz[col] * k_b[r] - k_z[r] * sQsum[col];
            s2 = static_cast<float>(v) * (sQf[col] * k_s[r]);
          } else {
            s2 = acc_f[nt][e] * (p.sm_scale * kLog2e);   // qk * sm_scale (quant_flash_attn.py:153)
          }
          float pv = fast_exp2(s2 - sLse2[col]);
          const int kvrow = n0 + row_l[r];
          if (kvrow >= p.Skv || (p.causal && kvrow > m0 + col)) pv = 0.f;
          pt[nt][e] = pv;
        }
    }

    // ---------------- dV += P^T dO   (left operand from registers, dO read transposed)
    {
      const uint32_t b_base = smem_u32(sDO + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < C::BM / 16; ++kk) {
        uint32_t a[4];
        a[0] = H16::pack(pt[2 * kk][0], pt[2 * kk][1]);
        a[1] = H16::pack(pt[2 * kk][2], pt[2 * kk][3]);
        a[2] = H16::pack(pt[2 * kk + 1][0], pt[2 * kk + 1][1]);
        a[3] = H16::pack(pt[2 * kk + 1][2], pt[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(b_base + kk * 16 * C::T_STRIDE + dp * 32, b0, b1, b2, b3);
          mma_16816<T>(dv_acc[2 * dp], a, b0, b1);
          mma_16816<T>(dv_acc[2 * dp + 1], a, b2, b3);
        }
      }
    }

    // ---------------- dP^T = V^ dO^T, dS^T = P^T * (dP^T - delta)
    {
      float dp_acc[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i) dp_acc[i][0] = dp_acc[i][1] = dp_acc[i][2] = dp_acc[i][3] = 0.f;
      const uint32_t a_base =
          smem_u32(sVop + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
      const uint32_t b_base = smem_u32(sDO + ((lane & 7) + ((lane >> 4) & 1) * 8) * C::T_STRIDE + ((lane >> 3) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(a_base + kk * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(b_base + np * 16 * C::T_STRIDE + kk * 32, b0, b1, b2, b3);
          mma_16816<T>(dp_acc[2 * np], a, b0, b1);
          mma_16816<T>(dp_acc[2 * np + 1], a, b2, b3);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = nt * 8 + 2 * t + (e & 1);
          pt[nt][e] = pt[nt][e] * (dp_acc[nt][e] - sDelta[col]);   // now dS^T
        }
    }

    // dS^T -> shared (for dQ), and as left operand of dK += dS^T Q
    {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint32_t lo = H16::pack(pt[nt][0], pt[nt][1]);
        uint32_t hi = H16::pack(pt[nt][2], pt[nt][3]);
        *reinterpret_cast<uint32_t*>(sDS + row_l[0] * C::DS_STRIDE + (nt * 8 + 2 * t) * 2) = lo;
        *reinterpret_cast<uint32_t*>(sDS + row_l[1] * C::DS_STRIDE + (nt * 8 + 2 * t) * 2) = hi;
      }
      const uint32_t b_base = smem_u32(sQs + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < C::BM / 16; ++kk) {
        uint32_t a[4];
        a[0] = H16::pack(pt[2 * kk][0], pt[2 * kk][1]);
        a[1] = H16::pack(pt[2 * kk][2], pt[2 * kk][3]);
        a[2] = H16::pack(pt[2 * kk + 1][0], pt[2 * kk + 1][1]);
        a[3] = H16::pack(pt[2 * kk + 1][2], pt[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(b_base + kk * 16 * C::T_STRIDE + dp * 32, b0, b1, b2, b3);
          mma_16816<T>(dk_acc[2 * dp], a, b0, b1);
          mma_16816<T>(dk_acc[2 * dp + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();

    // ---------------- dQ tile = dS K^ ; warp w owns D/4 columns, all BM rows
    {
      constexpr int DW = D / 4;          // columns per warp
      constexpr int MT = C::BM / 16;
      constexpr int NP = DW / 16;
      float dq_acc[MT][2 * NP][4];
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 2 * NP; ++j) dq_acc[i][j][0] = dq_acc[i][j][1] = dq_acc[i][j][2] = dq_acc[i][j][3] = 0.f;
      // A = dS (rows = query, k = kv) read from dS^T[kv][q] with the transposing load
      const uint32_t a_base = smem_u32(sDS + ((lane & 7) + ((lane >> 4) & 1) * 8) * C::DS_STRIDE + ((lane >> 3) & 1) * 16);
      const uint32_t b_base = smem_u32(sKs + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE +
                                       (warp * DW) * 2 + ((lane >> 4) & 1) * 16);
#pragma unroll
      for (int kk = 0; kk < C::BN / 16; ++kk) {
        uint32_t bfr[NP][4];
#pragma unroll
        for (int np = 0; np < NP; ++np)
          ldsm_x4_t(b_base + kk * 16 * C::T_STRIDE + np * 32, bfr[np][0], bfr[np][1], bfr[np][2], bfr[np][3]);
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
          uint32_t a[4];
          ldsm_x4_t(a_base + kk * 16 * C::DS_STRIDE + mi * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
          for (int np = 0; np < NP; ++np) {
            mma_16816<T>(dq_acc[mi][2 * np], a, bfr[np][0], bfr[np][1]);
            mma_16816<T>(dq_acc[mi][2 * np + 1], a, bfr[np][2], bfr[np][3]);
          }
        }
      }
#pragma unroll
      for (int mi = 0; mi < MT; ++mi)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int m = m0 + mi * 16 + g + r * 8;
          if (m < p.Sq) {
#pragma unroll
            for (int j = 0; j < 2 * NP; ++j) {
              float2 v = make_float2(dq_acc[mi][j][2 * r], dq_acc[mi][j][2 * r + 1]);
              atomicAdd(reinterpret_cast<float2*>(dqa + static_cast<int64_t>(m) * D + warp * DW + j * 8 + 2 * t), v);
            }
          }
        }
    }
  }

  // ---------------- epilogue: dK (scaled), dV, or the reference's fused dKV = dV + sm_scale*dK
  T* dkg = static_cast<T*>(p.dk) + b * p.dk_stride[0] + h * p.dk_stride[1];
  T* dvg = p.dkv_fused ? nullptr : static_cast<T*>(p.dv) + b * p.dv_stride[0] + h * p.dv_stride[1];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int n = n0 + row_l[r];
    if (n < p.Skv) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        float k0 = dk_acc[i][2 * r] * p.sm_scale, k1 = dk_acc[i][2 * r + 1] * p.sm_scale;
        float v0 = dv_acc[i][2 * r], v1 = dv_acc[i][2 * r + 1];
        if (p.dkv_fused) {
          *reinterpret_cast<uint32_t*>(dkg + n * p.dk_stride[2] + i * 8 + 2 * t) = H16::pack(v0 + k0, v1 + k1);
        } else {
          *reinterpret_cast<uint32_t*>(dkg + n * p.dk_stride[2] + i * 8 + 2 * t) = H16::pack(k0, k1);
          *reinterpret_cast<uint32_t*>(dvg + n * p.dv_stride[2] + i * 8 + 2 * t) = H16::pack(v0, v1);
        }
      }
    }
  }
}

// delta[row] = sum_d O * dO : one warp per row, 16-byte loads.  The reference multiplies in the
// 16-bit dtype before summing (quant_flash_attn.py:99); the product is formed in fp32 here.
template <typename T>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                        float* __restrict__ delta, int64_t so0, int64_t so1,
                                                        int64_t so2, int64_t sd0, int64_t sd1, int64_t sd2,
                                                        int64_t delta_stride, int H, int Sq, int D, int64_t rows) {
  using H16 = Half16<T>;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int m = static_cast<int>(row % Sq);
  const int64_t bh = row / Sq;
  const int h = static_cast<int>(bh % H);
  const int64_t b = bh / H;
  const T* op = o + b * so0 + h * so1 + m * so2;
  const T* dp = d_o + b * sd0 + h * sd1 + m * sd2;
  float acc = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    uint4 a = *reinterpret_cast<const uint4*>(op + c);
    uint4 d = *reinterpret_cast<const uint4*>(dp + c);
    float2 x, y;
    x = H16::unpack(a.x); y = H16::unpack(d.x); acc += x.x * y.x + x.y * y.y;
    x = H16::unpack(a.y); y = H16::unpack(d.y); acc += x.x * y.x + x.y * y.y;
    x = H16::unpack(a.z); y = H16::unpack(d.z); acc += x.x * y.x + x.y * y.y;
    x = H16::unpack(a.w); y = H16::unpack(d.w); acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[bh * delta_stride + m] = acc;
}

// dq = sm_scale * dq_accum, rounded to 16 bit (quant_flash_attn.py:164-166)
template <typename T>
__global__ void __launch_bounds__(256) bwd_dq_finalize_kernel(const float* __restrict__ acc, T* __restrict__ dq,
                                                              int64_t s0, int64_t s1, int64_t s2, int H, int Sq, int D,
                                                              float sm_scale, int64_t n_vec) {
  using H16 = Half16<T>;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const int vpr = D / 4;
  const int64_t row = i / vpr;
  const int c = static_cast<int>(i % vpr) * 4;
  const int m = static_cast<int>(row % Sq);
  const int64_t bh = row / Sq;
  const int h = static_cast<int>(bh % H);
  const int64_t b = bh / H;
  float4 v = *reinterpret_cast<const float4*>(acc + row * D + c);
  uint2 out;
  out.x = H16::pack(v.x * sm_scale, v.y * sm_scale);
  out.y = H16::pack(v.z * sm_scale, v.w * sm_scale);
  *reinterpret_cast<uint2*>(dq + b * s0 + h * s1 + m * s2 + c) = out;
}

template <typename T, int D, bool INT8>
static int launch_bwd(const BwdDev& dev, int B, cudaStream_t stream) {
  using C = BwdCfg<D, INT8>;
  auto kern = attn_bwd_mma_kernel<T, D, INT8>;
  static DeviceOnce attr_done;
  int rc = once_per_device(attr_done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    return QFA_OK;
  });
  if (rc != QFA_OK) return rc;
  const int64_t n_ctas = static_cast<int64_t>((dev.Skv + C::BN - 1) / C::BN) * B * dev.H;
  if (n_ctas > 0x7fffffffLL) return QFA_ERR_SHAPE;
  kern<<<static_cast<unsigned>(n_ctas), C::THREADS, C::SMEM, stream>>>(dev);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

// Runs the main kernel with `dq_accum` as the fp32 dQ accumulator (zero-filled here) and converts it.
int attn_bwd_mma_entry(const QfaBwdArgs& a, float* dq_accum, cudaStream_t stream) {
  BwdDev d;
  d.q = a.q;
  for (int i = 0; i < 3; ++i) {
    d.q_stride[i] = a.q_stride[i];
    d.do_stride[i] = a.do_stride[i];
    d.dk_stride[i] = a.dk_stride[i];
    d.dv_stride[i] = a.dv_stride[i];
  }
  d.qq = a.qq; d.k = a.k; d.v = a.v;
  d.d_o = a.d_o; d.lse = a.lse; d.delta = a.delta; d.lse_stride = a.lse_stride;
  d.dk = a.dk; d.dv = a.dv; d.dq_accum = dq_accum;
  d.H = static_cast<int>(a.H); d.Sq = static_cast<int>(a.Sq); d.Skv = static_cast<int>(a.Skv);
  d.sm_scale = a.sm_scale; d.causal = a.causal; d.dkv_fused = a.dkv_fused;
  d.kv_shared = (a.k.codes == a.v.codes && a.k.scale == a.v.scale && a.k.zp == a.v.zp &&
                 a.k.stride[0] == a.v.stride[0] && a.k.stride[1] == a.v.stride[1] && a.k.stride[2] == a.v.stride[2]);
  const int B = static_cast<int>(a.B);
  const int64_t n_acc = a.B * a.H * a.Sq * a.D;
  QFA_CUDA_TRY(cudaMemsetAsync(dq_accum, 0, n_acc * sizeof(float), stream));
  const bool i8 = a.mode == QFA_MODE_INT8;
  const bool bf = a.dtype == QFA_BF16;
  int rc = QFA_ERR_HEAD_DIM;
  if (a.D == 64) {
    if (i8) rc = bf ? launch_bwd<__nv_bfloat16, 64, true>(d, B, stream) : launch_bwd<__half, 64, true>(d, B, stream);
    else rc = bf ? launch_bwd<__nv_bfloat16, 64, false>(d, B, stream) : launch_bwd<__half, 64, false>(d, B, stream);
  } else if (a.D == 128) {
    if (i8) rc = bf ? launch_bwd<__nv_bfloat16, 128, true>(d, B, stream) : launch_bwd<__half, 128, true>(d, B, stream);
    else rc = bf ? launch_bwd<__nv_bfloat16, 128, false>(d, B, stream) : launch_bwd<__half, 128, false>(d, B, stream);
  }
  if (rc != QFA_OK) return rc;
  const int64_t n_vec = n_acc / 4;
  const int64_t blocks = (n_vec + 255) / 256;
  if (bf) {
    bwd_dq_finalize_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        dq_accum, static_cast<__nv_bfloat16*>(a.dq), a.dq_stride[0], a.dq_stride[1], a.dq_stride[2], d.H, d.Sq,
        static_cast<int>(a.D), a.sm_scale, n_vec);
  } else {
    bwd_dq_finalize_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        dq_accum, static_cast<__half*>(a.dq), a.dq_stride[0], a.dq_stride[1], a.dq_stride[2], d.H, d.Sq,
        static_cast<int>(a.D), a.sm_scale, n_vec);
  }
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

int attn_bwd_delta_entry(const void* o, const int64_t* so, const void* d_o, const int64_t* sd, float* delta,
                         int64_t delta_stride, int64_t B, int64_t H, int64_t Sq, int64_t D, int dtype,
                         cudaStream_t stream) {
  const int64_t rows = B * H * Sq;
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return QFA_ERR_SHAPE;
  if (dtype == QFA_BF16) {
    bwd_delta_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, so[0], so[1], so[2], sd[0],
        sd[1], sd[2], delta_stride, static_cast<int>(H), static_cast<int>(Sq), static_cast<int>(D), rows);
  } else {
    bwd_delta_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const __half*>(o), static_cast<const __half*>(d_o), delta, so[0], so[1], so[2], sd[0], sd[1], sd[2],
        delta_stride, static_cast<int>(H), static_cast<int>(Sq), static_cast<int>(D), rows);
  }
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

}  // namespace qfa
