// INT8 flash-attention forward on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   S  = Qc Kc^T         int8 x int8 -> int32, tcgen05.mma kind::i8, operands staged by TMA (128B/64B swizzle),
//                        accumulator in tensor memory
//   s  = s_q s_k (S - z_k sum(q) - z_q sum(k) + D z_q z_k) * sm_scale     fused in the softmax warps
//   P  = exp2(s*log2e - m), written back to tensor memory as 16-bit, aliasing S
//   O += P V^            tcgen05.mma kind::f16 with P read from tensor memory and V^ (dequantized V, written
//                        by the quantizer) as an MN-major shared-memory operand
//   LSE = m + log(l)     (quant_flash_attn.py:79)
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks over 128-token K/V tiles.
// Warp roles: warp 0 = TMA producer (+ per-column constants), warp 1 = MMA issuer, warp 2 = tensor
// memory allocator, warps 4-11 / 12-19 = softmax of query tile 0 / 1: two threads per row, one per
// 64-column half, so that four softmax warps are resident per scheduler; the halves exchange the
// row max through shared memory, no shuffles.  The element-wise math uses packed f32x2
// instructions.  The two query tiles ping-pong: while the softmax warps of one tile work, the
// tensor core runs the other tile's MMAs.  O is only rescaled when the running max
// grew by more than 2^8 (the softmax threads do it in place in tensor memory), which makes the
// rescale rare after the first tiles.
//
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, all roles
// leave their loops, tensor memory is freed and the status word is set.
#include <type_traits>

#include "qfa_common.cuh"
#include "sm100_ptx.cuh"

namespace qfa {

using namespace sm100;

struct TcFwdParams {
  const uint16_t* q_scale; const int8_t* q_zp; const int32_t* q_sum;
  const uint16_t* k_scale; const int8_t* k_zp; const int32_t* k_sum;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride;
  int H, Sq, Skv;
  float sm_scale;
  int causal;
  int32_t* status;
};

template <int D>
struct TcCfg {
  static constexpr int BM = 128, BN = 128, NQT = 2;
  static constexpr int KSTAGES = 2, VSTAGES = 2, MSTAGES = 4;
  static constexpr int Q_BYTES = BM * D;                 // int8
  static constexpr int K_BYTES = BN * D;                 // int8
  static constexpr int V_BYTES = BN * D * 2;             // 16-bit
  static constexpr int V_PANELS = D / 64;                // 64-element (128-byte) column panels
  static constexpr int V_PANEL_BYTES = BN * 128;
  static constexpr int M_BYTES = BN * 12;                // per column: z_k, -sum(k), s_k as three float arrays
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + NQT * Q_BYTES;
  static constexpr int V_OFF = K_OFF + KSTAGES * K_BYTES;
  static constexpr int M_OFF = V_OFF + VSTAGES * V_BYTES;
  static constexpr int X_OFF = M_OFF + MSTAGES * M_BYTES;   // row-max exchange between the two column halves
  static constexpr int X_BYTES = 2 * NQT * 2 * BM * 4;      // [parity][tile][half][row] floats
  static constexpr int BAR_OFF = X_OFF + X_BYTES;
  static constexpr int NBARS = 1 + 2 * KSTAGES + 2 * VSTAGES + 2 * MSTAGES + 3 * NQT + 4 * NQT;
  static constexpr int MISC_OFF = BAR_OFF + NBARS * 8;
  static constexpr int SMEM = MISC_OFF + 16 + 1024;      // + slack for 1024-byte alignment of the base
  static constexpr int SOFTMAX_THREADS = NQT * 2 * BM;   // two threads per query row (one per column half)
  static constexpr int THREADS = 128 + SOFTMAX_THREADS;
  // tensor memory columns
  static constexpr int S_COL = 0;                        // S_t at t*BN (int32), P_t aliases its first BN/2 columns
  static constexpr int O_COL = NQT * BN;                 // O_t at O_COL + t*D (fp32)
  static constexpr int TMEM_COLS = 512;
  static constexpr uint32_t QK_SWIZZLE_ROWS_BYTES = 8 * D;    // 8 rows of D bytes per swizzle atom
};

template <typename T, int D>
__global__ void __launch_bounds__(640, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const TcFwdParams p) {
  using C = TcCfg<D>;
  using H16 = Half16<T>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + C::BAR_OFF;
  // barrier indices
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  constexpr int B_QFULL = 0;
  constexpr int B_KFULL = 1, B_KEMPTY = B_KFULL + C::KSTAGES;
  constexpr int B_VFULL = B_KEMPTY + C::KSTAGES, B_VEMPTY = B_VFULL + C::VSTAGES;
  constexpr int B_MFULL = B_VEMPTY + C::VSTAGES, B_MEMPTY = B_MFULL + C::MSTAGES;
  constexpr int B_SFULL = B_MEMPTY + C::MSTAGES, B_PFULL = B_SFULL + C::NQT, B_ODONE = B_PFULL + C::NQT;
  constexpr int B_PAIR = B_ODONE + C::NQT;               // [tile][lane quarter]: the two warps sharing 32 rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::MISC_OFF + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // 1-D grid: consecutive CTAs are the query blocks of one head, so they share its K/V through L2
  const int m_blocks = (p.Sq + C::NQT * C::BM - 1) / (C::NQT * C::BM);
  const int bh = blockIdx.x / m_blocks;
  const int b = bh / p.H, h = bh % p.H;
  const int mrank = blockIdx.x % m_blocks;
  // heavy (late) query blocks first under the causal mask
  const int mblk = p.causal ? (m_blocks - 1 - mrank) : mrank;
  const int m0 = mblk * (C::NQT * C::BM);
  int n_t[C::NQT];
  int n_max = 0;
#pragma unroll
  for (int t = 0; t < C::NQT; ++t) {
    const int m0t = m0 + t * C::BM;
    int kv_end = p.causal ? min(p.Skv, m0t + C::BM) : p.Skv;
    n_t[t] = (m0t < p.Sq) ? (kv_end + C::BN - 1) / C::BN : 0;
    n_max = max(n_max, n_t[t]);
  }

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(BAR(B_QFULL), 1);
    for (int i = 0; i < C::KSTAGES; ++i) { mbar_init(BAR(B_KFULL + i), 1); mbar_init(BAR(B_KEMPTY + i), 1); }
    for (int i = 0; i < C::VSTAGES; ++i) { mbar_init(BAR(B_VFULL + i), 1); mbar_init(BAR(B_VEMPTY + i), 1); }
    for (int i = 0; i < C::MSTAGES; ++i) { mbar_init(BAR(B_MFULL + i), 32); mbar_init(BAR(B_MEMPTY + i), C::SOFTMAX_THREADS); }
    for (int t = 0; t < C::NQT; ++t) {
      mbar_init(BAR(B_SFULL + t), 1);
      mbar_init(BAR(B_PFULL + t), 2 * C::BM);
      mbar_init(BAR(B_ODONE + t), 1);
      for (int w = 0; w < 4; ++w) mbar_init(BAR(B_PAIR + t * 4 + w), 64);
    }
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // the softmax warpgroups hold a whole 128-column row per thread: move registers to them
  if (warp < 4) {
  // control warpgroup: give registers away (the softmax warpgroups hold a whole row per thread)
  asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  if (warp == 0) {
    // ================================================================ producer
    if (lane == 0) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
      int q_tiles = 0;
      for (int t = 0; t < C::NQT; ++t) q_tiles += (n_t[t] > 0);
      mbar_arrive_expect_tx(BAR(B_QFULL), q_tiles * C::Q_BYTES);
      for (int t = 0; t < C::NQT; ++t)
        if (n_t[t] > 0) tma_load_4d(sbase + C::Q_OFF + t * C::Q_BYTES, &tmQ, BAR(B_QFULL), 0, m0 + t * C::BM, h, b);
    }
    const int64_t tok_k0 = static_cast<int64_t>(bh) * p.Skv;
    bool ok = true;
    for (int j = 0; j < n_max && ok; ++j) {
      const int n0 = j * C::BN;
      const int ks = j % C::KSTAGES, vs = j % C::VSTAGES, ms = j % C::MSTAGES;
      // K tile
      ok = mbar_wait(BAR(B_KEMPTY + ks), ((j / C::KSTAGES) & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(BAR(B_KFULL + ks), C::K_BYTES);
        tma_load_4d(sbase + C::K_OFF + ks * C::K_BYTES, &tmK, BAR(B_KFULL + ks), 0, n0, h, b);
      }
      // per-column constants z_k, -sum(k), s_k
      ok = mbar_wait(BAR(B_MEMPTY + ms), ((j / C::MSTAGES) & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      float* meta = reinterpret_cast<float*>(smem + C::M_OFF + ms * C::M_BYTES);
#pragma unroll
      for (int i = 0; i < C::BN / 32; ++i) {
        const int col = i * 32 + lane;
        const int n = n0 + col;
        float sk = 0.f, zk = 0.f, nks = 0.f;
        if (n < p.Skv) {
          sk = half_bits_to_f32(p.k_scale[tok_k0 + n]);
          zk = static_cast<float>(p.k_zp[tok_k0 + n]);
          nks = -static_cast<float>(p.k_sum[tok_k0 + n]);
        }
        meta[col] = zk;
        meta[C::BN + col] = nks;
        meta[2 * C::BN + col] = sk;
      }
      mbar_arrive(BAR(B_MFULL + ms));
      // V tile (D/64 panels of 128 bytes x BN rows)
      ok = mbar_wait(BAR(B_VEMPTY + vs), ((j / C::VSTAGES) & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(BAR(B_VFULL + vs), C::V_BYTES);
        for (int pn = 0; pn < C::V_PANELS; ++pn)
          tma_load_4d(sbase + C::V_OFF + vs * C::V_BYTES + pn * C::V_PANEL_BYTES, &tmV, BAR(B_VFULL + vs), pn * 64, n0,
                      h, b);
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t kIdescQK = make_idesc(2, 1, 1, 0, 0, C::BM, C::BN);
      constexpr uint32_t kF16Fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t kIdescPV = make_idesc(1, kF16Fmt, kF16Fmt, 0, 1, C::BM, D);
      constexpr uint64_t kQKSwz = (D == 128) ? kSwizzle128B : kSwizzle64B;
      bool ok = mbar_wait(BAR(B_QFULL), 0, abort_flag);
      tc_fence_after_sync();

      auto issue_qk = [&](int j, int t) {
        const int ks = j % C::KSTAGES;
        const uint64_t da = make_smem_desc(sbase + C::Q_OFF + t * C::Q_BYTES, 16, C::QK_SWIZZLE_ROWS_BYTES, kQKSwz);
        const uint64_t db = make_smem_desc(sbase + C::K_OFF + ks * C::K_BYTES, 16, C::QK_SWIZZLE_ROWS_BYTES, kQKSwz);
#pragma unroll
        for (int k = 0; k < D / 32; ++k)
          mma_i8_ss(tmem + C::S_COL + t * C::BN, desc_advance(da, k * 32), desc_advance(db, k * 32), kIdescQK, k > 0);
        mma_commit(BAR(B_SFULL + t));
      };
      auto issue_pv = [&](int j, int t) {
        const int vs = j % C::VSTAGES;
        const uint64_t db = make_smem_desc(sbase + C::V_OFF + vs * C::V_BYTES, C::V_PANEL_BYTES, 1024, kSwizzle128B);
#pragma unroll
        for (int k = 0; k < C::BN / 16; ++k)
          mma_f16_ts(tmem + C::O_COL + t * D, tmem + C::S_COL + t * C::BN + k * 8, desc_advance(db, k * 2048), kIdescPV,
                     (j > 0 || k > 0) ? 1u : 0u);
        mma_commit(BAR(B_ODONE + t));
      };

      if (ok && n_max > 0) {
        ok = mbar_wait(BAR(B_KFULL + 0), 0, abort_flag);
        if (ok) {
          tc_fence_after_sync();
          for (int t = 0; t < C::NQT; ++t)
            if (0 < n_t[t]) issue_qk(0, t);
          mma_commit(BAR(B_KEMPTY + 0));
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int vs = j % C::VSTAGES;
        ok = mbar_wait(BAR(B_VFULL + vs), (j / C::VSTAGES) & 1, abort_flag);
        if (!ok) break;
        const int ks1 = (j + 1) % C::KSTAGES;
        bool kwaited = false;
        for (int t = 0; t < C::NQT && ok; ++t) {
          if (j < n_t[t]) {
            ok = mbar_wait(BAR(B_PFULL + t), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv(j, t);
          }
          if (j + 1 < n_t[t]) {
            if (!kwaited) {
              ok = mbar_wait(BAR(B_KFULL + ks1), ((j + 1) / C::KSTAGES) & 1, abort_flag);
              if (!ok) break;
              tc_fence_after_sync();
              kwaited = true;
            }
            issue_qk(j + 1, t);
          }
        }
        if (!ok) break;
        mma_commit(BAR(B_VEMPTY + vs));
        if (kwaited) mma_commit(BAR(B_KEMPTY + ks1));
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    // ================================================================ softmax
    // Two threads per query row: warps sw and sw+4 of a tile share the same 32 tensor-memory lanes and
    // take the left / right 64 columns of the S tile; they exchange the row max through shared memory.
    const int sw = warp - 4;
    const int t = sw >> 3;                         // query tile
    const int half = (sw >> 2) & 1;                // column half
    const int wq = warp & 3;                       // tensor-memory lane quarter this warp may access
    const int r = wq * 32 + lane;                  // row inside the tile
    const int row = m0 + t * C::BM + r;            // global query row
    constexpr int HC = C::BN / 2;                  // S columns per thread
    constexpr int HD = D / 2;                      // O columns per thread
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tmem + lane_sel + C::S_COL + t * C::BN + half * HC;
    const uint32_t tP = tmem + lane_sel + C::S_COL + t * C::BN + half * (HC / 2);
    const uint32_t tO = tmem + lane_sel + C::O_COL + t * D + half * HD;
    const uint32_t pair_bar = BAR(B_PAIR + t * 4 + wq);
    uint32_t pair_phase = 0;
    float* xch = reinterpret_cast<float*>(smem + C::X_OFF);
    float A = 0.f, zq = 0.f, alpha = 0.f;
    if (row < p.Sq) {
      const int64_t tk = static_cast<int64_t>(bh) * p.Sq + row;
      const int z = p.q_zp[tk];
      zq = static_cast<float>(z);
      A = static_cast<float>(D * z - p.q_sum[tk]);
      alpha = half_bits_to_f32(p.q_scale[tk]) * p.sm_scale * kLog2e;
    }
    const float2 A2 = make_float2(A, A), zq2 = make_float2(zq, zq), alpha2 = make_float2(alpha, alpha);
    const float2 negM2 = make_float2(-12582912.0f, -12582912.0f);
    float m_run = 0.f, l_run = 0.f;
    const int my_n = n_t[t];
    bool ok = true;
    for (int j = 0; j < n_max && ok; ++j) {
      const int ms = j % C::MSTAGES;
      if (j < my_n) {
        ok = mbar_wait(BAR(B_MFULL + ms), (j / C::MSTAGES) & 1, abort_flag);
        if (ok) ok = mbar_wait(BAR(B_SFULL + t), j & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t sreg[HC];
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sreg[c * 32]));
        tmem_wait_ld();
        const float* meta = reinterpret_cast<const float*>(smem + C::M_OFF + ms * C::M_BYTES) + half * HC;
        // logits in units of 1/alpha: s_k * (S + z_k*A - sum(k)*z_q); exact in fp32 up to the last multiply
        const int n0 = j * C::BN + half * HC;
        int col_limit = p.Skv - n0;                                   // columns >= limit are masked
        if (p.causal) col_limit = min(col_limit, row + 1 - n0);
        const bool masked = __any_sync(0xffffffffu, col_limit < HC);
        float tmax = -INFINITY;
#pragma unroll
        for (int c = 0; c < HC; c += 4) {
          const float4 y4 = *reinterpret_cast<const float4*>(meta + c);
          const float4 z4 = *reinterpret_cast<const float4*>(meta + C::BN + c);
          const float4 x4 = *reinterpret_cast<const float4*>(meta + 2 * C::BN + c);
          // int32 -> fp32 without the conversion pipe: |S| <= 128*128*D < 2^22, so the bit pattern of
          // 1.5*2^23 plus S is the float 1.5*2^23 + S
          float2 v0 = make_float2(__uint_as_float(sreg[c] + 0x4B400000u), __uint_as_float(sreg[c + 1] + 0x4B400000u));
          float2 v1 = make_float2(__uint_as_float(sreg[c + 2] + 0x4B400000u), __uint_as_float(sreg[c + 3] + 0x4B400000u));
          v0 = __fadd2_rn(v0, negM2);
          v1 = __fadd2_rn(v1, negM2);
          v0 = __ffma2_rn(make_float2(y4.x, y4.y), A2, v0);
          v1 = __ffma2_rn(make_float2(y4.z, y4.w), A2, v1);
          v0 = __ffma2_rn(make_float2(z4.x, z4.y), zq2, v0);
          v1 = __ffma2_rn(make_float2(z4.z, z4.w), zq2, v1);
          v0 = __fmul2_rn(v0, make_float2(x4.x, x4.y));
          v1 = __fmul2_rn(v1, make_float2(x4.z, x4.w));
          if (masked) {
            if (c + 0 >= col_limit) v0.x = -INFINITY;
            if (c + 1 >= col_limit) v0.y = -INFINITY;
            if (c + 2 >= col_limit) v1.x = -INFINITY;
            if (c + 3 >= col_limit) v1.y = -INFINITY;
          }
          sreg[c] = __float_as_uint(v0.x); sreg[c + 1] = __float_as_uint(v0.y);
          sreg[c + 2] = __float_as_uint(v1.x); sreg[c + 3] = __float_as_uint(v1.y);
          asm("max.f32 %0, %0, %1, %2;" : "+f"(tmax) : "f"(v0.x), "f"(v0.y));
          asm("max.f32 %0, %0, %1, %2;" : "+f"(tmax) : "f"(v1.x), "f"(v1.y));
        }
        mbar_arrive(BAR(B_MEMPTY + ms));
        // row max over both halves
        {
          float* xb = xch + ((j & 1) * C::NQT + t) * 2 * C::BM;
          xb[half * C::BM + r] = tmax;
          mbar_arrive(pair_bar);
          ok = mbar_wait(pair_bar, pair_phase, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          pair_phase ^= 1;
          tmax = fmaxf(tmax, xb[(half ^ 1) * C::BM + r]);
        }
        // running max with lazy rescale (both halves take the same decision)
        if (j == 0) {
          m_run = (tmax == -INFINITY) ? 0.f : tmax;
        } else {
          const bool grow = (tmax - m_run) * alpha > 8.0f;
          // the partner warp sees the same rows, so the vote has the same outcome there
          if (__any_sync(0xffffffffu, grow)) {
            ok = mbar_wait(BAR(B_ODONE + t), (j - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const float m_new = fmaxf(m_run, tmax);
            const float factor = fast_exp2((m_run - m_new) * alpha);
            // rare path: small chunks keep the live S row in registers
#pragma unroll 1
            for (int c = 0; c < HD / 8; ++c) {
              uint32_t oreg[8];
              tmem_ld8(tO + c * 8, oreg);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 8; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * factor);
              tmem_st8(tO + c * 8, oreg);
            }
            tmem_wait_st();
            l_run *= factor;
            m_run = m_new;
          }
        }
        const float neg_m = -m_run * alpha;
        const float2 negm2 = make_float2(neg_m, neg_m);
        float2 lsum2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int cc = 0; cc < HC; cc += 32) {
          uint32_t preg[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float2 e = __ffma2_rn(make_float2(__uint_as_float(sreg[cc + c]), __uint_as_float(sreg[cc + c + 1])),
                                        alpha2, negm2);
            const float p0 = fast_exp2(e.x);
            const float p1 = fast_exp2(e.y);
            lsum2 = __fadd2_rn(lsum2, make_float2(p0, p1));
            preg[c / 2] = H16::pack(p0, p1);        // P rounded to 16 bit (quant_flash_attn.py:75)
          }
          tmem_st16(tP + cc / 2, preg);
        }
        l_run += lsum2.x + lsum2.y;
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(BAR(B_PFULL + t));
      } else {
        // this query tile is done (causal): keep the per-column ring moving for the other tile
        ok = mbar_wait(BAR(B_MFULL + ms), (j / C::MSTAGES) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        mbar_arrive(BAR(B_MEMPTY + ms));
      }
    }
    // ---------------- epilogue: O / l -> 16 bit, LSE
    if (ok && my_n > 0) {
      // total row sum = sum of the two halves' partial sums
      float* xb = xch + t * 2 * C::BM;
      xb[half * C::BM + r] = l_run;
      mbar_arrive(pair_bar);
      ok = mbar_wait(pair_bar, pair_phase, abort_flag);
      if (ok) ok = mbar_wait(BAR(B_ODONE + t), (my_n - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        const float l_tot = l_run + xb[(half ^ 1) * C::BM + r];
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        T* orow = static_cast<T*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1] +
                  static_cast<int64_t>(row) * p.o_stride[2] + half * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t oreg[32];
          tmem_ld32(tO + c * 32, oreg);
          tmem_wait_ld();
          if (row < p.Sq) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = H16::pack(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv);
              v.y = H16::pack(__uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
              v.z = H16::pack(__uint_as_float(oreg[i + 4]) * inv, __uint_as_float(oreg[i + 5]) * inv);
              v.w = H16::pack(__uint_as_float(oreg[i + 6]) * inv, __uint_as_float(oreg[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
            }
          }
        }
        if (half == 0 && row < p.Sq)
          p.lse[static_cast<int64_t>(bh) * p.lse_stride + row] = (m_run * alpha + log2f(l_tot)) * kLn2;
      }
    }
  }

  // ================================================================ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
  if (tid == 0 && *abort_flag && p.status) *p.status = QFA_STATUS_WAIT_TIMEOUT;
}

template <typename T, int D>
static int launch_tc(const QfaFwdArgs& a, cudaStream_t stream) {
  using C = TcCfg<D>;
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapSwizzle qk_swz = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUtensorMapDataType vdt =
      std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  bool ok = make_tmap_4d(&tmQ, a.qq.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, a.Sq, a.H, a.B, a.qq.stride[2],
                         a.qq.stride[1], a.qq.stride[0], D, C::BM, qk_swz);
  ok = ok && make_tmap_4d(&tmK, a.k.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, a.Skv, a.H, a.B, a.k.stride[2],
                          a.k.stride[1], a.k.stride[0], D, C::BN, qk_swz);
  ok = ok && make_tmap_4d(&tmV, a.v_hat, vdt, 2, D, a.Skv, a.H, a.B, 2ull * D, 2ull * D * a.Skv,
                          2ull * D * a.Skv * a.H, 64, C::BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  TcFwdParams p;
  p.q_scale = a.qq.scale; p.q_zp = a.qq.zp; p.q_sum = a.qq.rowsum;
  p.k_scale = a.k.scale; p.k_zp = a.k.zp; p.k_sum = a.k.rowsum;
  p.o = a.o;
  for (int i = 0; i < 3; ++i) p.o_stride[i] = a.o_stride[i];
  p.lse = a.lse; p.lse_stride = a.lse_stride;
  p.H = static_cast<int>(a.H); p.Sq = static_cast<int>(a.Sq); p.Skv = static_cast<int>(a.Skv);
  p.sm_scale = a.sm_scale; p.causal = a.causal; p.status = a.status;
  auto kern = attn_fwd_tc_kernel<T, D>;
  static bool attr_done[64] = {};
  int devid = 0;
  QFA_CUDA_TRY(cudaGetDevice(&devid));
  if (devid < 64 && !attr_done[devid]) {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    attr_done[devid] = true;
  }
  const int64_t n_ctas = ((a.Sq + C::NQT * C::BM - 1) / (C::NQT * C::BM)) * a.B * a.H;
  if (n_ctas > 0x7fffffffLL) return QFA_ERR_SHAPE;
  kern<<<static_cast<unsigned>(n_ctas), C::THREADS, C::SMEM, stream>>>(tmQ, tmK, tmV, p);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

// The tcgen05 kernel takes int8-mode problems with the dequantized V supplied by the quantizer.
int attn_fwd_tc_supported(const QfaFwdArgs& a) {
  if (a.mode != QFA_MODE_INT8 || !a.v_hat) return 0;
  if (a.D != 128) return 0;
  if (!(a.sm_scale > 0.f)) return 0;
  if ((reinterpret_cast<uintptr_t>(a.v_hat) & 15) != 0) return 0;
  return 1;
}

int attn_fwd_tc_entry(const QfaFwdArgs& a, cudaStream_t stream) {
  if (a.D == 128) {
    return a.dtype == QFA_BF16 ? launch_tc<__nv_bfloat16, 128>(a, stream) : launch_tc<__half, 128>(a, stream);
  }
  return QFA_ERR_HEAD_DIM;
}

}  // namespace qfa
