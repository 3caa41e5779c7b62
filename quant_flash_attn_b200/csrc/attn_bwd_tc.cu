// INT8 flash-attention backward on tcgen05 (sm_100a), int8 mode.
//
// Two launches of ONE kernel template, following the split of the FA2 tutorial the reference ships
// (flash_attn_triton.py:393-435: a dK/dV pass, then a dQ pass, each recomputing P):
//
//   pass KV (rows = a 128-token K/V tile, walks the query tiles)      pass Q (rows = a 128-row query tile, walks K/V tiles)
//     T1 = Kc Qc^T          int8 kind::i8                               T1 = Qc Kc^T
//     T2 = V^ dO^T          kind::f16, both operands K-major            T2 = dO V^^T
//     P^T  = exp2(logit - LSE)              (quant_flash_attn.py:153-155)  P  = ...
//     dS^T = P^T * (T2 - delta)             (quant_flash_attn.py:157-158)  dS = ...
//     dV += P^T dO          P^T read from tensor memory                 --
//     dK += dS^T Q^         dS^T read from tensor memory                dQ += dS K^
//
// "rows" live in tensor-memory lanes, so the same code serves both passes with the roles of the row-side
// (stationary: codes + one 16-bit tensor, loaded once) and column-side (streamed by TMA, double buffered)
// operands swapped.  Logits come from the same int8 product + zero-point correction as the forward, so the
// recomputed P matches the saved LSE; Q^, K^, V^ are the dequantized 16-bit operands (straight-through
// gradients).  Tensor memory: T1 | T2 | acc1 | acc2 = 128 + 128 + D + D columns; P / dS are written back as
// packed 16-bit into the first halves of T1 / T2.
// Warp roles: producer (TMA + per-column constants), MMA issuer, tensor-memory allocator, sixteen softmax
// warps.  The element-wise stage has no row reductions (LSE and delta are inputs), so all sixteen warps share the
// one tile: a warp owns 16 rows x 64 columns and walks them in blocks of 16 columns, reading in the 16x256b
// fragment layout (a thread owns 2 rows x 4 columns of a block; the five per-column constants come in as 16-byte
// shared loads), with the next block's tensor-memory loads in flight while the current block is computed.
// P / dS of a block go back to tensor memory at once and the block is handed to the MMA issuer through its own
// mbarrier, so the accumulating MMAs of a 16-column k-step start while the later blocks are still being
// computed; only the last k-step and the next step's T1 / T2 remain on the critical path.  All waits are
// time-bounded.
#include <atomic>
#include <type_traits>

#include "qfa_common.cuh"
#include "sm100_ptx.cuh"

namespace qfa {

using namespace sm100;

struct TcBwdParams {
  // row side (per token of the stationary tile) and column side (per token of the streamed tiles)
  const uint16_t* r_scale; const int8_t* r_zp; const int32_t* r_sum;
  const uint16_t* c_scale; const int8_t* c_zp; const int32_t* c_sum;
  const float* lse;      // per query row, natural log
  const float* delta;    // per query row
  int64_t lse_stride;
  void* out1; int64_t out1_stride[3];    // pass KV: dV      pass Q: unused
  void* out2; int64_t out2_stride[3];    // pass KV: dK      pass Q: dQ
  int H, rows_total, cols_total;         // pass KV: rows = Skv, cols = Sq;  pass Q: rows = Sq, cols = Skv
  float sm_scale;
  int causal;
  int fused;             // REF, pass KV: write dV + sm_scale * dK into out2 (quant_flash_attn.py:161)
  unsigned int epoch;
  int32_t* status;
};

// REF = the reference's arithmetic (quant_flash_attn.py:133-166): 16-bit Q and the one dequantized K/V tensor
// feed 16-bit MMAs for the logits; the "codes" tiles are 16-bit tiles then, the streamed stage holds two 16-bit
// tiles [Y1 | Y2] (pass KV: Q and dO; pass Q: K^ = V^ alone), and there are no zero-point corrections.
template <int D, bool REF = false>
struct BwdTcCfg {
  static constexpr int BM = 128, BN = 128, STAGES = 2;
  static constexpr int C_BYTES = REF ? 128 * D * 2 : 128 * D;   // int8 tile, or (REF) a 16-bit tile in its place
  static constexpr int H_BYTES = 128 * D * 2;          // 16-bit tile
  static constexpr int PANELS = D / 64;
  static constexpr int PANEL_BYTES = 128 * 128;
  static constexpr int M_BYTES = 128 * 5 * 4;          // per column: z, -sum, s, -lse*log2e, -delta
  static constexpr int XC_OFF = 0;
  static constexpr int XH_OFF = XC_OFF + C_BYTES;
  static constexpr int ST_OFF = XH_OFF + H_BYTES;                      // stages: [Yc | Ya | Yb]
  static constexpr int ST_BYTES = REF ? 2 * H_BYTES : C_BYTES + 2 * H_BYTES;
  // where the right operands of the four products live inside a stage
  static constexpr int Y_T2B_KV = REF ? H_BYTES : C_BYTES, Y_T2B_Q = REF ? 0 : C_BYTES;     // T2: dO (KV) / V^ (Q)
  static constexpr int Y_ACC1B = REF ? H_BYTES : C_BYTES;                                   // dV += P^T dO
  static constexpr int Y_ACC2B = REF ? 0 : C_BYTES + H_BYTES;                               // dK += dS^T Q / dQ += dS K^
  static constexpr int M_OFF = ST_OFF + STAGES * ST_BYTES;
  static constexpr int BAR_OFF = M_OFF + STAGES * M_BYTES;
  static constexpr int KSTEPS = BN / 16;               // 16-column blocks = k-steps of the accumulating MMAs
  static constexpr int HANDOFFS = KSTEPS / 2;           // P / dS are handed to the MMA issuer 32 columns at a time
  static constexpr int NBARS = 1 + 3 * STAGES + 3 + HANDOFFS;
  static constexpr int MISC_OFF = BAR_OFF + NBARS * 8;
  static constexpr int SMEM = MISC_OFF + 16 + 1024;
  static constexpr int SOFTMAX_WARPS = 16;
  static constexpr int THREADS = 128 + SOFTMAX_WARPS * 32;
  static constexpr int T1_COL = 0, T2_COL = 128, ACC1_COL = 256, ACC2_COL = 256 + D;
  static constexpr int TMEM_COLS = 512;
  // P / dS (16-bit, two per 32-bit column) of column half c overwrite the first 32 columns of that half of
  // T1 / T2, so warps that share rows never write columns another warp still has to read: k-step kk of the
  // accumulating MMAs reads its left operand at this column offset
  __host__ __device__ static constexpr int p_col(int kk) { return (kk / 4) * 64 + (kk % 4) * 8; }
  static_assert(SMEM <= 232448, "shared memory budget");
};

struct BwdRow2 {
  float2 a2[2], A2[2], z2[2], nlse2[2], ndelta2[2];
};

// One block of 16 columns for the two rows (g, g+8) of a thread: T1 fragments (int32 logits) + T2 fragments
// (fp32 dP) -> P and dS packed to 16 bit in the 16x128b store layout (word 2n + row).  `meta` points at this
// thread's five 16-byte words of the block (z, -sum, s, -lse*log2e, -delta of its four columns).  KV_PASS: LSE /
// delta belong to the columns (queries) and the causal mask hides columns BELOW the row; otherwise they belong
// to the rows and the mask hides columns ABOVE the row.  Visible columns of row k: lo[k] <= 8n + e < hi[k].
template <typename T, bool KV_PASS, bool MASKED>
__device__ __forceinline__ void bwd_block(const uint32_t (&s)[8], const uint32_t (&d)[8], const float4* meta,
                                          const int (&lo)[2], const int (&hi)[2], const BwdRow2& rc, uint32_t (&pw)[4],
                                          uint32_t (&gw)[4]) {
  using H16 = Half16<T>;
  const float2 negM2 = make_float2(-12582912.0f, -12582912.0f);
  const float4 z4 = lds128(meta), n4 = lds128(meta + 1), s4 = lds128(meta + 2);
  float4 l4 = make_float4(0.f, 0.f, 0.f, 0.f), d4 = l4;
  if (KV_PASS) { l4 = lds128(meta + 3); d4 = lds128(meta + 4); }
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const float2 z2 = n ? make_float2(z4.z, z4.w) : make_float2(z4.x, z4.y);
    const float2 n2 = n ? make_float2(n4.z, n4.w) : make_float2(n4.x, n4.y);
    const float2 s2 = n ? make_float2(s4.z, s4.w) : make_float2(s4.x, s4.y);
    const float2 l2 = n ? make_float2(l4.z, l4.w) : make_float2(l4.x, l4.y);
    const float2 d2 = n ? make_float2(d4.z, d4.w) : make_float2(d4.x, d4.y);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint32_t s0 = s[4 * n + 2 * k], s1 = s[4 * n + 2 * k + 1];
      const uint32_t g0 = d[4 * n + 2 * k], g1 = d[4 * n + 2 * k + 1];
      // exact integer logits (see the forward kernel), then scale and subtract the saved LSE
      float2 v = make_float2(__uint_as_float(s0 + 0x4B400000u), __uint_as_float(s1 + 0x4B400000u));
      v = __fadd2_rn(v, negM2);
      v = __ffma2_rn(z2, rc.A2[k], v);
      v = __ffma2_rn(n2, rc.z2[k], v);
      v = __fmul2_rn(v, s2);
      v = __ffma2_rn(v, rc.a2[k], KV_PASS ? l2 : rc.nlse2[k]);
      if (MASKED) {
        if (8 * n < lo[k] || 8 * n >= hi[k]) v.x = -INFINITY;
        if (8 * n + 1 < lo[k] || 8 * n + 1 >= hi[k]) v.y = -INFINITY;
      }
      const float p0 = fast_exp2(v.x), p1 = fast_exp2(v.y);
      float2 dd = __fadd2_rn(make_float2(__uint_as_float(g0), __uint_as_float(g1)), KV_PASS ? d2 : rc.ndelta2[k]);
      dd = __fmul2_rn(make_float2(p0, p1), dd);
      pw[2 * n + k] = H16::pack(p0, p1);              // P rounded to 16 bit (quant_flash_attn.py:156)
      gw[2 * n + k] = H16::pack(dd.x, dd.y);          // dS rounded to 16 bit (quant_flash_attn.py:159-160)
    }
  }
}

// REF counterpart: s holds fp32 q.k^ (un-scaled: the reference multiplies by sm_scale after the product,
// quant_flash_attn.py:153); rc.a2 = sm_scale * log2e.  `meta` words 3, 4 carry -lse*log2e and -delta per column in
// pass KV.
template <typename T, bool KV_PASS, bool MASKED>
__device__ __forceinline__ void bwd_block_ref(const uint32_t (&s)[8], const uint32_t (&d)[8], const float4* meta,
                                              const int (&lo)[2], const int (&hi)[2], const BwdRow2& rc,
                                              uint32_t (&pw)[4], uint32_t (&gw)[4]) {
  using H16 = Half16<T>;
  float4 l4 = make_float4(0.f, 0.f, 0.f, 0.f), d4 = l4;
  if (KV_PASS) { l4 = lds128(meta + 3); d4 = lds128(meta + 4); }
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const float2 l2 = n ? make_float2(l4.z, l4.w) : make_float2(l4.x, l4.y);
    const float2 d2 = n ? make_float2(d4.z, d4.w) : make_float2(d4.x, d4.y);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float2 v = make_float2(__uint_as_float(s[4 * n + 2 * k]), __uint_as_float(s[4 * n + 2 * k + 1]));
      v = __ffma2_rn(v, rc.a2[k], KV_PASS ? l2 : rc.nlse2[k]);
      if (MASKED) {
        if (8 * n < lo[k] || 8 * n >= hi[k]) v.x = -INFINITY;
        if (8 * n + 1 < lo[k] || 8 * n + 1 >= hi[k]) v.y = -INFINITY;
      }
      const float p0 = fast_exp2(v.x), p1 = fast_exp2(v.y);
      float2 dd = __fadd2_rn(make_float2(__uint_as_float(d[4 * n + 2 * k]), __uint_as_float(d[4 * n + 2 * k + 1])),
                             KV_PASS ? d2 : rc.ndelta2[k]);
      dd = __fmul2_rn(make_float2(p0, p1), dd);
      pw[2 * n + k] = H16::pack(p0, p1);              // P rounded to 16 bit (quant_flash_attn.py:156)
      gw[2 * n + k] = H16::pack(dd.x, dd.y);          // dS rounded to 16 bit (quant_flash_attn.py:159-160)
    }
  }
}

__device__ __forceinline__ void tmem_st_16x128b_x2(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}

template <typename T, int D, bool KV_PASS, bool REF>
__global__ void __launch_bounds__(BwdTcCfg<D, REF>::THREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmXc, const __grid_constant__ CUtensorMap tmXh,
                   const __grid_constant__ CUtensorMap tmYc, const __grid_constant__ CUtensorMap tmYa,
                   const __grid_constant__ CUtensorMap tmYb, const TcBwdParams p) {
  using C = BwdTcCfg<D, REF>;
  using H16 = Half16<T>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  auto BAR = [&](int i) { return sbase + C::BAR_OFF + 8u * i; };
  constexpr int B_XFULL = 0;
  constexpr int B_YFULL = 1, B_YEMPTY = B_YFULL + C::STAGES, B_MFULL = B_YEMPTY + C::STAGES;
  constexpr int B_T1 = B_MFULL + C::STAGES, B_T2 = B_T1 + 1, B_ACC = B_T2 + 1, B_PD = B_ACC + 1;   // B_PD + k-step
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::MISC_OFF + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r_blocks = (p.rows_total + C::BM - 1) / C::BM;
  const int c_blocks = (p.cols_total + C::BN - 1) / C::BN;
  const int bh = blockIdx.x / r_blocks;
  const int b = bh / p.H, h = bh % p.H;
  const int rrank = blockIdx.x % r_blocks;
  // heavy row blocks first under the causal mask: early K/V tiles (pass KV), late query tiles (pass Q)
  const int rblk = (p.causal && !KV_PASS) ? (r_blocks - 1 - rrank) : rrank;
  const int r0 = rblk * C::BM;
  // column tiles this row block meets
  int j_begin = 0, j_end = c_blocks;
  if (p.causal) {
    if (KV_PASS) j_begin = r0 / C::BN;                                   // queries >= first token of the tile
    else j_end = min(c_blocks, (r0 + C::BM + C::BN - 1) / C::BN);        // tokens <= last query of the tile
  }
  const int n_steps = max(0, j_end - j_begin);

  if (tid == 0) {
    *abort_flag = launch_aborted(p.epoch) ? 1 : 0;
    mbar_init(BAR(B_XFULL), 1);
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(BAR(B_YFULL + i), 1);
      mbar_init(BAR(B_YEMPTY + i), 1);
      mbar_init(BAR(B_MFULL + i), 1);
    }
    mbar_init(BAR(B_T1), 1);
    mbar_init(BAR(B_T2), 1);
    mbar_init(BAR(B_ACC), 1);
    for (int i = 0; i < C::HANDOFFS; ++i) mbar_init(BAR(B_PD + i), C::SOFTMAX_WARPS / 2);   // the 8 warps of a column half
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
  const int64_t tok_r0 = static_cast<int64_t>(bh) * p.rows_total;
  const int64_t tok_c0 = static_cast<int64_t>(bh) * p.cols_total;
  // queries index LSE / delta: they are the columns in pass KV, the rows in pass Q
  const int64_t lse0 = static_cast<int64_t>(bh) * p.lse_stride;

  if (warp < 4) {
  // (No register hand-over between the warp groups: the kernel needs fewer than 96 registers per thread without
  // it, and `setmaxnreg` 56 / 104 measured the same speed.)
  if (warp == 0) {
    // ================================================================ producer
    if (lane == 0) {
      prefetch_tmap(&tmXc); prefetch_tmap(&tmXh); prefetch_tmap(&tmYc); prefetch_tmap(&tmYa); prefetch_tmap(&tmYb);
      mbar_arrive_expect_tx(BAR(B_XFULL), C::C_BYTES + C::H_BYTES);
      if constexpr (REF) {
        for (int pn = 0; pn < C::PANELS; ++pn)
          tma_load_4d(sbase + C::XC_OFF + pn * C::PANEL_BYTES, &tmXc, BAR(B_XFULL), pn * 64, r0, h, b);
      } else {
        tma_load_4d(sbase + C::XC_OFF, &tmXc, BAR(B_XFULL), 0, r0, h, b);
      }
      for (int pn = 0; pn < C::PANELS; ++pn)
        tma_load_4d(sbase + C::XH_OFF + pn * C::PANEL_BYTES, &tmXh, BAR(B_XFULL), pn * 64, r0, h, b);
    }
    bool ok = true;
    for (int it = 0; it < n_steps && ok; ++it) {
      const int c0 = (j_begin + it) * C::BN;
      const int st = it % C::STAGES;
      ok = mbar_wait(BAR(B_YEMPTY + st), ((it / C::STAGES) & 1) ^ 1, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t stage = sbase + C::ST_OFF + st * C::ST_BYTES;
      if (lane == 0) {
        if constexpr (REF) {
          // [Y1 | Y2]: pass KV streams Q and dO, pass Q the one K^ = V^ tile
          mbar_arrive_expect_tx(BAR(B_YFULL + st), KV_PASS ? 2 * C::H_BYTES : C::H_BYTES);
          for (int pn = 0; pn < C::PANELS; ++pn) {
            tma_load_4d(stage + pn * C::PANEL_BYTES, &tmYc, BAR(B_YFULL + st), pn * 64, c0, h, b);
            if (KV_PASS)
              tma_load_4d(stage + C::H_BYTES + pn * C::PANEL_BYTES, &tmYa, BAR(B_YFULL + st), pn * 64, c0, h, b);
          }
        } else {
          mbar_arrive_expect_tx(BAR(B_YFULL + st), C::ST_BYTES);
          tma_load_4d(stage, &tmYc, BAR(B_YFULL + st), 0, c0, h, b);
          for (int pn = 0; pn < C::PANELS; ++pn) {
            tma_load_4d(stage + C::C_BYTES + pn * C::PANEL_BYTES, &tmYa, BAR(B_YFULL + st), pn * 64, c0, h, b);
            tma_load_4d(stage + C::C_BYTES + C::H_BYTES + pn * C::PANEL_BYTES, &tmYb, BAR(B_YFULL + st), pn * 64, c0, h, b);
          }
        }
      }
      // per-column constants (the stage's previous readers are done: Y-empty is committed after the step's last MMA,
      // which is issued after the softmax warps finished the step).  Layout for the softmax threads: thread q of a
      // quad owns columns 8n+2q, 8n+2q+1; the constants of the two column groups of a 16-column block are packed
      // into five 16-byte words {z}, {-sum}, {s}, {-lse*log2e}, {-delta}
      float* meta = reinterpret_cast<float*>(smem + C::M_OFF + st * C::M_BYTES);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = i * 32 + lane;
        const int c = c0 + col;
        float z = 0.f, ns = 0.f, s = 0.f, nl = -INFINITY, nd = 0.f;
        if (c < p.cols_total) {
          if constexpr (!REF) {
            s = half_bits_to_f32(p.c_scale[tok_c0 + c]);
            z = static_cast<float>(p.c_zp[tok_c0 + c]);
            ns = -static_cast<float>(p.c_sum[tok_c0 + c]);
          }
          nl = 0.f;
          if (KV_PASS) {
            nl = -p.lse[lse0 + c] * kLog2e;
            nd = -p.delta[lse0 + c];
          }
        }
        const int n8 = col >> 3, qq = (col >> 1) & 3, e = col & 1;
        float* dst = meta + (((n8 >> 1) * 4 + qq) * 5) * 4 + (n8 & 1) * 2 + e;
        dst[0] = z;
        dst[4] = ns;
        dst[8] = s;
        dst[12] = nl;      // columns past the end: -inf reference -> P = 0 (pass Q masks them by index)
        dst[16] = nd;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_MFULL + st));
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t kF = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t kIdescT1 = REF ? make_idesc(1, kF, kF, 0, 0, 128, 128) : make_idesc(2, 1, 1, 0, 0, 128, 128);
      constexpr uint32_t kIdescT2 = make_idesc(1, kF, kF, 0, 0, 128, 128);       // both operands K-major
      constexpr uint32_t kIdescAcc = make_idesc(1, kF, kF, 0, 1, 128, D);        // B MN-major
      constexpr uint64_t kCSwz = (D == 128) ? kSwizzle128B : kSwizzle64B;
      constexpr int kT2B = KV_PASS ? C::Y_T2B_KV : C::Y_T2B_Q;
      bool ok = mbar_wait(BAR(B_XFULL), 0, abort_flag, p.epoch);
      tc_fence_after_sync();
      for (int it = 0; it < n_steps && ok; ++it) {
        const int st = it % C::STAGES;
        const uint32_t stage = sbase + C::ST_OFF + st * C::ST_BYTES;
        ok = mbar_wait(BAR(B_YFULL + st), (it / C::STAGES) & 1, abort_flag, p.epoch);
        if (!ok) break;
        tc_fence_after_sync();
        // T1 = Xc Yc^T (int8; REF: 16-bit tiles in their place), T2 = Xh Ya^T (16 bit, K-major x K-major).  They
        // overwrite the P / dS of the previous step: the tensor pipe runs MMAs in issue order, so they start after
        // that step's accumulating MMAs
        {
          if constexpr (REF) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint32_t off = (k / 4) * C::PANEL_BYTES + (k % 4) * 32;
              const uint64_t ha = make_smem_desc(sbase + C::XC_OFF + off, 16, 1024, kSwizzle128B);
              const uint64_t hb = make_smem_desc(stage + off, 16, 1024, kSwizzle128B);
              mma_f16_ss(tmem + C::T1_COL, ha, hb, kIdescT1, k > 0);
            }
          } else {
            const uint64_t da = make_smem_desc(sbase + C::XC_OFF, 16, 8 * D, kCSwz);
            const uint64_t db = make_smem_desc(stage, 16, 8 * D, kCSwz);
#pragma unroll
            for (int k = 0; k < D / 32; ++k)
              mma_i8_ss(tmem + C::T1_COL, desc_advance(da, k * 32), desc_advance(db, k * 32), kIdescT1, k > 0);
          }
          mma_commit(BAR(B_T1));
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k / 4) * C::PANEL_BYTES + (k % 4) * 32;
            const uint64_t ha = make_smem_desc(sbase + C::XH_OFF + off, 16, 1024, kSwizzle128B);
            const uint64_t hb = make_smem_desc(stage + kT2B + off, 16, 1024, kSwizzle128B);
            mma_f16_ss(tmem + C::T2_COL, ha, hb, kIdescT2, k > 0);
          }
          mma_commit(BAR(B_T2));
        }
        // accumulate with P / dS read from tensor memory, one 16-column k-step at a time as the softmax warps hand
        // the blocks over (the two column halves advance side by side)
        const uint64_t db1 = make_smem_desc(stage + C::Y_ACC1B, C::PANEL_BYTES, 1024, kSwizzle128B);   // dO (pass KV)
        const uint64_t db2 = make_smem_desc(stage + C::Y_ACC2B, C::PANEL_BYTES, 1024, kSwizzle128B);   // Q^ / Q or K^
#pragma unroll
        for (int i = 0; i < C::HANDOFFS; ++i) {
          const int hf = (i & 1) * 2 + (i >> 1);           // handoff index: column half * 2 + 32-column part
          const int kk0 = 2 * hf;                          // its two k-steps
          ok = mbar_wait(BAR(B_PD + hf), it & 1, abort_flag, p.epoch);
          if (!ok) break;
          tc_fence_after_sync();
          if (KV_PASS) {    // acc1 (dV) += P^T dO : right operand = the Ya tile (dO) viewed MN-major
#pragma unroll
            for (int kk = kk0; kk < kk0 + 2; ++kk)
              mma_f16_ts(tmem + C::ACC1_COL, tmem + C::T1_COL + C::p_col(kk), desc_advance(db1, kk * 2048), kIdescAcc,
                         (it > 0 || i > 0 || kk > kk0) ? 1u : 0u);
          }
          // acc2 (dK or dQ) += dS Yb : Yb = Q^ (pass KV) or K^ (pass Q), MN-major
#pragma unroll
          for (int kk = kk0; kk < kk0 + 2; ++kk)
            mma_f16_ts(tmem + C::ACC2_COL, tmem + C::T2_COL + C::p_col(kk), desc_advance(db2, kk * 2048), kIdescAcc,
                       (it > 0 || i > 0 || kk > kk0) ? 1u : 0u);
        }
        if (!ok) break;
        mma_commit(BAR(B_YEMPTY + st));
        if (it == n_steps - 1) mma_commit(BAR(B_ACC));
      }
    }
  }
  } else {
    // ================================================================ softmax-side math
    // warp (wq, hh, ch): rows 32*wq + 16*hh .. +15 of the tile, columns 64*ch .. +63
    const int sw = warp - 4;
    const int wq = warp & 3;
    const int hh = (sw >> 2) & 1;
    const int ch = sw >> 3;
    const int g = lane >> 2, q = lane & 3;
    const uint32_t lanes = static_cast<uint32_t>(wq * 32 + hh * 16) << 16;
    const uint32_t tT1 = tmem + lanes + C::T1_COL + 64 * ch, tT2 = tmem + lanes + C::T2_COL + 64 * ch;
    int rowk[2];
    BwdRow2 rc;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      rowk[k] = r0 + wq * 32 + hh * 16 + g + 8 * k;
      float A = 0.f, z = 0.f, a = 0.f, nl = -INFINITY, nd = 0.f;
      if (rowk[k] < p.rows_total) {
        if constexpr (REF) {
          a = p.sm_scale * kLog2e;
        } else {
          const int64_t tk = tok_r0 + rowk[k];
          const int zi = p.r_zp[tk];
          z = static_cast<float>(zi);
          A = static_cast<float>(D * zi - p.r_sum[tk]);
          a = half_bits_to_f32(p.r_scale[tk]) * p.sm_scale * kLog2e;
        }
        nl = 0.f;
        if (!KV_PASS) {
          nl = -p.lse[lse0 + rowk[k]] * kLog2e;
          nd = -p.delta[lse0 + rowk[k]];
        }
      }
      rc.a2[k] = make_float2(a, a);
      rc.A2[k] = make_float2(A, A);
      rc.z2[k] = make_float2(z, z);
      rc.nlse2[k] = make_float2(nl, nl);        // rows past the end: -inf -> P = 0
      rc.ndelta2[k] = make_float2(nd, nd);
    }
    bool ok = true;
    for (int it = 0; it < n_steps && ok; ++it) {
      const int st = it % C::STAGES;
      const int c0 = (j_begin + it) * C::BN;
      ok = mbar_wait(BAR(B_MFULL + st), (it / C::STAGES) & 1, abort_flag, p.epoch);
      if (ok) ok = mbar_wait(BAR(B_T1), it & 1, abort_flag, p.epoch);
      if (ok) ok = mbar_wait(BAR(B_T2), it & 1, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const float4* meta = reinterpret_cast<const float4*>(smem + C::M_OFF + st * C::M_BYTES) + (16 * ch + q) * 5;
      // visible column range of each row, relative to (tile start + 64*ch + 2q)
      int lo[2], hi[2];
      bool any_masked = false;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        int first = 0, last = p.cols_total - c0;                  // [first, last) in tile coordinates
        if (p.causal) {
          if (KV_PASS) first = max(first, rowk[k] - c0);          // query >= token
          else last = min(last, rowk[k] + 1 - c0);                // token <= query
        }
        any_masked |= (first > 0) || (last < C::BN);
        lo[k] = first - 64 * ch - 2 * q;
        hi[k] = last - 64 * ch - 2 * q;
      }
      const bool masked = __any_sync(0xffffffffu, any_masked);
      uint32_t sreg[2][8], dreg[2][8];
      tmem_ld_16x256b_x2(tT1, sreg[0]);
      tmem_ld_16x256b_x2(tT2, dreg[0]);
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        tmem_wait_ld_use(sreg[blk & 1], dreg[blk & 1]);
        if (blk + 1 < 4) {
          tmem_ld_16x256b_x2(tT1 + (blk + 1) * 16, sreg[(blk + 1) & 1]);
          tmem_ld_16x256b_x2(tT2 + (blk + 1) * 16, dreg[(blk + 1) & 1]);
        }
        int lo_b[2], hi_b[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) { lo_b[k] = lo[k] - blk * 16; hi_b[k] = hi[k] - blk * 16; }
        uint32_t pw[4], gw[4];
        if constexpr (REF) {
          if (masked) bwd_block_ref<T, KV_PASS, true>(sreg[blk & 1], dreg[blk & 1], meta + blk * 20, lo_b, hi_b, rc, pw, gw);
          else bwd_block_ref<T, KV_PASS, false>(sreg[blk & 1], dreg[blk & 1], meta + blk * 20, lo_b, hi_b, rc, pw, gw);
        } else {
          if (masked) bwd_block<T, KV_PASS, true>(sreg[blk & 1], dreg[blk & 1], meta + blk * 20, lo_b, hi_b, rc, pw, gw);
          else bwd_block<T, KV_PASS, false>(sreg[blk & 1], dreg[blk & 1], meta + blk * 20, lo_b, hi_b, rc, pw, gw);
        }
        // P / dS of this block go to 32-bit columns [8 blk, 8 blk + 8) of this half of T1 / T2: the int32 / fp32
        // values that lived there were consumed by this warp in an earlier (or this) block
        tmem_st_16x128b_x2(tT1 + blk * 8, pw);
        tmem_st_16x128b_x2(tT2 + blk * 8, gw);
        if (blk & 1) {
          // two blocks = two k-steps of the accumulating MMAs are ready
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR(B_PD + 2 * ch + (blk >> 1)));
        }
      }
    }
    // ---------------- epilogue: accumulators -> 16 bit.  dK and dQ carry sm_scale (quant_flash_attn.py:161,164)
    if (ok && n_steps > 0) {
      ok = mbar_wait(BAR(B_ACC), 0, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      // this warp writes its 16 rows x D/2 columns of each accumulator
      if (KV_PASS && p.fused) {
        // dKV = dV + sm_scale * dK in one tensor (quant_flash_attn.py:161)
        const uint32_t tA1 = tmem + lanes + C::ACC1_COL + ch * (D / 2), tA2 = tmem + lanes + C::ACC2_COL + ch * (D / 2);
        T* obase = static_cast<T*>(p.out2) + b * p.out2_stride[0] + h * p.out2_stride[1] + ch * (D / 2) + 2 * q;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r1[16], r2[16];
          if (n_steps > 0) {
            tmem_ld_16x256b_x4(tA1 + c * 32, r1);
            tmem_ld_16x256b_x4(tA2 + c * 32, r2);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r1[i] = r2[i] = 0u;
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (rowk[k] < p.rows_total) {
              T* orow = obase + static_cast<int64_t>(rowk[k]) * p.out2_stride[2] + c * 32;
#pragma unroll
              for (int n = 0; n < 4; ++n)
                *reinterpret_cast<uint32_t*>(orow + 8 * n) = H16::pack(
                    __uint_as_float(r1[4 * n + 2 * k]) + p.sm_scale * __uint_as_float(r2[4 * n + 2 * k]),
                    __uint_as_float(r1[4 * n + 2 * k + 1]) + p.sm_scale * __uint_as_float(r2[4 * n + 2 * k + 1]));
            }
          }
        }
      } else
      for (int which = KV_PASS ? 0 : 1; which < 2; ++which) {
        const uint32_t tA = tmem + lanes + (which == 0 ? C::ACC1_COL : C::ACC2_COL) + ch * (D / 2);
        const float scale = (which == 0) ? 1.0f : p.sm_scale;
        const int64_t* os = (which == 0) ? p.out1_stride : p.out2_stride;
        T* obase = static_cast<T*>(which == 0 ? p.out1 : p.out2) + b * os[0] + h * os[1] + ch * (D / 2) + 2 * q;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t oreg[16];
          if (n_steps > 0) {
            tmem_ld_16x256b_x4(tA + c * 32, oreg);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) oreg[i] = 0u;       // a row block that meets no column tile: zero gradient
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (rowk[k] < p.rows_total) {
              T* orow = obase + static_cast<int64_t>(rowk[k]) * os[2] + c * 32;
#pragma unroll
              for (int n = 0; n < 4; ++n)
                *reinterpret_cast<uint32_t*>(orow + 8 * n) =
                    H16::pack(__uint_as_float(oreg[4 * n + 2 * k]) * scale, __uint_as_float(oreg[4 * n + 2 * k + 1]) * scale);
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
  if (tid == 0 && *abort_flag && p.status) *p.status = QFA_STATUS_WAIT_TIMEOUT;
}

template <typename T, int D, bool KV_PASS, bool REF>
static int launch_bwd_tc(const QfaBwdArgs& a, cudaStream_t stream) {
  using C = BwdTcCfg<D, REF>;
  const CUtensorMapSwizzle cswz = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUtensorMapDataType hdt =
      std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // row side / column side operands
  const QfaQuantTensor& X = KV_PASS ? a.k : a.qq;
  const QfaQuantTensor& Y = KV_PASS ? a.qq : a.k;
  const int64_t Sx = KV_PASS ? a.Skv : a.Sq, Sy = KV_PASS ? a.Sq : a.Skv;
  auto map16 = [&](CUtensorMap* m, const void* base, int64_t S, const int64_t* stride_or_null) {
    // contiguous (B,H,S,D) unless strides are given (dO, Q)
    const uint64_t ss = stride_or_null ? 2ull * stride_or_null[2] : 2ull * D;
    const uint64_t sh = stride_or_null ? 2ull * stride_or_null[1] : 2ull * D * S;
    const uint64_t sb = stride_or_null ? 2ull * stride_or_null[0] : 2ull * D * S * a.H;
    return make_tmap_4d(m, base, hdt, 2, D, S, a.H, a.B, ss, sh, sb, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  CUtensorMap tmXc, tmXh, tmYc, tmYa, tmYb;
  bool ok;
  if (REF) {
    // K^ = V^ = a.v_hat (the dequantized K/V tensor, contiguous); Q and dO with the caller's strides
    if (KV_PASS) {
      ok = map16(&tmXc, a.v_hat, Sx, nullptr) && map16(&tmXh, a.v_hat, Sx, nullptr) &&
           map16(&tmYc, a.q, Sy, a.q_stride) && map16(&tmYa, a.d_o, Sy, a.do_stride);
    } else {
      ok = map16(&tmXc, a.q, Sx, a.q_stride) && map16(&tmXh, a.d_o, Sx, a.do_stride) &&
           map16(&tmYc, a.v_hat, Sy, nullptr);
      tmYa = tmYc;
    }
    tmYb = tmYc;
  } else {
    const void* xh = KV_PASS ? a.v_hat : a.d_o;          // stationary 16-bit operand of T2
    const void* ya = KV_PASS ? a.d_o : a.v_hat;          // streamed 16-bit operand of T2 (also B of acc1 in pass KV)
    const void* yb = KV_PASS ? a.q_hat : a.k_hat;        // streamed MN-major operand of acc2
    ok = make_tmap_4d(&tmXc, X.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, Sx, a.H, a.B, X.stride[2], X.stride[1],
                      X.stride[0], D, 128, cswz);
    ok = ok && make_tmap_4d(&tmYc, Y.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, Sy, a.H, a.B, Y.stride[2], Y.stride[1],
                            Y.stride[0], D, 128, cswz);
    ok = ok && map16(&tmXh, xh, Sx, KV_PASS ? nullptr : a.do_stride);
    ok = ok && map16(&tmYa, ya, Sy, KV_PASS ? a.do_stride : nullptr);
    ok = ok && map16(&tmYb, yb, Sy, nullptr);
  }
  if (!ok) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  TcBwdParams p;
  p.r_scale = X.scale; p.r_zp = X.zp; p.r_sum = X.rowsum;
  p.c_scale = Y.scale; p.c_zp = Y.zp; p.c_sum = Y.rowsum;
  p.lse = a.lse; p.delta = a.delta; p.lse_stride = a.lse_stride;
  p.out1 = KV_PASS ? a.dv : nullptr;
  p.out2 = KV_PASS ? a.dk : a.dq;
  for (int i = 0; i < 3; ++i) {
    p.out1_stride[i] = KV_PASS ? a.dv_stride[i] : 0;
    p.out2_stride[i] = KV_PASS ? a.dk_stride[i] : a.dq_stride[i];
  }
  p.H = static_cast<int>(a.H);
  p.rows_total = static_cast<int>(Sx);
  p.cols_total = static_cast<int>(Sy);
  p.sm_scale = a.sm_scale; p.causal = a.causal; p.status = a.status;
  p.fused = (REF && a.dkv_fused) ? 1 : 0;
  p.epoch = next_launch_epoch();
  auto kern = attn_bwd_tc_kernel<T, D, KV_PASS, REF>;
  static DeviceOnce attr_done;
  int rc = once_per_device(attr_done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    return QFA_OK;
  });
  if (rc != QFA_OK) return rc;
  const int64_t n_ctas = ((Sx + C::BM - 1) / C::BM) * a.B * a.H;
  if (n_ctas > 0x7fffffffLL) return QFA_ERR_SHAPE;
  kern<<<static_cast<unsigned>(n_ctas), C::THREADS, C::SMEM, stream>>>(tmXc, tmXh, tmYc, tmYa, tmYb, p);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

int attn_bwd_tc_supported(const QfaBwdArgs& a) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (a.D != 128 && a.D != 64) return 0;
  if (a.do_stride[0] % 8 || a.do_stride[1] % 8 || a.do_stride[2] % 8) return 0;
  if (a.mode == QFA_MODE_REF) {
    // the reference's operator with more than 32 query rows: fused dKV, one K/V tensor supplied dequantized (v_hat)
    if (!a.dkv_fused || a.causal || a.Sq <= 32 || !a.q || !a.v_hat || !al(a.v_hat)) return 0;
    if (a.k.codes != a.v.codes || a.k.scale != a.v.scale || a.k.zp != a.v.zp) return 0;
    return 1;
  }
  if (a.mode != QFA_MODE_INT8 || a.dkv_fused) return 0;
  if (!a.q_hat || !a.k_hat || !a.v_hat) return 0;
  if (!(a.sm_scale > 0.f)) return 0;
  if (!al(a.q_hat) || !al(a.k_hat) || !al(a.v_hat)) return 0;
  return 1;
}

template <typename T, int D, bool REF>
static int bwd_tc_two_passes(const QfaBwdArgs& a, cudaStream_t stream) {
  const int rc = launch_bwd_tc<T, D, true, REF>(a, stream);
  if (rc) return rc;
  return launch_bwd_tc<T, D, false, REF>(a, stream);
}

int attn_bwd_tc_entry(const QfaBwdArgs& a, cudaStream_t stream) {
  const bool bf = a.dtype == QFA_BF16;
  if (a.mode == QFA_MODE_REF) {
    if (a.D == 128) return bf ? bwd_tc_two_passes<__nv_bfloat16, 128, true>(a, stream) : bwd_tc_two_passes<__half, 128, true>(a, stream);
    return bf ? bwd_tc_two_passes<__nv_bfloat16, 64, true>(a, stream) : bwd_tc_two_passes<__half, 64, true>(a, stream);
  }
  if (a.D == 128) return bf ? bwd_tc_two_passes<__nv_bfloat16, 128, false>(a, stream) : bwd_tc_two_passes<__half, 128, false>(a, stream);
  return bf ? bwd_tc_two_passes<__nv_bfloat16, 64, false>(a, stream) : bwd_tc_two_passes<__half, 64, false>(a, stream);
}

}  // namespace qfa
