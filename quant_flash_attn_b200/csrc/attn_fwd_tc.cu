// INT8 flash-attention forward on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   S  = sum((q - z_q)(k - z_k))   the exact integer dot product of the centered codes, by one of two routes with
//                        bit-identical results:
//                          int8 MMA : Qc Kc^T as int8 x int8 -> int32 (tcgen05.mma kind::i8) plus the three zero-point
//                                     terms - z_k sum(q) - z_q sum(k) + D z_q z_k, added by the softmax warps;
//                          centered : (Qc - z_q)(Kc - z_k)^T as fp16 x fp16 -> fp32 (kind::f16), exact because the
//                                     operands are integers of at most 9 bits and the sums stay below 2^24
//                        operands staged in shared memory (TMA, 128B/64B swizzle), accumulator in tensor memory
//   s  = s_q s_k S * sm_scale      fused in the softmax warps
//   P  = exp2(s*log2e - m), written back to tensor memory as 16-bit, aliasing S
//   O += P V^            tcgen05.mma kind::f16 with P read from tensor memory and V^ (dequantized V, written
//                        by the quantizer) as an MN-major shared-memory operand
//   LSE = m + log(l)     (quant_flash_attn.py:79)
//
// One CTA owns two 128-row query tiles of one (batch, head) and walks over 128-token K/V tiles.
// Warp roles: warp 0 = TMA producer (+ per-column constants, tensor memory allocation), warp 1 = MMA issuer,
// warps 2-9 / 10-17 = softmax of query tile 0 / 1 (two warps per 32-lane quarter of
// tensor memory, 16 rows each).  A softmax warp reads S in the 16x256b fragment layout (a thread owns
// 2 rows x 32 columns), so the per-column constants are read from shared memory once per two rows,
// row max / sum are quad shuffles, and the element-wise math
// runs on packed f32x2 instructions in a single pass per tile: P is formed against a lazily raised
// reference instead of the exact running max, and O, l and P are rescaled (by exact powers of two)
// only when a tile exceeds the reference by more than 2^8.  The two query tiles ping-pong: while
// the softmax warps of one tile work, the tensor core runs the other tile's MMAs.
//
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, all roles
// leave their loops, tensor memory is freed and the status word is set.
#include <atomic>
#include <type_traits>

#include "qfa_common.cuh"
#include "sm100_ptx.cuh"

namespace qfa {

using namespace sm100;

struct TcFwdParams {
  const int8_t* q_codes; int64_t q_stride[3];       // CTR: the softmax warps read and center the codes of Q
  const int8_t* kv_codes; int64_t kv_stride[3];     // RAW: the softmax warps read and dequantize the K/V codes
  const uint16_t* q_scale; const int8_t* q_zp; const int32_t* q_sum;
  const uint16_t* k_scale; const int8_t* k_zp; const int32_t* k_sum;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride;
  int H, Hkv, Sq, Skv;      // Hkv K/V heads serve H query heads (H / Hkv query heads each)
  float sm_scale;
  int causal;
  unsigned int epoch;   // distinguishes launches for the device-wide abort word
  int32_t* status;
};

// REF = the reference's arithmetic (quant_flash_attn.py:50-79): Q stays 16-bit (scaled by sm_scale and rounded
// in shared memory), the one dequantized K/V tensor is both operands, logits come from a 16-bit MMA in fp32; no
// int8 tiles, no per-column constants.
//
// CTR = int8-mode arithmetic on the 16-bit tensor path.  code - zero_point lies in [-255, 255] and is exact in fp16,
// and a dot product of D <= 128 such pairs stays below 2^24, so a `kind::f16` MMA over the CENTERED codes returns
// the integer sum((q - z_q)(k - z_k)) exactly, as fp32: the four-term zero-point correction and the int32 -> fp32
// step of the int8 MMA route disappear from the softmax warps (2 instead of 7 packed operations per pair of
// logits before the exponential).  Q is centered by the softmax warps from its int8 codes while the first K/V
// tiles arrive; K arrives centered (fp16, one extra output of the quantizer) because 16+ CTAs share each K tile.
enum : int { kModeI8 = 0, kModeRef = 1, kModeCtr = 2 };

// NQT = query tiles per CTA.  Two tiles ping-pong on one SM; with at most 128 query rows per head there is only one
// tile, and the one-tile instantiation (half the softmax warps, tensor memory and Q buffer) lets TWO CTAs -- two
// heads -- share an SM instead (REF mode, whose K/V ring is small enough for that).
//
// SHORT (REF, one tile, at most 32 query rows -- the reference's own benchmark regime): only the first 32 rows of
// the 128-row MMA tile are real.  Rows of an MMA are independent, so nothing is stored for the other 96: the Q
// buffer holds 32 rows and the operand descriptor simply runs on into whatever follows it in shared memory; the
// resulting logits, their "P" and their rows of O are never looked at.  That frees the shared memory for a THIRD
// K/V stage with two CTAs per SM.  Tensor-memory lanes 0-31 are reachable from two of the eight warps only; the other
// six have no softmax to do and become dedicated converters: decoupled from the softmax hand-overs, they stream the
// int8 codes through a register double buffer into the stage ring, up to three tiles ahead of the MMAs.
template <int D, int MODE = kModeI8, int NQT_ = 2, bool SHORT_ = false>
struct TcCfg {
  static constexpr bool REF = MODE == kModeRef, CTR = MODE == kModeCtr, SHORT = SHORT_;
  static_assert(!SHORT || (REF && NQT_ == 1), "the short-query layout exists for the one-tile REF kernel only");
  static constexpr int BM = 128, BN = 128, NQT = NQT_;
  static constexpr int QROWS = SHORT ? 32 : BM;          // rows of a query tile that exist in shared memory
  static constexpr int KSTAGES = REF ? 0 : 2, VSTAGES = SHORT ? 3 : 2, MSTAGES = REF ? 0 : 4;
  static constexpr int Q_BYTES = QROWS * D * (MODE != kModeI8 ? 2 : 1); // int8 codes, or 16-bit rows as D/64 panels of 128-byte rows
  static constexpr int Q_PANEL_BYTES = QROWS * 128;
  static constexpr int K_BYTES = BN * D * (CTR ? 2 : 1);  // int8 codes, or (CTR) fp16 panels like a V^ tile
  static constexpr int V_BYTES = BN * D * 2;             // 16-bit
  static constexpr int V_PANELS = D / 64;                // 64-element (128-byte) column panels
  static constexpr int V_PANEL_BYTES = BN * 128;
  static constexpr int M_BYTES = BN * (CTR ? 4 : 12);    // per column: z_k, -sum(k), s_k as three float arrays; CTR: s_k
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + NQT * Q_BYTES;
  static constexpr int V_OFF = K_OFF + KSTAGES * K_BYTES;
  static constexpr int M_OFF = V_OFF + VSTAGES * V_BYTES;
  static constexpr int BAR_OFF = M_OFF + MSTAGES * M_BYTES;
  static constexpr int NBARS = 1 + 2 * KSTAGES + 2 * VSTAGES + 2 * MSTAGES + 3 * NQT + 1;   // + "Q scaled" (REF)
  static constexpr int MISC_OFF = BAR_OFF + NBARS * 8;
  static constexpr int SMEM = MISC_OFF + 16 + 1024;      // + slack for 1024-byte alignment of the base
  static constexpr int SOFTMAX_THREADS = 2 * NQT * BM;   // one warp per 16 rows; a thread owns 2 rows x 32 columns
  // Two control warps (producer, MMA issuer) and sixteen softmax warps.  Every thread keeps the 96 registers of
  // the launch: moving registers from the control warps to the softmax warps with `setmaxnreg` (56 / 104, measured)
  // was 4 % SLOWER -- the MMA issuer's hand-over loop is on the critical path of every K/V step and spilled at 56.
  static constexpr int CTRL_WARPS = 2;
  static constexpr int CTRL_THREADS = 32 * CTRL_WARPS;
  static constexpr int THREADS = CTRL_THREADS + SOFTMAX_THREADS;
  static constexpr int LIVE_WARPS = SHORT ? 2 : SOFTMAX_THREADS / 32 / NQT;   // warps of a tile that run the softmax
  static constexpr int CONV_WARPS = SHORT ? 6 : SOFTMAX_THREADS / 32;         // warps that fill a V stage (RAW)
  // tensor memory columns
  static constexpr int S_COL = 0;                        // S_t at t*BN (int32), P_t aliases its first BN/2 columns
  static constexpr int O_COL = NQT * BN;                 // O_t at O_COL + t*D (fp32)
  // RAW (REF with one tile): the K/V tiles are dequantized inside the kernel, by the softmax warps, from the int8
  // codes in global memory.  Every K/V tile serves a single CTA here, so a dequantized copy in HBM (2 bytes written
  // and read per element on top of the code byte) would dominate a problem of this shape.
  static constexpr bool RAW = REF && NQT == 1;
  static constexpr int TMEM_COLS = NQT == 2 ? 512 : 256;   // a power of two >= NQT * (BN + D)
  static constexpr int CTAS_PER_SM = NQT == 2 ? 1 : 2;
  static constexpr uint32_t QK_SWIZZLE_ROWS_BYTES = 8 * D;    // 8 rows of D bytes per swizzle atom
};

// Per-row constants of a softmax thread (each thread owns two rows).  With a = s_q*sm_scale*log2(e):
//   logit*log2e - ref = a * s_k * (S + A*z_k - z_q*sum(k)) - ref,    A = D*z_q - sum(q)
// Every value is kept as a pair of equal halves because the math runs on packed f32x2 instructions.
struct RowConst2 {
  float2 a2[2], A2[2], zq2[2], nref2[2];
};

// One block of 16 columns for the two rows (g, g+8) of a thread.  s holds the int32 accumulators in the
// 16x256b fragment layout: element [4n + 2*row + e] is column 8n + 2q + e.  `meta` points at this thread's three
// 16-byte words of the block: z_k, -sum(k), s_k of its four columns, loaded once and used for both rows.  lim[k] = first masked column of row k relative to
// (block start + 2q).  pw receives P packed to 16 bit in the 16x128b store layout (word 2n + row).
// REF counterpart of softmax_block: s holds fp32 logits q~.k^ (q~ = q * sm_scale rounded, quant_flash_attn.py:52,68);
// P = exp2(s * log2e - ref).
template <typename T, bool MASKED, bool MAX_ONLY>
__device__ __forceinline__ void softmax_block_ref(const uint32_t (&s)[8], const int (&lim)[2], const RowConst2& rc,
                                                  float (&emax)[2], float2 (&lsum2)[2], uint32_t* pw) {
  using H16 = Half16<T>;
  const float2 l2e = make_float2(kLog2e, kLog2e);
#pragma unroll
  for (int n = 0; n < 2; ++n) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float2 v = make_float2(__uint_as_float(s[4 * n + 2 * k]), __uint_as_float(s[4 * n + 2 * k + 1]));
      v = __ffma2_rn(v, l2e, rc.nref2[k]);
      if (MASKED) {
        if (8 * n >= lim[k]) v.x = -INFINITY;
        if (8 * n + 1 >= lim[k]) v.y = -INFINITY;
      }
      asm("max.f32 %0, %0, %1, %2;" : "+f"(emax[k]) : "f"(v.x), "f"(v.y));
      if (!MAX_ONLY) {
        const float p0 = fast_exp2(v.x), p1 = fast_exp2(v.y);
        lsum2[k] = __fadd2_rn(lsum2[k], make_float2(p0, p1));
        pw[2 * n + k] = H16::pack(p0, p1);            // P rounded to 16 bit (quant_flash_attn.py:75)
      }
    }
  }
}

// CTR counterpart: s holds the exact integer sum((q - z_q)(k - z_k)) as fp32; `meta` points at this thread's one
// 16-byte word of the block, s_k of its four columns.  logit*log2e - ref = (S * s_k) * a - ref.
template <typename T, bool MASKED, bool MAX_ONLY>
__device__ __forceinline__ void softmax_block_ctr(const uint32_t (&s)[8], const float4 x4, const int (&lim)[2],
                                                  const RowConst2& rc, float (&emax)[2], float2 (&lsum2)[2],
                                                  uint32_t* pw) {
  using H16 = Half16<T>;
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const float2 x2 = n ? make_float2(x4.z, x4.w) : make_float2(x4.x, x4.y);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      float2 v = make_float2(__uint_as_float(s[4 * n + 2 * k]), __uint_as_float(s[4 * n + 2 * k + 1]));
      v = __fmul2_rn(v, x2);
      v = __ffma2_rn(v, rc.a2[k], rc.nref2[k]);
      if (MASKED) {
        if (8 * n >= lim[k]) v.x = -INFINITY;
        if (8 * n + 1 >= lim[k]) v.y = -INFINITY;
      }
      asm("max.f32 %0, %0, %1, %2;" : "+f"(emax[k]) : "f"(v.x), "f"(v.y));
      if (!MAX_ONLY) {
        const float p0 = fast_exp2(v.x), p1 = fast_exp2(v.y);
        lsum2[k] = __fadd2_rn(lsum2[k], make_float2(p0, p1));
        pw[2 * n + k] = H16::pack(p0, p1);            // P rounded to 16 bit (quant_flash_attn.py:75)
      }
    }
  }
}

template <typename T, int BN, bool MASKED, bool MAX_ONLY>
__device__ __forceinline__ void softmax_block(const uint32_t (&s)[8], const float4* meta, const int (&lim)[2],
                                              const RowConst2& rc, float (&emax)[2], float2 (&lsum2)[2],
                                              uint32_t* pw) {
  using H16 = Half16<T>;
  const float2 negM2 = make_float2(-12582912.0f, -12582912.0f);
  const float4 y4 = lds128(meta), z4 = lds128(meta + 1), x4 = lds128(meta + 2);
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const float2 y2 = n ? make_float2(y4.z, y4.w) : make_float2(y4.x, y4.y);
    const float2 z2 = n ? make_float2(z4.z, z4.w) : make_float2(z4.x, z4.y);
    const float2 x2 = n ? make_float2(x4.z, x4.w) : make_float2(x4.x, x4.y);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint32_t s0 = s[4 * n + 2 * k], s1 = s[4 * n + 2 * k + 1];
      // int32 -> fp32 without the conversion pipe: |S| <= 128*128*D < 2^22, so the bit pattern of 1.5*2^23
      // plus S is the float 1.5*2^23 + S.  Everything up to the multiply by s_k is exact integer arithmetic
      // in fp32 (|S + z_k*A - sum(k)*z_q| <= 255*255*D < 2^24): with large scales one integer step is several
      // percent of a logit, so nothing may round before that point.
      float2 v = make_float2(__uint_as_float(s0 + 0x4B400000u), __uint_as_float(s1 + 0x4B400000u));
      v = __fadd2_rn(v, negM2);
      v = __ffma2_rn(y2, rc.A2[k], v);
      v = __ffma2_rn(z2, rc.zq2[k], v);
      v = __fmul2_rn(v, x2);
      v = __ffma2_rn(v, rc.a2[k], rc.nref2[k]);
      if (MASKED) {
        if (8 * n >= lim[k]) v.x = -INFINITY;
        if (8 * n + 1 >= lim[k]) v.y = -INFINITY;
      }
      asm("max.f32 %0, %0, %1, %2;" : "+f"(emax[k]) : "f"(v.x), "f"(v.y));
      if (!MAX_ONLY) {
        const float p0 = fast_exp2(v.x), p1 = fast_exp2(v.y);
        lsum2[k] = __fadd2_rn(lsum2[k], make_float2(p0, p1));
        pw[2 * n + k] = H16::pack(p0, p1);            // P rounded to 16 bit (quant_flash_attn.py:75)
      }
    }
  }
}

template <typename T, int D, int MODE, int NQT, bool SHORT>
__global__ void __launch_bounds__(TcCfg<D, MODE, NQT, SHORT>::THREADS, TcCfg<D, MODE, NQT, SHORT>::CTAS_PER_SM)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const TcFwdParams p) {
  using C = TcCfg<D, MODE, NQT, SHORT>;
  constexpr bool REF = C::REF, CTR = C::CTR;
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
  constexpr int B_QSCALED = B_ODONE + C::NQT;       // REF: the softmax warps have scaled Q in shared memory
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
    *abort_flag = launch_aborted(p.epoch) ? 1 : 0;     // a CTA of this launch already gave up: drain quickly
    mbar_init(BAR(B_QFULL), 1);
    for (int i = 0; i < C::KSTAGES; ++i) { mbar_init(BAR(B_KFULL + i), 1); mbar_init(BAR(B_KEMPTY + i), 1); }
    // a V stage is filled by one TMA transaction, or (RAW) by the softmax warps, one arrival each
    for (int i = 0; i < C::VSTAGES; ++i) {
      mbar_init(BAR(B_VFULL + i), C::RAW ? C::CONV_WARPS : 1);
      mbar_init(BAR(B_VEMPTY + i), 1);
    }
    for (int i = 0; i < C::MSTAGES; ++i) { mbar_init(BAR(B_MFULL + i), 1); mbar_init(BAR(B_MEMPTY + i), C::SOFTMAX_THREADS / 32); }
    for (int t = 0; t < C::NQT; ++t) {
      mbar_init(BAR(B_SFULL + t), 1);
      mbar_init(BAR(B_PFULL + t), C::LIVE_WARPS);   // one arrival per softmax warp of the tile
      mbar_init(BAR(B_ODONE + t), 1);
    }
    mbar_init(BAR(B_QSCALED), C::SHORT ? C::LIVE_WARPS : C::SOFTMAX_THREADS / 32);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < C::CTRL_WARPS) {
  if (warp == 0) {
    // ================================================================ producer
    if (lane == 0 && CTR) { prefetch_tmap(&tmK); prefetch_tmap(&tmV); }
    if (lane == 0 && !CTR) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
      int q_tiles = 0;
      for (int t = 0; t < C::NQT; ++t) q_tiles += (n_t[t] > 0);
      mbar_arrive_expect_tx(BAR(B_QFULL), q_tiles * C::Q_BYTES);
      for (int t = 0; t < C::NQT; ++t) {
        if (n_t[t] == 0) continue;
        if constexpr (REF) {      // 16-bit rows: D/64 panels of 128-byte rows, like the V^ tiles
          for (int pn = 0; pn < C::V_PANELS; ++pn)
            tma_load_4d(sbase + C::Q_OFF + t * C::Q_BYTES + pn * C::Q_PANEL_BYTES, &tmQ, BAR(B_QFULL), pn * 64,
                        m0 + t * C::BM, h, b);
        } else {
          tma_load_4d(sbase + C::Q_OFF + t * C::Q_BYTES, &tmQ, BAR(B_QFULL), 0, m0 + t * C::BM, h, b);
        }
      }
    }
    const int hkv = h / (p.H / p.Hkv);            // the K/V head this query head reads
    const int64_t tok_k0 = (static_cast<int64_t>(b) * p.Hkv + hkv) * p.Skv;
    bool ok = true;
    for (int j = 0; j < n_max && ok; ++j) {
      const int n0 = j * C::BN;
      const int vs = j % C::VSTAGES;
      if constexpr (!REF) {
        const int ks = j % C::KSTAGES, ms = j % C::MSTAGES;
        // K tile
        ok = mbar_wait(BAR(B_KEMPTY + ks), ((j / C::KSTAGES) & 1) ^ 1, abort_flag, p.epoch);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(BAR(B_KFULL + ks), C::K_BYTES);
          if constexpr (CTR) {
            for (int pn = 0; pn < C::V_PANELS; ++pn)
              tma_load_4d(sbase + C::K_OFF + ks * C::K_BYTES + pn * C::V_PANEL_BYTES, &tmK, BAR(B_KFULL + ks), pn * 64,
                          n0, hkv, b);
          } else {
            tma_load_4d(sbase + C::K_OFF + ks * C::K_BYTES, &tmK, BAR(B_KFULL + ks), 0, n0, hkv, b);
          }
        }
        // per-column constants z_k, -sum(k), s_k
        ok = mbar_wait(BAR(B_MEMPTY + ms), ((j / C::MSTAGES) & 1) ^ 1, abort_flag, p.epoch);
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
            if (!CTR) {
              zk = static_cast<float>(p.k_zp[tok_k0 + n]);
              nks = -static_cast<float>(p.k_sum[tok_k0 + n]);
            }
          }
          // layout for the softmax threads: thread q of a quad owns columns 8n+2q, 8n+2q+1; the constants of two
          // column groups (n even, n odd) are packed into three 16-byte words {z_k}, {-sum(k)}, {s_k} (CTR: {s_k})
          const int n8 = col >> 3, qq = (col >> 1) & 3, e = col & 1;
          if constexpr (CTR) {
            meta[((n8 >> 1) * 4 + qq) * 4 + (n8 & 1) * 2 + e] = sk;
          } else {
            float* dst = meta + (((n8 >> 1) * 4 + qq) * 3) * 4 + (n8 & 1) * 2 + e;
            dst[0] = zk;
            dst[4] = nks;
            dst[8] = sk;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_MFULL + ms));
      }
      if (!ok) break;
      if constexpr (C::RAW) break;                // nothing to stream: the softmax warps fill the V stages
      // V tile (D/64 panels of 128 bytes x BN rows)
      ok = mbar_wait(BAR(B_VEMPTY + vs), ((j / C::VSTAGES) & 1) ^ 1, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(BAR(B_VFULL + vs), C::V_BYTES);
        for (int pn = 0; pn < C::V_PANELS; ++pn)
          tma_load_4d(sbase + C::V_OFF + vs * C::V_BYTES + pn * C::V_PANEL_BYTES, &tmV, BAR(B_VFULL + vs), pn * 64, n0,
                      hkv, b);
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t kF16Fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      // logits: int8 x int8 -> int32, or (REF) 16-bit x 16-bit -> fp32 with both operands K-major
      constexpr uint32_t kIdescQK = REF ? make_idesc(1, kF16Fmt, kF16Fmt, 0, 0, C::BM, C::BN)
                                  : CTR ? make_idesc(1, 0, 0, 0, 0, C::BM, C::BN)       // centered codes are fp16 for both T
                                        : make_idesc(2, 1, 1, 0, 0, C::BM, C::BN);
      constexpr uint32_t kIdescPV = make_idesc(1, kF16Fmt, kF16Fmt, 0, 1, C::BM, D);
      constexpr uint64_t kQKSwz = (D == 128) ? kSwizzle128B : kSwizzle64B;
      bool ok = CTR ? true : mbar_wait(BAR(B_QFULL), 0, abort_flag, p.epoch);
      // REF: Q * sm_scale, rounded, in place; CTR: Q codes centered into shared memory by the softmax warps
      if ((REF || CTR) && ok) ok = mbar_wait(BAR(B_QSCALED), 0, abort_flag, p.epoch);
      tc_fence_after_sync();

      auto issue_qk = [&](int j, int t) {
        if constexpr (REF || CTR) {
          // REF: K^ is the V^ tile of stage j (the same tensor); CTR: the centered K tile of its own ring.  Both:
          // rows = keys, 128-byte swizzled panels of 64 columns
          const uint32_t kv = CTR ? sbase + C::K_OFF + (j % (CTR ? C::KSTAGES : 1)) * C::K_BYTES
                                  : sbase + C::V_OFF + (j % C::VSTAGES) * C::V_BYTES;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k / 4) * C::V_PANEL_BYTES + (k % 4) * 32;
            // (SHORT: the 128-row descriptor runs past the 32 rows of Q that exist; see TcCfg)
            const uint32_t offa = (k / 4) * C::Q_PANEL_BYTES + (k % 4) * 32;
            const uint64_t da = make_smem_desc(sbase + C::Q_OFF + t * C::Q_BYTES + offa, 16, 1024, kSwizzle128B);
            const uint64_t db = make_smem_desc(kv + off, 16, 1024, kSwizzle128B);
            mma_f16_ss(tmem + C::S_COL + t * C::BN, da, db, kIdescQK, k > 0);
          }
        } else {
          const int ks = j % C::KSTAGES;
          const uint64_t da = make_smem_desc(sbase + C::Q_OFF + t * C::Q_BYTES, 16, C::QK_SWIZZLE_ROWS_BYTES, kQKSwz);
          const uint64_t db = make_smem_desc(sbase + C::K_OFF + ks * C::K_BYTES, 16, C::QK_SWIZZLE_ROWS_BYTES, kQKSwz);
#pragma unroll
          for (int k = 0; k < D / 32; ++k)
            mma_i8_ss(tmem + C::S_COL + t * C::BN, desc_advance(da, k * 32), desc_advance(db, k * 32), kIdescQK, k > 0);
        }
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
      // the tile the logits of step j need: the K stage (int8 mode) or the V^ stage itself (REF)
      auto wait_k = [&](int j) {
        if constexpr (REF) return mbar_wait(BAR(B_VFULL + j % C::VSTAGES), (j / C::VSTAGES) & 1, abort_flag, p.epoch);
        else return mbar_wait(BAR(B_KFULL + j % C::KSTAGES), (j / C::KSTAGES) & 1, abort_flag, p.epoch);
      };
      auto release_k = [&](int j) {
        if constexpr (!REF) mma_commit(BAR(B_KEMPTY + j % C::KSTAGES));
      };

      if (ok && n_max > 0) {
        ok = wait_k(0);
        if (ok) {
          tc_fence_after_sync();
          for (int t = 0; t < C::NQT; ++t)
            if (0 < n_t[t]) issue_qk(0, t);
          release_k(0);
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int vs = j % C::VSTAGES;
        ok = mbar_wait(BAR(B_VFULL + vs), (j / C::VSTAGES) & 1, abort_flag, p.epoch);
        if (!ok) break;
        bool kwaited = false;
        for (int t = 0; t < C::NQT && ok; ++t) {
          if (j < n_t[t]) {
            ok = mbar_wait(BAR(B_PFULL + t), j & 1, abort_flag, p.epoch);
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv(j, t);
          }
          if (j + 1 < n_t[t]) {
            if (!kwaited) {
              ok = wait_k(j + 1);
              if (!ok) break;
              tc_fence_after_sync();
              kwaited = true;
            }
            issue_qk(j + 1, t);
          }
        }
        if (!ok) break;
        mma_commit(BAR(B_VEMPTY + vs));
        if (kwaited) release_k(j + 1);
      }
    }
  }
  } else {
    // ================================================================ softmax
    // One warp per 16 rows of a query tile.  S is read in the 16x256b fragment layout: thread (g, q) of the
    // warp owns rows g, g+8 of its 16-lane half and columns 8n+2q, 8n+2q+1, so the three per-column constants
    // are fetched from shared memory once per two rows and row reductions are two quad shuffles.
    // P = exp2(logit - ref) is formed in the same pass that finds the tile max, against a reference that is
    // only raised (by a whole number: exact power-of-two rescale of O, l and P) when a tile exceeds it by
    // more than kGrow; after the first tiles that almost never happens.
    const int sw = warp - C::CTRL_WARPS;
    const int t = sw >> 3;                         // query tile of this warpgroup
    const int hh = (sw >> 2) & 1;                  // which 16 lanes of the quarter
    const int wq = warp & 3;                       // tensor-memory lane quarter this warp may access
    const int g = lane >> 2, q = lane & 3;
    const uint32_t lanes = static_cast<uint32_t>(wq * 32 + hh * 16) << 16;
    const uint32_t tS = tmem + lanes + C::S_COL + t * C::BN;
    const uint32_t tO = tmem + lanes + C::O_COL + t * D;
    int rowk[2];
    RowConst2 rc;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      rowk[k] = m0 + t * C::BM + wq * 32 + hh * 16 + g + 8 * k;
      float A = 0.f, zq = 0.f, a = 0.f;
      if (!REF && rowk[k] < p.Sq) {
        const int64_t tk = static_cast<int64_t>(bh) * p.Sq + rowk[k];
        const int z = p.q_zp[tk];
        zq = static_cast<float>(z);
        A = static_cast<float>(D * z - p.q_sum[tk]);
        a = half_bits_to_f32(p.q_scale[tk]) * p.sm_scale * kLog2e;
      }
      rc.a2[k] = make_float2(a, a);
      rc.A2[k] = make_float2(A, A);
      rc.zq2[k] = make_float2(zq, zq);
      rc.nref2[k] = make_float2(0.f, 0.f);
    }
    // largest excess over the reference that may be fixed by rescaling P in registers (P must not have
    // overflowed its 16-bit type); beyond that the tile is recomputed from S, which is still intact
    constexpr float kInRegMax = std::is_same<T, __half>::value ? 15.0f : 100.0f;
    // how far (in powers of two) a tile may exceed the reference before the reference is raised.  P is stored in
    // T: fp16 keeps P <= 2^14 inside its range; bf16 has fp32's exponent range and constant relative
    // precision, so P, l and O may carry a factor up to 2^64 and the rescale path becomes rare even for
    // heavy-tailed logits
    constexpr float kGrow = std::is_same<T, __half>::value ? 14.0f : 64.0f;
    // a reference is set this far above the maximum it is derived from: row maxima of later tiles usually exceed
    // it by a few standard deviations of the logits, and starting above moves many rows out of the rescale path.
    // The result does not depend on the reference; P merely starts at 2^-margin instead of 1 (fp16 keeps its
    // largest P well inside the normal range)
    constexpr float kMargin = std::is_same<T, __half>::value ? 4.0f : 32.0f;
    float ref[2] = {0.f, 0.f}, l_run[2] = {0.f, 0.f};
    const int my_n = n_t[t];
    const bool rows_dead = m0 + t * C::BM + wq * 32 + hh * 16 >= p.Sq;      // warp-uniform
    bool ok = true;
    // RAW: K^ = V^ tile `jt` = (code - zp) * fp16(scale) rounded to T (quant_flash_attn.py:65-66), from the codes in
    // global memory into V stage jt % VSTAGES, in the 128-byte-swizzled panel layout a TMA load would produce.  The
    // loads are issued before the wait for the stage, so they are in flight while the P.V that still reads it ends.
    constexpr int CPR = D / 16;                                     // 16-code chunks per key
    const int hkv_c = h / (p.H / p.Hkv);
    const int8_t* code_base = p.kv_codes + static_cast<int64_t>(b) * p.kv_stride[0] + static_cast<int64_t>(hkv_c) * p.kv_stride[1];
    const int64_t code_tok0 = (static_cast<int64_t>(b) * p.Hkv + hkv_c) * p.Skv;
    // Chunk `idx` of a tile = 16 codes of one key.  Consecutive groups of four chunks walk down the keys inside one
    // 64-column panel before moving to the next panel: the eight lanes of a quarter warp then store two rows of
    // the same panel, whose 16-byte pieces land in eight different bank groups under the 128-byte swizzle (a whole
    // 256-byte row per quarter warp would hit four bank groups twice).
    auto chunk_row = [](int idx) { return (idx >> 2) % C::BN; };
    auto chunk_col = [](int idx) { return (idx & 3) + 4 * (idx / (4 * C::BN)); };
    // the codes of chunk `idx` of tile jt and the key's scale / zp
    auto load_chunk = [&](int jt, int idx, uint4& raw, uint32_t& szp) {
      const int key = jt * C::BN + chunk_row(idx);
      raw = make_uint4(0, 0, 0, 0);
      szp = 0;
      if (key < p.Skv) {
        raw = __ldg(reinterpret_cast<const uint4*>(code_base + static_cast<int64_t>(key) * p.kv_stride[2] + 16 * chunk_col(idx)));
        szp = static_cast<uint32_t>(p.k_scale[code_tok0 + key]) |
              (static_cast<uint32_t>(static_cast<uint8_t>(p.k_zp[code_tok0 + key])) << 16);
      }
    };
    // ... dequantized and stored into V stage vs (keys past the end: zeros)
    auto store_chunk = [&](int vs, int idx, const uint4& raw, uint32_t szp) {
      const int r = chunk_row(idx), c = chunk_col(idx);
      const uint16_t sc = static_cast<uint16_t>(szp & 0xffffu);
      const int zp = static_cast<int8_t>(szp >> 16);
      uint4 lo, hi;
      if constexpr (std::is_same<T, __half>::value) {
        // code - zp is exact in fp16 and its product with the fp16 scale is rounded once: the same bits as the
        // fp32 product (exact, 20 significant bits) rounded to fp16
        const __half2 s2 = __half2half2(__ushort_as_half(sc));
        auto cv = [&](uint32_t w, uint32_t& o0, uint32_t& o1) {
          center4(w, zp, o0, o1);
          const __half2 a0 = __hmul2(*reinterpret_cast<const __half2*>(&o0), s2);
          const __half2 a1 = __hmul2(*reinterpret_cast<const __half2*>(&o1), s2);
          o0 = *reinterpret_cast<const uint32_t*>(&a0);
          o1 = *reinterpret_cast<const uint32_t*>(&a1);
        };
        cv(raw.x, lo.x, lo.y); cv(raw.y, lo.z, lo.w); cv(raw.z, hi.x, hi.y); cv(raw.w, hi.z, hi.w);
      } else {
        const float sf = half_bits_to_f32(sc), zf = static_cast<float>(zp);
        float f[4];
        dequant4(raw.x, zf, sf, f); lo.x = H16::pack(f[0], f[1]); lo.y = H16::pack(f[2], f[3]);
        dequant4(raw.y, zf, sf, f); lo.z = H16::pack(f[0], f[1]); lo.w = H16::pack(f[2], f[3]);
        dequant4(raw.z, zf, sf, f); hi.x = H16::pack(f[0], f[1]); hi.y = H16::pack(f[2], f[3]);
        dequant4(raw.w, zf, sf, f); hi.z = H16::pack(f[0], f[1]); hi.w = H16::pack(f[2], f[3]);
      }
      uint8_t* rowp = smem + C::V_OFF + vs * C::V_BYTES + (c / 4) * C::V_PANEL_BYTES + r * 128;
      const int ch = 2 * (c % 4);
      *reinterpret_cast<uint4*>(rowp + ((ch ^ (r & 7)) << 4)) = lo;
      *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ (r & 7)) << 4)) = hi;
    };
    // the stage is complete as far as this warp is concerned
    auto publish_stage = [&](int vs) {
      // generic-proxy writes must be visible to the tensor core's (async proxy) operand reads
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_VFULL + vs));
    };
    auto wait_stage_free = [&](int jt) -> bool {
      bool good = mbar_wait(BAR(B_VEMPTY + jt % C::VSTAGES), ((jt / C::VSTAGES) & 1) ^ 1, abort_flag, p.epoch);
      return __all_sync(0xffffffffu, good);
    };
    // all softmax warps share the conversion of a tile (the one-tile kernel with 33 to 128 query rows)
    auto convert_tile = [&](int jt) -> bool {
      constexpr int NCH = C::BN * CPR / C::SOFTMAX_THREADS;         // chunks per thread
      uint4 raw[NCH];
      uint32_t szp[NCH];
#pragma unroll
      for (int i = 0; i < NCH; ++i) load_chunk(jt, tid - C::CTRL_THREADS + i * C::SOFTMAX_THREADS, raw[i], szp[i]);
      if (!wait_stage_free(jt)) return false;
#pragma unroll
      for (int i = 0; i < NCH; ++i) store_chunk(jt % C::VSTAGES, tid - C::CTRL_THREADS + i * C::SOFTMAX_THREADS, raw[i], szp[i]);
      publish_stage(jt % C::VSTAGES);
      return true;
    };
    if constexpr (C::SHORT) {
      if (wq != 0) {
        // ---------------- dedicated converter warp (tensor-memory lanes 0-31 are out of its reach): walks the K/V
        // tiles on its own, paced only by the release of the stages, one tile of codes in registers ahead
        const int crank = sw - (sw > 2 ? 1 : 0) - (sw > 6 ? 1 : 0);          // 0..5 among the converter warps
        const int ctid = crank * 32 + lane;
        constexpr int CTHREADS = C::CONV_WARPS * 32;
        constexpr int NSLOT = (C::BN * CPR + CTHREADS - 1) / CTHREADS;
        uint4 rawA[NSLOT], rawB[NSLOT];
        uint32_t szA[NSLOT], szB[NSLOT];
        auto issue = [&](int jt, uint4 (&raw)[NSLOT], uint32_t (&szp)[NSLOT]) {
#pragma unroll
          for (int i = 0; i < NSLOT; ++i) {
            const int idx = ctid + i * CTHREADS;
            if (idx < C::BN * CPR) load_chunk(jt, idx, raw[i], szp[i]);
          }
        };
        auto emit = [&](int jt, const uint4 (&raw)[NSLOT], const uint32_t (&szp)[NSLOT]) -> bool {
          if (!wait_stage_free(jt)) return false;
#pragma unroll
          for (int i = 0; i < NSLOT; ++i) {
            const int idx = ctid + i * CTHREADS;
            if (idx < C::BN * CPR) store_chunk(jt % C::VSTAGES, idx, raw[i], szp[i]);
          }
          publish_stage(jt % C::VSTAGES);
          return true;
        };
        if (n_max > 0) issue(0, rawA, szA);
        for (int jt = 0; jt < n_max && ok; jt += 2) {
          if (jt + 1 < n_max) issue(jt + 1, rawB, szB);
          ok = emit(jt, rawA, szA);
          if (!ok || jt + 1 >= n_max) break;
          if (jt + 2 < n_max) issue(jt + 2, rawA, szA);
          ok = emit(jt + 1, rawB, szB);
        }
      }
    }
    if (!(C::SHORT && wq != 0)) {
    if constexpr (C::RAW && !C::SHORT) {
      for (int jt = 0; jt < C::VSTAGES && jt < n_max && ok; ++jt) ok = convert_tile(jt);
    }
    if constexpr (REF) {
      // q~ = (q * sm_scale) rounded to T (quant_flash_attn.py:52), in place in shared memory: an element-wise
      // pass does not care about the swizzled placement of the 16-byte chunks.  All sixteen warps share it.
      ok = mbar_wait(BAR(B_QFULL), 0, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        uint4* qs = reinterpret_cast<uint4*>(smem + C::Q_OFF);
        // (SHORT: the two softmax warps alone; the converters are already streaming codes)
        const int c0 = C::SHORT ? hh * 32 + lane : tid - C::CTRL_THREADS;
        constexpr int cstep = C::SHORT ? C::LIVE_WARPS * 32 : C::SOFTMAX_THREADS;
        for (int c = c0; c < C::NQT * C::Q_BYTES / 16; c += cstep) {
          uint4 v = qs[c];
          float2 f;
          f = H16::unpack(v.x); v.x = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
          f = H16::unpack(v.y); v.y = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
          f = H16::unpack(v.z); v.z = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
          f = H16::unpack(v.w); v.w = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
          qs[c] = v;
        }
        // generic-proxy writes must be visible to the tensor core's (async proxy) operand reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_QSCALED));
      }
    }
    if constexpr (CTR) {
      // Q' = q - z_q as fp16 (exact), written in the layout the 16-bit MMA reads: per tile D/64 panels of 128-byte
      // rows, 16-byte chunks XOR-swizzled with the row number (the placement a 128-byte-swizzled TMA load would
      // produce).  A thread converts 16 codes per turn; rows past the end of Q become zeros.
      constexpr int CPR = D / 16;                        // 16-code chunks per row
      const int8_t* qbase = p.q_codes + static_cast<int64_t>(b) * p.q_stride[0] + static_cast<int64_t>(h) * p.q_stride[1];
      for (int idx = tid - C::CTRL_THREADS; idx < C::NQT * C::BM * CPR; idx += C::SOFTMAX_THREADS) {
        const int r256 = idx / CPR, c = idx % CPR;
        const int row = m0 + r256;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (row < p.Sq) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(qbase + static_cast<int64_t>(row) * p.q_stride[2] + 16 * c));
          const int z = p.q_zp[static_cast<int64_t>(bh) * p.Sq + row];
          center4(v.x, z, lo.x, lo.y); center4(v.y, z, lo.z, lo.w); center4(v.z, z, hi.x, hi.y); center4(v.w, z, hi.z, hi.w);
        }
        const int t_ = r256 / C::BM, r = r256 % C::BM;
        uint8_t* rowp = smem + C::Q_OFF + t_ * C::Q_BYTES + (c / 4) * C::Q_PANEL_BYTES + r * 128;
        const int ch = 2 * (c % 4);
        *reinterpret_cast<uint4*>(rowp + ((ch ^ (r & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(rowp + (((ch + 1) ^ (r & 7)) << 4)) = hi;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(B_QSCALED));
    }
    for (int j = 0; j < n_max && ok; ++j) {
      const int ms = REF ? 0 : j % (REF ? 1 : C::MSTAGES);
      if (j < my_n) {
        if (!REF) ok = mbar_wait(BAR(B_MFULL + ms), (j / (REF ? 1 : C::MSTAGES)) & 1, abort_flag, p.epoch);
        const float4* meta = reinterpret_cast<const float4*>(smem + C::M_OFF + ms * C::M_BYTES) + (CTR ? 1 : 3) * q;
        // CTR: the per-key scales of all of this thread's columns are fetched BEFORE the wait for the logits.  While
        // the warps work on a tile the tensor core streams the other tile's operands out of shared memory at the
        // pipe's full rate, and a load issued then waits behind that stream; issued here it completes during
        // the wait.  (32 registers, which the packed P takes over block by block.)
        float4 xt[C::BN / 16];
        if constexpr (CTR) {
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
#pragma unroll
          for (int blk = 0; blk < C::BN / 16; ++blk) {
            xt[blk] = lds128(meta + blk * 4);
          }
        }
        if (ok) ok = mbar_wait(BAR(B_SFULL + t), j & 1, abort_flag, p.epoch);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (C::RAW && rows_dead) {
          // all sixteen rows of this warp lie past the last query: their logits need no softmax and their P is never
          // used (rows of an MMA are independent and these rows of O are not stored).  The warp only keeps the
          // hand-over barrier in step and does its share of the dequantization.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR(B_PFULL + t));
          if (!C::SHORT && j + C::VSTAGES < my_n) {
            ok = convert_tile(j + C::VSTAGES);
            if (!ok) break;
          }
          continue;
        }
        const int n0 = j * C::BN;
        int lim[2];                                   // first masked column of each row, relative to 2q
        bool any_masked = false;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          int cl = p.Skv - n0;
          if (p.causal) cl = min(cl, rowk[k] + 1 - n0);
          any_masked |= cl < C::BN;
          lim[k] = cl - 2 * q;
        }
        const bool masked = __any_sync(0xffffffffu, any_masked);
        float emax[2] = {-INFINITY, -INFINITY};
        float2 lsum2[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) lsum2[k] = make_float2(0.f, 0.f);
        uint32_t pw[32];                              // P of rows (g, g+8), 64 packed columns

        // processes the whole tile in blocks of 16 columns; the tensor-memory load of the next block is in
        // flight while the current one is computed.  MAXONLY computes only the row maxima (first tile)
        // RELOAD (the rare recompute): the scales are read again from shared memory, block by block
        auto run_tile = [&](auto maxonly_tag, auto masked_tag, auto reload_tag) {
          constexpr bool MAXONLY = decltype(maxonly_tag)::value;
          constexpr bool MASKED = decltype(masked_tag)::value;
          constexpr bool RELOAD = decltype(reload_tag)::value;
          constexpr int NBLK = C::BN / 16;
          uint32_t sreg[2][8];
          tmem_ld_16x256b_x2(tS, sreg[0]);
#pragma unroll
          for (int blk = 0; blk < NBLK; ++blk) {
            float4 xk;
            if constexpr (CTR) xk = RELOAD ? meta[blk * 4] : xt[blk];
            tmem_wait_ld_use(sreg[blk & 1]);
            if (blk + 1 < NBLK) tmem_ld_16x256b_x2(tS + (blk + 1) * 16, sreg[(blk + 1) & 1]);
            int lim_b[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) lim_b[k] = lim[k] - blk * 16;
            if constexpr (REF)
              softmax_block_ref<T, MASKED, MAXONLY>(sreg[blk & 1], lim_b, rc, emax, lsum2, pw + blk * 4);
            else if constexpr (CTR)
              softmax_block_ctr<T, MASKED, MAXONLY>(sreg[blk & 1], xk, lim_b, rc, emax, lsum2, pw + blk * 4);
            else
              softmax_block<T, C::BN, MASKED, MAXONLY>(sreg[blk & 1], meta + blk * 12, lim_b, rc, emax, lsum2,
                                                       pw + blk * 4);
          }
        };
        auto quad_max = [&]() {
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            emax[k] = fmaxf(emax[k], __shfl_xor_sync(0xffffffffu, emax[k], 1));
            emax[k] = fmaxf(emax[k], __shfl_xor_sync(0xffffffffu, emax[k], 2));
          }
        };

        if (j == 0) {
          // no reference yet: take the exact row max of the first tile
          if (masked) run_tile(std::true_type{}, std::true_type{}, std::false_type{}); else run_tile(std::true_type{}, std::false_type{}, std::false_type{});
          quad_max();
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            ref[k] = (emax[k] == -INFINITY) ? 0.f : emax[k] + kMargin;
            rc.nref2[k] = make_float2(-ref[k], -ref[k]);
            emax[k] = -INFINITY;
          }
        }
        if (masked) run_tile(std::false_type{}, std::true_type{}, std::false_type{}); else run_tile(std::false_type{}, std::false_type{}, std::false_type{});
        quad_max();

        // ---- rare: some row exceeded its reference by more than 2^kGrow
        const bool grow = emax[0] > kGrow || emax[1] > kGrow;
        if (__any_sync(0xffffffffu, grow)) {
          float kf[2], factor[2];
          bool redo = false;
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            // raise by a whole number (2^-kf is exact) to kMargin above the tile's maximum.  Rows whose P is
            // rescaled in registers need a representable factor, so their step is capped; rows that force the
            // recompute may step further: a factor that underflows to zero then drops contributions that are
            // below 2^-24 of the new ones anyway
            kf[k] = 0.f;
            if (emax[k] > kGrow) {
              kf[k] = ceilf(emax[k]) + kMargin;
              if (emax[k] <= kInRegMax) kf[k] = fminf(kf[k], 120.0f);
            }
            factor[k] = fast_exp2(-kf[k]);
            redo |= emax[k] > kInRegMax;
          }
          if (j > 0) {
            ok = mbar_wait(BAR(B_ODONE + t), (j - 1) & 1, abort_flag, p.epoch);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            // O of this warp's 16 rows, in the same fragment layout (the other 16 lanes of the quarter belong
            // to the partner warp, which may be rescaling them at the same time)
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t oreg[16];
              tmem_ld_16x256b_x4(tO + c * 32, oreg);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * factor[(i >> 1) & 1]);
              tmem_st_16x256b_x4(tO + c * 32, oreg);
            }
            tmem_wait_st();
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            l_run[k] *= factor[k];
            ref[k] += kf[k];
            rc.nref2[k] = make_float2(-ref[k], -ref[k]);
          }
          if (__any_sync(0xffffffffu, redo)) {
            // P may have overflowed its 16-bit type: recompute the tile against the new reference
#pragma unroll
            for (int k = 0; k < 2; ++k) { lsum2[k] = make_float2(0.f, 0.f); emax[k] = -INFINITY; }
            run_tile(std::false_type{}, std::true_type{}, std::true_type{});
          } else {
            // exact power-of-two rescale of the P already packed in registers and of its row sums
            uint32_t f2[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) { f2[k] = H16::pack(factor[k], factor[k]); lsum2[k].x *= factor[k]; lsum2[k].y *= factor[k]; }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              typename H16::T2 va = __hmul2(*reinterpret_cast<typename H16::T2*>(&pw[i]),
                                            *reinterpret_cast<const typename H16::T2*>(&f2[i & 1]));
              pw[i] = *reinterpret_cast<uint32_t*>(&va);
            }
          }
        }
        // one arrival per warp (the warp's reads of the constants are ordered before it by __syncwarp)
        __syncwarp();
        if (!REF && lane == 0) mbar_arrive(BAR(B_MEMPTY + ms));
#pragma unroll
        for (int k = 0; k < 2; ++k) l_run[k] += lsum2[k].x + lsum2[k].y;
        tmem_st_16x128b_x16(tS, pw);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_PFULL + t));
        if constexpr (C::RAW && !C::SHORT) {
          // the warps are idle now until the next logits arrive (P.V and the next Q.K^T run meanwhile): dequantize
          // the tile after the next one into the stage this step's P.V is about to release
          if (j + C::VSTAGES < my_n) {
            ok = convert_tile(j + C::VSTAGES);
            if (!ok) break;
          }
        }
      } else {
        // this query tile is done (causal): keep the per-column ring moving for the other tile
        if constexpr (!REF) {
          ok = mbar_wait(BAR(B_MFULL + ms), (j / C::MSTAGES) & 1, abort_flag, p.epoch);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (lane == 0) mbar_arrive(BAR(B_MEMPTY + ms));
        }
      }
    }
    // ---------------- epilogue: O / l -> 16 bit, LSE = (ref + log2 l) ln 2
    if (ok && my_n > 0 && !(C::RAW && rows_dead)) {
      ok = mbar_wait(BAR(B_ODONE + t), (my_n - 1) & 1, abort_flag, p.epoch);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        // row sums: the four threads of a quad hold partial sums of the same rows
        float inv[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          float l = l_run[k];
          l += __shfl_xor_sync(0xffffffffu, l, 1);
          l += __shfl_xor_sync(0xffffffffu, l, 2);
          if (q == 0 && rowk[k] < p.Sq)
            p.lse[static_cast<int64_t>(bh) * p.lse_stride + rowk[k]] = (ref[k] + log2f(l)) * kLn2;
          inv[k] = l > 0.f ? 1.f / l : 0.f;
        }
        T* obase = static_cast<T*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t oreg[16];
          tmem_ld_16x256b_x4(tO + c * 32, oreg);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            if (rowk[k] < p.Sq) {
              T* orow = obase + static_cast<int64_t>(rowk[k]) * p.o_stride[2] + c * 32 + 2 * q;
#pragma unroll
              for (int n = 0; n < 4; ++n)
                *reinterpret_cast<uint32_t*>(orow + 8 * n) =
                    H16::pack(__uint_as_float(oreg[4 * n + 2 * k]) * inv[k], __uint_as_float(oreg[4 * n + 2 * k + 1]) * inv[k]);
            }
          }
        }
      }
    }
    }   // softmax (not converter) warps
  }

  // ================================================================ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
  if (tid == 0 && *abort_flag && p.status) *p.status = QFA_STATUS_WAIT_TIMEOUT;
}

template <typename T, int D, int MODE, int NQT = 2, bool SHORT = false>
static int launch_tc(const QfaFwdArgs& a, cudaStream_t stream) {
  using C = TcCfg<D, MODE, NQT, SHORT>;
  constexpr bool REF = C::REF, CTR = C::CTR;
  CUtensorMap tmQ, tmK, tmV;
  const CUtensorMapSwizzle qk_swz = (D == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUtensorMapDataType vdt =
      std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int64_t Hkv = a.Hkv ? a.Hkv : a.H;
  bool ok;
  if (REF) {
    // 16-bit Q with the caller's strides, in 64-column panels; the K tensor map is not used (K^ is the V^ tile)
    ok = make_tmap_4d(&tmQ, a.q, vdt, 2, D, a.Sq, a.H, a.B, 2ull * a.q_stride[2], 2ull * a.q_stride[1],
                      2ull * a.q_stride[0], 64, C::QROWS, CU_TENSOR_MAP_SWIZZLE_128B);
  } else if (CTR) {
    // centered K: fp16 contiguous (B, Hkv, Skv, D), panels like V^; Q is not loaded by TMA in this mode
    ok = make_tmap_4d(&tmK, a.k_ctr, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, D, a.Skv, Hkv, a.B, 2ull * D, 2ull * D * a.Skv,
                      2ull * D * a.Skv * Hkv, 64, C::BN, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    ok = make_tmap_4d(&tmQ, a.qq.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, a.Sq, a.H, a.B, a.qq.stride[2],
                      a.qq.stride[1], a.qq.stride[0], D, C::BM, qk_swz);
    ok = ok && make_tmap_4d(&tmK, a.k.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, D, a.Skv, Hkv, a.B, a.k.stride[2],
                            a.k.stride[1], a.k.stride[0], D, C::BN, qk_swz);
  }
  if (C::RAW)
    tmV = tmQ;                                         // placeholder: the kernel dequantizes the codes itself
  else
    ok = ok && make_tmap_4d(&tmV, a.v_hat, vdt, 2, D, a.Skv, Hkv, a.B, 2ull * D, 2ull * D * a.Skv,
                            2ull * D * a.Skv * Hkv, 64, C::BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (REF) tmK = tmV;
  if (CTR) tmQ = tmK;                                  // placeholder: the kernel does not read it
  if (!ok) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  TcFwdParams p;
  p.kv_codes = a.k.codes;
  for (int i = 0; i < 3; ++i) p.kv_stride[i] = a.k.stride[i];
  p.q_codes = a.qq.codes;
  for (int i = 0; i < 3; ++i) p.q_stride[i] = a.qq.stride[i];
  p.q_scale = a.qq.scale; p.q_zp = a.qq.zp; p.q_sum = a.qq.rowsum;
  p.k_scale = a.k.scale; p.k_zp = a.k.zp; p.k_sum = a.k.rowsum;
  p.o = a.o;
  for (int i = 0; i < 3; ++i) p.o_stride[i] = a.o_stride[i];
  p.lse = a.lse; p.lse_stride = a.lse_stride;
  p.H = static_cast<int>(a.H); p.Hkv = static_cast<int>(Hkv); p.Sq = static_cast<int>(a.Sq); p.Skv = static_cast<int>(a.Skv);
  p.sm_scale = a.sm_scale; p.causal = a.causal; p.status = a.status;
  p.epoch = next_launch_epoch();
  auto kern = attn_fwd_tc_kernel<T, D, MODE, NQT, SHORT>;
  static DeviceOnce attr_done;
  int rc = once_per_device(attr_done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    return QFA_OK;
  });
  if (rc != QFA_OK) return rc;
  const int64_t n_ctas = ((a.Sq + C::NQT * C::BM - 1) / (C::NQT * C::BM)) * a.B * a.H;
  if (n_ctas > 0x7fffffffLL) return QFA_ERR_SHAPE;
  kern<<<static_cast<unsigned>(n_ctas), C::THREADS, C::SMEM, stream>>>(tmQ, tmK, tmV, p);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

// ------------------------------------------------------------------ self-test of the bounded wait
// One thread waits on an mbarrier that nothing ever arrives at, with a short budget; the wait must give up, raise
// the abort flag and the device-wide abort word (shared with the forward kernels of this file) and report
// QFA_STATUS_WAIT_TIMEOUT through `status`.  The kernel returns normally and the context stays usable.
__global__ void wait_timeout_selftest_kernel(unsigned long long budget_ns, unsigned int epoch, int32_t* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, abort_flag, epoch, budget_ns);
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && status) *status = QFA_STATUS_WAIT_TIMEOUT;
}

int wait_timeout_selftest_entry(uint64_t budget_ns, int32_t* status, cudaStream_t stream) {
  if (!status) return QFA_ERR_NULL;
  if (budget_ns == 0 || budget_ns > 100ull * 1000 * 1000) return QFA_ERR_SHAPE;      // at most 100 ms
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(budget_ns, next_launch_epoch(), status);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

// The tcgen05 kernel takes int8-mode problems with the dequantized V supplied by the quantizer, and REF-mode
// problems with more than 16 query rows: 16-bit Q and K^ = V^ feed a 16-bit MMA for the logits.  With more than 128
// query rows the one K/V tensor must be supplied dequantized (v_hat); up to 128 the kernel dequantizes the codes
// itself and v_hat is ignored.  (Up to 16 query rows the short-query kernels are the faster path.)
int attn_fwd_tc_supported(const QfaFwdArgs& a) {
  if (a.D != 128 && a.D != 64) return 0;
  if (a.mode == QFA_MODE_REF) {
    // Up to 16 query rows the mma.sync short-query kernels are as fast or faster (Z256 H16 NKV4096 D128 at 16 rows:
    // 1.17 ms against 1.23 ms here); from 17 rows on this kernel wins (32 rows: 0.70 against 1.06 ms).
    if (a.causal || a.Sq <= 16 || !a.q) return 0;
    if (a.k.codes != a.v.codes || a.k.scale != a.v.scale || a.k.zp != a.v.zp) return 0;
    if (a.Hkv != 0 && a.Hkv != a.H) return 0;
    if (a.Sq <= 128) return 1;                        // one query tile: the kernel dequantizes K/V itself
    return (a.v_hat && (reinterpret_cast<uintptr_t>(a.v_hat) & 15) == 0) ? 1 : 0;
  }
  if (!a.v_hat || (reinterpret_cast<uintptr_t>(a.v_hat) & 15) != 0) return 0;
  if (a.mode == QFA_MODE_INT8) return a.sm_scale > 0.f ? 1 : 0;      // (k_ctr, when given, was validated by the caller)
  return 0;
}

int attn_fwd_tc_entry(const QfaFwdArgs& a, cudaStream_t stream) {
  const bool bf = a.dtype == QFA_BF16;
  if (a.mode == QFA_MODE_REF && a.Sq <= 32) {      // at most 32 query rows: dedicated converter warps, three K/V stages
    if (a.D == 128) return bf ? launch_tc<__nv_bfloat16, 128, kModeRef, 1, true>(a, stream) : launch_tc<__half, 128, kModeRef, 1, true>(a, stream);
    if (a.D == 64) return bf ? launch_tc<__nv_bfloat16, 64, kModeRef, 1, true>(a, stream) : launch_tc<__half, 64, kModeRef, 1, true>(a, stream);
    return QFA_ERR_HEAD_DIM;
  }
  if (a.mode == QFA_MODE_REF && a.Sq <= 128) {      // one query tile per head: two heads per SM
    if (a.D == 128) return bf ? launch_tc<__nv_bfloat16, 128, kModeRef, 1>(a, stream) : launch_tc<__half, 128, kModeRef, 1>(a, stream);
    if (a.D == 64) return bf ? launch_tc<__nv_bfloat16, 64, kModeRef, 1>(a, stream) : launch_tc<__half, 64, kModeRef, 1>(a, stream);
    return QFA_ERR_HEAD_DIM;
  }
  if (a.mode == QFA_MODE_REF) {
    if (a.D == 128) return bf ? launch_tc<__nv_bfloat16, 128, kModeRef>(a, stream) : launch_tc<__half, 128, kModeRef>(a, stream);
    if (a.D == 64) return bf ? launch_tc<__nv_bfloat16, 64, kModeRef>(a, stream) : launch_tc<__half, 64, kModeRef>(a, stream);
    return QFA_ERR_HEAD_DIM;
  }
  if (a.k_ctr) {   // int8-mode arithmetic on centered fp16 operands
    if (a.D == 128) return bf ? launch_tc<__nv_bfloat16, 128, kModeCtr>(a, stream) : launch_tc<__half, 128, kModeCtr>(a, stream);
    if (a.D == 64) return bf ? launch_tc<__nv_bfloat16, 64, kModeCtr>(a, stream) : launch_tc<__half, 64, kModeCtr>(a, stream);
    return QFA_ERR_HEAD_DIM;
  }
  if (a.D == 128) return bf ? launch_tc<__nv_bfloat16, 128, kModeI8>(a, stream) : launch_tc<__half, 128, kModeI8>(a, stream);
  if (a.D == 64) return bf ? launch_tc<__nv_bfloat16, 64, kModeI8>(a, stream) : launch_tc<__half, 64, kModeI8>(a, stream);
  return QFA_ERR_HEAD_DIM;
}

}  // namespace qfa
