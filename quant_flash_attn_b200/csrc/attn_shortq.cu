// Short-query attention over one quantized K/V tensor: the reference's own operating regime
// (quant_flash_attn.py: one program per head holds ALL of Q, test_speed.py:57 uses N_CTX_Q = 16).
//
// With 16..32 query rows per head the problem is bound by reading the int8 K/V codes, not by tensor-core
// math, and a 64-row query tile would waste 3/4 of every MMA.  These kernels therefore
//   * give one CTA the whole head (all query rows, every K/V tile), as the reference does
//     (quant_flash_attn.py:37-56, :120-141),
//   * split each 64-token K/V tile BY COLUMNS among the 4 warps (16 tokens each), every warp working on all
//     query rows with its own online-softmax state; the warps' partial results are merged once at the end,
//   * dequantize K/V exactly as the reference ((code - zp) * scale rounded to the 16-bit dtype,
//     quant_flash_attn.py:65-66) while staging it into shared memory; the codes of the next four tiles are
//     in flight as bulk copies into a shared-memory ring (the kernels are bound by the latency of that stream:
//     with one tile in flight per CTA they reached a fifth of the HBM bandwidth),
//   * in the backward keep dQ in registers for the whole walk (no atomics, no scratch) and write each
//     dKV tile exactly once, dKV = dV + sm_scale*dK (quant_flash_attn.py:161).
// REF mode only (16-bit Q, K and V the same tensor), Sq <= 32.
#include "qfa_common.cuh"
#include "sm100_ptx.cuh"

namespace qfa {

struct ShortQDev {
  const void* q;
  int64_t q_stride[3];
  QfaQuantTensor kv;
  // forward
  void* o;
  int64_t o_stride[3];
  float* lse;
  // backward
  const void* d_o;
  int64_t do_stride[3];
  const float* lse_in;
  const float* delta;
  void* dq;
  int64_t dq_stride[3];
  void* dkv;
  int64_t dkv_stride[3];
  int64_t lse_stride;
  int H, Sq, Skv;
  float sm_scale;
  unsigned int epoch;    // launch epoch for the bounded waits (next_launch_epoch)
  int32_t* status;
};

template <int D, int MT>
struct SqCfg {
  static constexpr int BN = 64, THREADS = 128;
  static constexpr int ROWS = 16 * MT;
  static constexpr int T_STRIDE = 2 * D + 16;                // padded 16-bit rows: conflict-free ldmatrix
  static constexpr int CHUNKS = BN * D / 16 / THREADS;       // 16-code chunks per thread per tile
  static constexpr int CPR = D / 16;
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = Q_OFF + ROWS * T_STRIDE;     // backward only
  static constexpr int KV_OFF_FWD = Q_OFF + ROWS * T_STRIDE;
  static constexpr int KV_OFF_BWD = DO_OFF + ROWS * T_STRIDE;
  static constexpr int TILES_FWD = KV_OFF_FWD + BN * T_STRIDE;
  static constexpr int MERGE_FWD = 4 * ROWS * D * 4 + 4 * ROWS * 8;      // O partials + (m, l) per warp
  static constexpr int DS_STRIDE = 2 * ROWS + 16;            // dS^T rows [kv][q], 16 bit
  static constexpr int DS_OFF = KV_OFF_BWD + BN * T_STRIDE;
  static constexpr int TILES_BWD = DS_OFF + BN * DS_STRIDE;
  static constexpr int MERGE_BWD = 4 * ROWS * D * 4;
  // ring of raw code tiles filled by bulk copies + (scale, zero point) per key + one mbarrier per stage; it sits
  // behind the larger of the tile / merge regions so that the final merge never overlaps it
  // (the forward keeps four tiles in flight with three CTAs per SM; the backward two tiles with four CTAs per SM)
  static constexpr int NST_FWD = 4, NST_BWD = 2;
  static constexpr int CODE_BYTES = BN * D;
  static constexpr int ring_bytes(int nst) { return nst * CODE_BYTES + nst * BN * 8 + nst * 8 + 16; }
  static constexpr int RING_OFF_FWD = ((TILES_FWD > MERGE_FWD ? TILES_FWD : MERGE_FWD) + 127) / 128 * 128;
  static constexpr int RING_OFF_BWD = ((TILES_BWD > MERGE_BWD ? TILES_BWD : MERGE_BWD) + 127) / 128 * 128;
  static constexpr int SMEM_FWD = RING_OFF_FWD + ring_bytes(NST_FWD);
  static constexpr int SMEM_BWD = RING_OFF_BWD + ring_bytes(NST_BWD);
};

// 16 int8 codes -> 16 values (code - zp) * scale rounded to T, written as 32 bytes.
template <typename T>
__device__ __forceinline__ void dequant16_store(uint8_t* dst, const uint4& codes, float zp, float scale) {
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
// fp16 fast path: 0x6400 | (code ^ 0x80) is the half 1024 + (code + 128); subtracting 1152 + zp is exact and the
// product with the fp16 scale is rounded once, exactly like the fp32 product rounded to fp16.
template <>
__device__ __forceinline__ void dequant16_store<__half>(uint8_t* dst, const uint4& codes, float zp, float scale) {
  const __half2 off = __float2half2_rn(1152.0f + zp);
  const __half2 sc = __float2half2_rn(scale);
  auto cvt2 = [&](uint32_t w, uint32_t sel) -> uint32_t {
    uint32_t h = __byte_perm(w ^ 0x80808080u, 0x64646464u, sel);   // two halves 1024 + u
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&h), off), sc);
    return *reinterpret_cast<uint32_t*>(&v);
  };
  uint4 lo, hi;
  lo.x = cvt2(codes.x, 0x4140); lo.y = cvt2(codes.x, 0x4342);
  lo.z = cvt2(codes.y, 0x4140); lo.w = cvt2(codes.y, 0x4342);
  hi.x = cvt2(codes.z, 0x4140); hi.y = cvt2(codes.z, 0x4342);
  hi.z = cvt2(codes.w, 0x4140); hi.w = cvt2(codes.w, 0x4342);
  *reinterpret_cast<uint4*>(dst) = lo;
  *reinterpret_cast<uint4*>(dst + 16) = hi;
}

// K/V code tiles streamed through a shared-memory ring: one thread issues an untiled bulk copy per 64-token tile
// (the rows of a head are contiguous), NST tiles ahead of the consumer; the per-key scale / zero point of a tile
// travel through registers for one iteration and then into the ring's metadata slot.  commit() waits for the
// tile's bytes (bounded wait) and dequantizes it into the padded 16-bit tile the MMAs read.
template <int D, int MT, int NST>
struct KvRing {
  using C = SqCfg<D, MT>;
  uint8_t* codes;            // [NST][BN * D]
  float2* meta;              // [NST][BN] (scale, zero point)
  uint32_t bar0;             // NST mbarriers
  volatile int* abort_flag;
  const int8_t* src;
  const uint16_t* scale;
  const int8_t* zp;
  int skv, n_tiles;
  unsigned int epoch;
  float2 pend;
  int pend_slot;

  __device__ __forceinline__ void issue(int tile) {
    const int s = tile % NST;
    const int rows = min(C::BN, skv - tile * C::BN);
    const uint32_t bytes = static_cast<uint32_t>(rows) * D;
    sm100::mbar_arrive_expect_tx(bar0 + 8 * s, bytes);
    sm100::bulk_load_1d(smem_u32(codes + s * C::CODE_BYTES), src + static_cast<int64_t>(tile) * C::CODE_BYTES, bytes, bar0 + 8 * s);
  }
  __device__ __forceinline__ float2 load_meta(int tile, int tid) const {
    const int n = tile * C::BN + tid;
    return n < skv ? make_float2(half_bits_to_f32(scale[n]), static_cast<float>(zp[n])) : make_float2(0.f, 0.f);
  }
  // all threads; ends with the stages of the first NST tiles in flight.  The caller's next __syncthreads makes
  // the metadata visible.
  __device__ __forceinline__ void init(uint8_t* base, const ShortQDev& p, const int8_t* kvc, int64_t tok0, int tiles, int tid) {
    codes = base;
    meta = reinterpret_cast<float2*>(base + NST * C::CODE_BYTES);
    uint8_t* bars = base + NST * C::CODE_BYTES + NST * C::BN * 8;
    bar0 = smem_u32(bars);
    abort_flag = reinterpret_cast<volatile int*>(bars + NST * 8);
    src = kvc; scale = p.kv.scale + tok0; zp = p.kv.zp + tok0; skv = p.Skv; n_tiles = tiles;
    epoch = p.epoch;
    pend_slot = -1;
    if (tid == 0) {
      *abort_flag = sm100::launch_aborted(p.epoch) ? 1 : 0;   // a CTA of this launch already gave up: drain quickly
      for (int s = 0; s < NST; ++s) sm100::mbar_init(bar0 + 8 * s, 1);
      sm100::fence_barrier_init();
    }
    __syncthreads();
    for (int tl = 0; tl < NST && tl < n_tiles; ++tl) {
      if (tid == 0) issue(tl);
      if (tid < C::BN) meta[tl * C::BN + tid] = load_meta(tl, tid);
    }
  }
  // dequantize tile `tile` into sKV; false if the wait was abandoned
  template <typename T>
  __device__ __forceinline__ bool commit(uint8_t* sKV, int tile, int tid) const {
    const int s = tile % NST;
    if (!sm100::mbar_wait(bar0 + 8 * s, (tile / NST) & 1, abort_flag, epoch)) return false;
    const uint8_t* cs = codes + s * C::CODE_BYTES;
    const float2* ms = meta + s * C::BN;
#pragma unroll
    for (int i = 0; i < C::CHUNKS; ++i) {
      const int c = tid + i * C::THREADS;
      int r = c / C::CPR, cc = c % C::CPR;
      if constexpr (C::CPR == 8) {
        // Head dim 128: a quarter warp (the unit a 16-byte shared-memory access is split into) takes chunks 0-3 of
        // one row and chunks 4-7 of its neighbour instead of one whole row.  Its loads then cover two different
        // 64-byte halves of the 128-byte code rows, and its stores land 272 + 128 bytes apart in the padded tile,
        // i.e. in the other four 16-byte bank groups: both are conflict-free (a whole 256-byte row per quarter
        // warp hits four bank groups twice on every store).
        const int quad = c >> 2, k = quad & 3;
        r = 2 * (quad >> 2) + (k & 1);
        cc = 4 * (((k >> 1) ^ k) & 1) + (c & 3);
      }
      uint4 v = make_uint4(0, 0, 0, 0);
      float2 m = make_float2(0.f, 0.f);
      if (tile * C::BN + r < skv) {          // rows past the end were not copied: keep them zero
        v = *reinterpret_cast<const uint4*>(cs + r * D + cc * 16);
        m = ms[r];
      }
      dequant16_store<T>(sKV + r * C::T_STRIDE + cc * 32, v, m.y, m.x);
    }
    return true;
  }
  // after the __syncthreads that follows commit(tile): stage and metadata slot of `tile` are free again
  __device__ __forceinline__ void refill(int tile, int tid) {
    if (tid < C::BN && pend_slot >= 0) meta[pend_slot * C::BN + tid] = pend;     // loaded one iteration ago
    pend_slot = -1;
    if (tile + NST < n_tiles) {
      if (tid == 0) issue(tile + NST);
      if (tid < C::BN) { pend = load_meta(tile + NST, tid); pend_slot = tile % NST; }
    }
  }
};

// ------------------------------------------------------------------------------------------------ forward
template <typename T, int D, int MT>
__global__ void __launch_bounds__(128) attn_fwd_shortq_kernel(ShortQDev p) {
  using C = SqCfg<D, MT>;
  using H16 = Half16<T>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sQ = smem + C::Q_OFF;
  uint8_t* sKV = smem + C::KV_OFF_FWD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.x;
  const int b = bh / p.H, h = bh % p.H;
  const int64_t tok0 = static_cast<int64_t>(bh) * p.Skv;
  const int8_t* kvc = p.kv.codes + b * p.kv.stride[0] + h * p.kv.stride[1];

  // Q -> (q * sm_scale) rounded to T (quant_flash_attn.py:52), rows >= Sq are zero
  {
    const T* q = static_cast<const T*>(p.q) + b * p.q_stride[0] + h * p.q_stride[1];
    for (int c = tid; c < C::ROWS * (D / 8); c += C::THREADS) {
      const int r = c / (D / 8), cc = c % (D / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < p.Sq) v = *reinterpret_cast<const uint4*>(q + r * p.q_stride[2] + cc * 8);
      float2 f;
      f = H16::unpack(v.x); v.x = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.y); v.y = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.z); v.z = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      f = H16::unpack(v.w); v.w = H16::pack(f.x * p.sm_scale, f.y * p.sm_scale);
      *reinterpret_cast<uint4*>(sQ + r * C::T_STRIDE + cc * 16) = v;
    }
  }
  KvRing<D, MT, C::NST_FWD> st;
  const int n_tiles = (p.Skv + C::BN - 1) / C::BN;
  st.init(smem + C::RING_OFF_FWD, p, kvc, tok0, n_tiles, tid);
  __syncthreads();
  // Q as MMA left operand, kept in registers for the whole walk (every warp works on all query rows)
  uint32_t qa[MT][D / 16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const uint32_t a_base = smem_u32(sQ + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldsm_x4(a_base + kk * 32, qa[mt][kk][0], qa[mt][kk][1], qa[mt][kk][2], qa[mt][kk][3]);
  }

  float o_acc[MT][D / 8][4];
  float m_run[MT][2], l_run[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o_acc[mt][i][0] = o_acc[mt][i][1] = o_acc[mt][i][2] = o_acc[mt][i][3] = 0.f;
  }
  const int r0 = warp * 16;     // this warp's K/V rows inside the tile
  bool failed = false;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int n0 = tile * C::BN;
    __syncthreads();
    const bool arrived = st.template commit<T>(sKV, tile, tid);
    if (!__syncthreads_and(arrived)) { failed = true; break; }
    st.refill(tile, tid);
    if (n0 + r0 >= p.Skv) continue;       // this warp's 16 tokens are all past the end (warp-uniform)

    // S = Q K^T for 16 tokens: two 8-column MMA tiles
    float s[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[mt][0][e] = s[mt][1][e] = 0.f;
    const uint32_t b_base = smem_u32(sKV + (r0 + (lane & 7) + ((lane >> 4) & 1) * 8) * C::T_STRIDE + ((lane >> 3) & 1) * 16);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(b_base + kk * 32, b0, b1, b2, b3);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_16816<T>(s[mt][0], qa[mt][kk], b0, b1);
        mma_16816<T>(s[mt][1], qa[mt][kk], b2, b3);
      }
    }
    const bool ragged = n0 + r0 + 16 > p.Skv;
    // V as right operand of P.V: the same shared-memory rows, read transposed
    const uint32_t v_base = smem_u32(sKV + (r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float v[4] = {s[mt][0][2 * r] * kLog2e, s[mt][0][2 * r + 1] * kLog2e, s[mt][1][2 * r] * kLog2e,
                      s[mt][1][2 * r + 1] * kLog2e};
        if (ragged) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (n0 + r0 + (e >> 1) * 8 + 2 * t + (e & 1) >= p.Skv) v[e] = -INFINITY;
        }
        float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][r], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = fast_exp2(m_run[mt][r] - m_use);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = fast_exp2(v[e] - m_use);
        l_run[mt][r] = l_run[mt][r] * alpha[r] + (v[0] + v[1] + v[2] + v[3]);
        m_run[mt][r] = m_new;
        s[mt][0][2 * r] = v[0]; s[mt][0][2 * r + 1] = v[1]; s[mt][1][2 * r] = v[2]; s[mt][1][2 * r + 1] = v[3];
      }
      uint32_t a[4];
      a[0] = H16::pack(s[mt][0][0], s[mt][0][1]);
      a[1] = H16::pack(s[mt][0][2], s[mt][0][3]);
      a[2] = H16::pack(s[mt][1][0], s[mt][1][1]);
      a[3] = H16::pack(s[mt][1][2], s[mt][1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_base + dp * 32, b0, b1, b2, b3);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o_acc[mt][2 * dp][e] *= alpha[e >> 1];
          o_acc[mt][2 * dp + 1][e] *= alpha[e >> 1];
        }
        mma_16816<T>(o_acc[mt][2 * dp], a, b0, b1);
        mma_16816<T>(o_acc[mt][2 * dp + 1], a, b2, b3);
      }
    }
  }

  if (failed) {
    if (tid == 0 && p.status) *p.status = QFA_STATUS_WAIT_TIMEOUT;
    return;
  }
  // ---------------- merge the four warps' partial (m, l, O) and write O, LSE (quant_flash_attn.py:77-83)
  __syncthreads();
  float* sO = reinterpret_cast<float*>(smem);                          // [4][ROWS][D]
  float2* sML = reinterpret_cast<float2*>(smem + 4 * C::ROWS * D * 4);  // [4][ROWS] (m, l)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[mt][r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = mt * 16 + g + 8 * r;
      if (t == 0) sML[warp * C::ROWS + row] = make_float2(m_run[mt][r], l);
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(&sO[(warp * C::ROWS + row) * D + i * 8 + 2 * t]) =
            make_float2(o_acc[mt][i][2 * r], o_acc[mt][i][2 * r + 1]);
    }
  __syncthreads();
  T* o = static_cast<T*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1];
  for (int c = tid; c < C::ROWS * (D / 8); c += C::THREADS) {
    const int row = c / (D / 8), cc = (c % (D / 8)) * 8;
    if (row >= p.Sq) continue;
    float2 ml[4];
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) { ml[w] = sML[w * C::ROWS + row]; m = fmaxf(m, ml[w].x); }
    float wgt[4], l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) { wgt[w] = (ml[w].x == -INFINITY) ? 0.f : fast_exp2(ml[w].x - m); l += wgt[w] * ml[w].y; }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float4 x0 = *reinterpret_cast<const float4*>(&sO[(w * C::ROWS + row) * D + cc]);
      const float4 x1 = *reinterpret_cast<const float4*>(&sO[(w * C::ROWS + row) * D + cc + 4]);
      acc[0] += wgt[w] * x0.x; acc[1] += wgt[w] * x0.y; acc[2] += wgt[w] * x0.z; acc[3] += wgt[w] * x0.w;
      acc[4] += wgt[w] * x1.x; acc[5] += wgt[w] * x1.y; acc[6] += wgt[w] * x1.z; acc[7] += wgt[w] * x1.w;
    }
    uint4 out;
    out.x = H16::pack(acc[0] * inv, acc[1] * inv); out.y = H16::pack(acc[2] * inv, acc[3] * inv);
    out.z = H16::pack(acc[4] * inv, acc[5] * inv); out.w = H16::pack(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(o + row * p.o_stride[2] + cc) = out;
    if (cc == 0) p.lse[static_cast<int64_t>(bh) * p.lse_stride + row] = (m + log2f(l)) * kLn2;
  }
}

// ------------------------------------------------------------------------------------------------ backward
// Per 64-token tile and warp (16 tokens): S^T = K^ Q^T, P^T = exp(S^T*sm - LSE), dP^T = V^ dO^T,
// dS^T = P^T*(dP^T - delta), dKV rows = P^T dO + sm * dS^T Q  (written once), dQ += dS K^ (registers).
template <typename T, int D, int MT>
__global__ void __launch_bounds__(128, MT == 1 ? 4 : 1) attn_bwd_shortq_kernel(ShortQDev p) {
  using C = SqCfg<D, MT>;
  using H16 = Half16<T>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* sQ = smem + C::Q_OFF;
  uint8_t* sDO = smem + C::DO_OFF;
  uint8_t* sKV = smem + C::KV_OFF_BWD;
  uint8_t* sDS = smem + C::DS_OFF;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.x;
  const int b = bh / p.H, h = bh % p.H;
  const int64_t tok0 = static_cast<int64_t>(bh) * p.Skv;
  const int8_t* kvc = p.kv.codes + b * p.kv.stride[0] + h * p.kv.stride[1];
  {
    const T* q = static_cast<const T*>(p.q) + b * p.q_stride[0] + h * p.q_stride[1];
    const T* d_o = static_cast<const T*>(p.d_o) + b * p.do_stride[0] + h * p.do_stride[1];
    for (int c = tid; c < C::ROWS * (D / 8); c += C::THREADS) {
      const int r = c / (D / 8), cc = c % (D / 8);
      uint4 vq = make_uint4(0, 0, 0, 0), vd = make_uint4(0, 0, 0, 0);
      if (r < p.Sq) {
        vq = *reinterpret_cast<const uint4*>(q + r * p.q_stride[2] + cc * 8);      // raw q (quant_flash_attn.py:153)
        vd = *reinterpret_cast<const uint4*>(d_o + r * p.do_stride[2] + cc * 8);
      }
      *reinterpret_cast<uint4*>(sQ + r * C::T_STRIDE + cc * 16) = vq;
      *reinterpret_cast<uint4*>(sDO + r * C::T_STRIDE + cc * 16) = vd;
    }
  }
  // per-column (query) constants of this thread's S^T fragment: columns mt*16 + nt*8 + 2t + e
  float lse2[MT][2][2], dlt[MT][2][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int qi = mt * 16 + nt * 8 + 2 * t + e;
        const bool ok = qi < p.Sq;
        lse2[mt][nt][e] = ok ? p.lse_in[static_cast<int64_t>(bh) * p.lse_stride + qi] * kLog2e : INFINITY;
        dlt[mt][nt][e] = ok ? p.delta[static_cast<int64_t>(bh) * p.lse_stride + qi] : 0.f;
      }
  KvRing<D, MT, C::NST_BWD> st;
  const int n_tiles = (p.Skv + C::BN - 1) / C::BN;
  st.init(smem + C::RING_OFF_BWD, p, kvc, tok0, n_tiles, tid);
  bool failed = false;

  float dq_acc[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dq_acc[mt][i][0] = dq_acc[mt][i][1] = dq_acc[mt][i][2] = dq_acc[mt][i][3] = 0.f;
  const int r0 = warp * 16;
  const float sm2 = p.sm_scale * kLog2e;
  T* dkv = static_cast<T*>(p.dkv) + b * p.dkv_stride[0] + h * p.dkv_stride[1];

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int n0 = tile * C::BN;
    __syncthreads();
    const bool arrived = st.template commit<T>(sKV, tile, tid);
    if (!__syncthreads_and(arrived)) { failed = true; break; }
    st.refill(tile, tid);
    if (n0 + r0 >= p.Skv) continue;       // warp-uniform

    // left operand K^ = V^ rows of this warp; right operands Q and dO as (n = query, k = d)
    const uint32_t a_base = smem_u32(sKV + (r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
    const uint32_t bq_base = smem_u32(sQ + ((lane & 7) + ((lane >> 4) & 1) * 8) * C::T_STRIDE + ((lane >> 3) & 1) * 16);
    const uint32_t bd_base = smem_u32(sDO + ((lane & 7) + ((lane >> 4) & 1) * 8) * C::T_STRIDE + ((lane >> 3) & 1) * 16);
    float st_[MT][2][4], dp_[MT][2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) { st_[mt][nt][e] = 0.f; dp_[mt][nt][e] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a_base + kk * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(bq_base + mt * 16 * C::T_STRIDE + kk * 32, b0, b1, b2, b3);
        mma_16816<T>(st_[mt][0], a, b0, b1);
        mma_16816<T>(st_[mt][1], a, b2, b3);
        ldsm_x4(bd_base + mt * 16 * C::T_STRIDE + kk * 32, b0, b1, b2, b3);
        mma_16816<T>(dp_[mt][0], a, b0, b1);
        mma_16816<T>(dp_[mt][1], a, b2, b3);
      }
    }
    // P^T and dS^T (rows = tokens g, g+8 of this warp; columns = queries)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kvrow = n0 + r0 + g + 8 * (e >> 1);
          float pv = fast_exp2(st_[mt][nt][e] * sm2 - lse2[mt][nt][e & 1]);
          if (kvrow >= p.Skv) pv = 0.f;
          st_[mt][nt][e] = pv;
          dp_[mt][nt][e] = pv * (dp_[mt][nt][e] - dlt[mt][nt][e & 1]);
        }
    // dS^T -> shared (left operand of dQ += dS K^ needs it transposed)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        *reinterpret_cast<uint32_t*>(sDS + (r0 + g) * C::DS_STRIDE + (mt * 16 + nt * 8 + 2 * t) * 2) =
            H16::pack(dp_[mt][nt][0], dp_[mt][nt][1]);
        *reinterpret_cast<uint32_t*>(sDS + (r0 + g + 8) * C::DS_STRIDE + (mt * 16 + nt * 8 + 2 * t) * 2) =
            H16::pack(dp_[mt][nt][2], dp_[mt][nt][3]);
      }
    // dKV rows of this warp = P^T dO + sm * dS^T Q  (k = queries).  One 16-column group of D at a time, written
    // out at once: the accumulator of the whole row (D/8 x 4 registers) would cost a resident CTA per SM
    {
      const uint32_t bdo_t = smem_u32(sDO + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
      const uint32_t bq_t = smem_u32(sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
      uint32_t ap[MT][4], ads[MT][4];
      // sm_scale * dS^T as the left operand of the dK product, so that dV and sm*dK share one accumulator
      const float sm = p.sm_scale;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        ap[mt][0] = H16::pack(st_[mt][0][0], st_[mt][0][1]); ap[mt][1] = H16::pack(st_[mt][0][2], st_[mt][0][3]);
        ap[mt][2] = H16::pack(st_[mt][1][0], st_[mt][1][1]); ap[mt][3] = H16::pack(st_[mt][1][2], st_[mt][1][3]);
        ads[mt][0] = H16::pack(sm * dp_[mt][0][0], sm * dp_[mt][0][1]); ads[mt][1] = H16::pack(sm * dp_[mt][0][2], sm * dp_[mt][0][3]);
        ads[mt][2] = H16::pack(sm * dp_[mt][1][0], sm * dp_[mt][1][1]); ads[mt][3] = H16::pack(sm * dp_[mt][1][2], sm * dp_[mt][1][3]);
      }
      const int n_lo = n0 + r0 + g, n_hi = n_lo + 8;
      T* row_lo = dkv + static_cast<int64_t>(n_lo) * p.dkv_stride[2] + 2 * t;
      T* row_hi = dkv + static_cast<int64_t>(n_hi) * p.dkv_stride[2] + 2 * t;
#pragma unroll
      for (int dpp = 0; dpp < D / 16; ++dpp) {
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(bdo_t + mt * 16 * C::T_STRIDE + dpp * 32, b0, b1, b2, b3);
          mma_16816<T>(acc[0], ap[mt], b0, b1);
          mma_16816<T>(acc[1], ap[mt], b2, b3);
          ldsm_x4_t(bq_t + mt * 16 * C::T_STRIDE + dpp * 32, b0, b1, b2, b3);
          mma_16816<T>(acc[0], ads[mt], b0, b1);
          mma_16816<T>(acc[1], ads[mt], b2, b3);
        }
        if (n_lo < p.Skv) {
          *reinterpret_cast<uint32_t*>(row_lo + dpp * 16) = H16::pack(acc[0][0], acc[0][1]);
          *reinterpret_cast<uint32_t*>(row_lo + dpp * 16 + 8) = H16::pack(acc[1][0], acc[1][1]);
        }
        if (n_hi < p.Skv) {
          *reinterpret_cast<uint32_t*>(row_hi + dpp * 16) = H16::pack(acc[0][2], acc[0][3]);
          *reinterpret_cast<uint32_t*>(row_hi + dpp * 16 + 8) = H16::pack(acc[1][2], acc[1][3]);
        }
      }
    }
    __syncwarp();
    // dQ += dS K^ over this warp's 16 tokens: A = dS (from dS^T, transposing load), B = K^ (transposing load)
    {
      const uint32_t a_t = smem_u32(sDS + (r0 + (lane & 7) + ((lane >> 4) & 1) * 8) * C::DS_STRIDE + ((lane >> 3) & 1) * 16);
      const uint32_t b_t = smem_u32(sKV + (r0 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::T_STRIDE + ((lane >> 4) & 1) * 16);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        ldsm_x4_t(a_t + mt * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int dpp = 0; dpp < D / 16; ++dpp) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(b_t + dpp * 32, b0, b1, b2, b3);
          mma_16816<T>(dq_acc[mt][2 * dpp], a, b0, b1);
          mma_16816<T>(dq_acc[mt][2 * dpp + 1], a, b2, b3);
        }
      }
    }
  }

  if (failed) {
    if (tid == 0 && p.status) *p.status = QFA_STATUS_WAIT_TIMEOUT;
    return;
  }
  // ---------------- dQ = sm_scale * sum over the four warps (quant_flash_attn.py:164-166)
  __syncthreads();
  float* sD = reinterpret_cast<float*>(smem);      // [4][ROWS][D]
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = mt * 16 + g + 8 * r;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<float2*>(&sD[(warp * C::ROWS + row) * D + i * 8 + 2 * t]) =
            make_float2(dq_acc[mt][i][2 * r], dq_acc[mt][i][2 * r + 1]);
    }
  __syncthreads();
  T* dq = static_cast<T*>(p.dq) + b * p.dq_stride[0] + h * p.dq_stride[1];
  for (int c = tid; c < C::ROWS * (D / 8); c += C::THREADS) {
    const int row = c / (D / 8), cc = (c % (D / 8)) * 8;
    if (row >= p.Sq) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float4 x0 = *reinterpret_cast<const float4*>(&sD[(w * C::ROWS + row) * D + cc]);
      const float4 x1 = *reinterpret_cast<const float4*>(&sD[(w * C::ROWS + row) * D + cc + 4]);
      acc[0] += x0.x; acc[1] += x0.y; acc[2] += x0.z; acc[3] += x0.w;
      acc[4] += x1.x; acc[5] += x1.y; acc[6] += x1.z; acc[7] += x1.w;
    }
    uint4 out;
    out.x = H16::pack(acc[0] * p.sm_scale, acc[1] * p.sm_scale); out.y = H16::pack(acc[2] * p.sm_scale, acc[3] * p.sm_scale);
    out.z = H16::pack(acc[4] * p.sm_scale, acc[5] * p.sm_scale); out.w = H16::pack(acc[6] * p.sm_scale, acc[7] * p.sm_scale);
    *reinterpret_cast<uint4*>(dq + row * p.dq_stride[2] + cc) = out;
  }
}

// ------------------------------------------------------------------------------------------------ host
template <typename K>
static int set_smem(K kern, int bytes, DeviceOnce& done) {
  return once_per_device(done, [&]() -> int {
    QFA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return QFA_OK;
  });
}

template <typename T, int D, int MT>
static int launch_fwd_sq(const ShortQDev& d, int64_t heads, cudaStream_t stream) {
  using C = SqCfg<D, MT>;
  static DeviceOnce done;
  int rc = set_smem(attn_fwd_shortq_kernel<T, D, MT>, C::SMEM_FWD, done);
  if (rc) return rc;
  attn_fwd_shortq_kernel<T, D, MT><<<static_cast<unsigned>(heads), C::THREADS, C::SMEM_FWD, stream>>>(d);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}
template <typename T, int D, int MT>
static int launch_bwd_sq(const ShortQDev& d, int64_t heads, cudaStream_t stream) {
  using C = SqCfg<D, MT>;
  static DeviceOnce done;
  int rc = set_smem(attn_bwd_shortq_kernel<T, D, MT>, C::SMEM_BWD, done);
  if (rc) return rc;
  attn_bwd_shortq_kernel<T, D, MT><<<static_cast<unsigned>(heads), C::THREADS, C::SMEM_BWD, stream>>>(d);
  note_launch();
  QFA_CUDA_TRY(cudaGetLastError());
  return QFA_OK;
}

static bool same_tensor(const QfaQuantTensor& a, const QfaQuantTensor& b) {
  return a.codes == b.codes && a.scale == b.scale && a.zp == b.zp && a.stride[0] == b.stride[0] &&
         a.stride[1] == b.stride[1] && a.stride[2] == b.stride[2];
}

// the code tiles travel as untiled bulk copies: the rows of a head must be contiguous and 16-byte aligned
static bool bulk_copyable(const QfaQuantTensor& t, int64_t D) {
  return t.stride[2] == D && (reinterpret_cast<uintptr_t>(t.codes) & 15) == 0 && t.stride[0] % 16 == 0 && t.stride[1] % 16 == 0;
}
int attn_fwd_shortq_supported(const QfaFwdArgs& a) {
  return a.mode == QFA_MODE_REF && !a.causal && a.Sq <= 32 && same_tensor(a.k, a.v) && (a.D == 64 || a.D == 128) &&
         a.B * a.H <= 0x7fffffffLL && bulk_copyable(a.k, a.D);
}
int attn_bwd_shortq_supported(const QfaBwdArgs& a) {
  return a.mode == QFA_MODE_REF && !a.causal && a.dkv_fused && a.Sq <= 32 && same_tensor(a.k, a.v) &&
         (a.D == 64 || a.D == 128) && a.B * a.H <= 0x7fffffffLL && bulk_copyable(a.k, a.D);
}

#define QFA_SQ_DISPATCH(FN, dev, heads, stream)                                                            \
  do {                                                                                                     \
    const bool bf = dtype == QFA_BF16;                                                                     \
    if (D == 64) {                                                                                         \
      if (mt == 1) return bf ? FN<__nv_bfloat16, 64, 1>(dev, heads, stream) : FN<__half, 64, 1>(dev, heads, stream);   \
      return bf ? FN<__nv_bfloat16, 64, 2>(dev, heads, stream) : FN<__half, 64, 2>(dev, heads, stream);    \
    }                                                                                                      \
    if (mt == 1) return bf ? FN<__nv_bfloat16, 128, 1>(dev, heads, stream) : FN<__half, 128, 1>(dev, heads, stream);   \
    return bf ? FN<__nv_bfloat16, 128, 2>(dev, heads, stream) : FN<__half, 128, 2>(dev, heads, stream);    \
  } while (0)

int attn_fwd_shortq_entry(const QfaFwdArgs& a, cudaStream_t stream) {
  ShortQDev d = {};
  d.q = a.q;
  for (int i = 0; i < 3; ++i) { d.q_stride[i] = a.q_stride[i]; d.o_stride[i] = a.o_stride[i]; }
  d.kv = a.k; d.o = a.o; d.lse = a.lse; d.lse_stride = a.lse_stride;
  d.H = static_cast<int>(a.H); d.Sq = static_cast<int>(a.Sq); d.Skv = static_cast<int>(a.Skv); d.sm_scale = a.sm_scale;
  d.status = a.status;
  d.epoch = next_launch_epoch();
  const int dtype = a.dtype, mt = a.Sq <= 16 ? 1 : 2;
  const int64_t D = a.D, heads = a.B * a.H;
  QFA_SQ_DISPATCH(launch_fwd_sq, d, heads, stream);
}

int attn_bwd_shortq_entry(const QfaBwdArgs& a, cudaStream_t stream) {
  ShortQDev d = {};
  d.q = a.q;
  for (int i = 0; i < 3; ++i) {
    d.q_stride[i] = a.q_stride[i]; d.do_stride[i] = a.do_stride[i];
    d.dq_stride[i] = a.dq_stride[i]; d.dkv_stride[i] = a.dk_stride[i];
  }
  d.kv = a.k; d.d_o = a.d_o; d.lse_in = a.lse; d.delta = a.delta; d.lse_stride = a.lse_stride;
  d.dq = a.dq; d.dkv = a.dk;
  d.H = static_cast<int>(a.H); d.Sq = static_cast<int>(a.Sq); d.Skv = static_cast<int>(a.Skv); d.sm_scale = a.sm_scale;
  d.status = a.status;
  d.epoch = next_launch_epoch();
  const int dtype = a.dtype, mt = a.Sq <= 16 ? 1 : 2;
  const int64_t D = a.D, heads = a.B * a.H;
  QFA_SQ_DISPATCH(launch_bwd_sq, d, heads, stream);
}

}  // namespace qfa
