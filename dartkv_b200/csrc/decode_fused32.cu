// Tensor-core fused decode attention with the arithmetic of the reference's Triton attention kernels
// (src/dart/fused_attention.py:149-262): key = code * scale + zero and value = code * scale + zero in
// fp32 with no rounding to the cache dtype, fp32 logits, fp32 online softmax.  Same page geometry, work
// split and staging as decode_fast.cu (which reproduces the per-op rounded dequantization instead).
//
// Because nothing is rounded per element, the affine map leaves the inner loop:
//   logit[t,h]  = sum_ch (q[h,ch] * s[ch]) * code[t,ch]  +  sum_ch q[h,ch] * z[ch]
//   out[h,ch]   = sum_t  (p[t,h] * s[t,grp]) * code[t,ch] +  sum_t  p[t,h] * z[t,grp]
// The packed 2-bit codes become MMA operands with ONE logic op per register: `word & mask` leaves a
// code in mantissa bits 2p..2p+1 of each 16-bit half with a zero exponent, which read as fp16 is the
// subnormal code * 4^p * 2^-24 -- exact, and the tensor cores take subnormal fp16 operands at full
// accuracy.  The power of two is constant per accumulator row (a row always reads the same code
// position), so it is folded into the fp32 scaling that follows the MMA.  The other operand carries
// the weights q*s (per page) and p*s (per token) as fp16 after an exact power-of-two normalisation
// chosen from the largest scale in sight, so no input magnitude overflows or underflows the format.
// The zero-point terms are plain fp32 dot products.  A promoted channel's code is low + 4 * high: its
// high plane is just more contraction steps with weight 4 * q * s.
//
// As in decode_fast.cu a 32-bit register of codes pairs two elements along the MMA's non-contraction
// direction, so the contraction index is doubled, (channel, j) for K and (token, j) for V, against a
// block-diagonal weight operand whose columns are (query head, j').  For V the pair is arranged as
// (channel of value group 0, channel of value group 1), which lets one operand carry both groups'
// scales.  Algorithmic HBM bytes per page and (batch, kv head): 10880.

#include <atomic>

#include "decode_fast_common.cuh"

namespace {

#ifndef FUSED_QK_UNROLL
#define FUSED_QK_UNROLL 16
#endif
#ifndef FUSED_PV_UNROLL
#define FUSED_PV_UNROLL 4
#endif

constexpr int kQkUnroll = FUSED_QK_UNROLL, kPvUnroll = FUSED_PV_UNROLL;
constexpr int kUStride = 36;   // 32-bit words per group of 8 local tokens in a warp's weight table (4 pad)

struct FusedPairSmem {
  uint8_t stage[2][kStageBytes];
  // per-page tables, double-buffered like the stages so that one warp of the pair may set up the next page while
  // the other still reads this page's
  uint2 w_low[2][128];           // per channel: fp16 q*s*f of heads (0,1) and (2,3)
  uint2 w_high[2][32];           // per promoted slot: fp16 4*q*s*f of its channel, zero past the last slot
  uint2 w_high_lo[2][32];        // what the fp16 rounding of w_high dropped, as fp16: the high plane carries most of a
                                 // promoted (outlier) channel's magnitude, so its weights get a second term
  uint32_t u[2][8 * kUStride];   // per warp: [local token][head] = fp16 p*s*fv of (value group 0 | group 1 << 16)
  float bias_part[2][2][4];      // [table][warp]: partial sum_ch q*z per head
  uint64_t bar[2];
};

struct FusedBlockSmem {
  float qf[128][4];              // [channel][head] query as fp32 (zero for absent heads)
  float merge_m[kWarps][4];
  float merge_l[kWarps][4];
  int slot_map[128];
  float q_absmax;
};

template <int DT>
__device__ __forceinline__ float md_to_float(uint32_t bits16) {
  if (DT == DARTKV_BF16) return __uint_as_float(bits16 << 16);
  return __half2float(__ushort_as_half((uint16_t)bits16));
}
// both halves of a packed pair of 16-bit floats
template <int DT>
__device__ __forceinline__ void md_pair_to_float(uint32_t pair, float& lo, float& hi) {
  if (DT == DARTKV_BF16) {
    lo = __uint_as_float(pair << 16);
    hi = __uint_as_float(pair & 0xFFFF0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pair));
    lo = f.x;
    hi = f.y;
  }
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// Power of two f with bound * f < 2^15 (so bound * f fits fp16), and 1/f; bound >= 0 finite.
__device__ __forceinline__ void pow2_normaliser(float bound, float& f, float& f_inv) {
  int eb = (int)(__float_as_uint(bound) >> 23);   // bound < 2^(eb - 126)
  eb = min(max(eb, 15), 253);
  f = __uint_as_float((uint32_t)(268 - eb) << 23);       // 2^(141 - eb)
  f_inv = __uint_as_float((uint32_t)(eb - 14) << 23);    // 2^(eb - 141)
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// per-warp running state of the online softmax and the output accumulators
struct WarpState {
  float o_acc[4][4];   // [m-tile][c-reg], in units of 4^p * 2^-24 / fv_run
  float m_run, l_run;  // head c, log2 domain
  float zs[2];         // this thread's share of sum_t p * z for (head c, value group j)
  float fv_run, fv_inv_run;
};

// One warp's share of a staged page.  HF: which four codes of every 16-bit half this warp owns;
// GN: value groups per token (1 or 2).
template <int DT, int GN>
__device__ __forceinline__ void fused_page_half(const int HF, const int tb, const dartkv_cache_desc& d, FusedPairSmem& ps, const uint8_t* blob,
                                                uint32_t* utab, int prom_steps, float scale2, float f_inv, int g, int c,
                                                uint32_t sel_w, uint32_t mask_u, int mask_below, WarpState& st) {
  // ---- logits: S[token pair][(head, j')] over the doubled contraction (channel, j).  Row g of m-tile mt
  // reads code position 2mt, row g+8 position 2mt+1.
  // Even and odd contraction steps use separate accumulators so consecutive MMAs are independent.
  float s_acc[2][4], s_odd[2][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s_acc[mt][i] = s_odd[mt][i] = 0.0f;
  {
    const uint8_t* low_thread = blob + 4 * g + 32 * c;                               // + 256 * step (+128)
    const uint8_t* w_thread = reinterpret_cast<const uint8_t*>(ps.w_low[tb]) + 8 * c + 4 * (g >> 2);   // + 64 * step (+32)
#ifndef FUSED_SKIP_QK
#pragma unroll kQkUnroll
    for (int ks = 0; ks < 16; ++ks) {
      uint32_t w0 = *reinterpret_cast<const uint32_t*>(low_thread + 256 * ks);
      uint32_t w1 = *reinterpret_cast<const uint32_t*>(low_thread + 256 * ks + 128);
      w0 >>= 8 * HF; w1 >>= 8 * HF;   // HF is a run-time value: one copy of this code serves both warps of a pair
      const uint32_t b0 = prmt(*reinterpret_cast<const uint32_t*>(w_thread + 64 * ks), 0u, sel_w);
      const uint32_t b1 = prmt(*reinterpret_cast<const uint32_t*>(w_thread + 64 * ks + 32), 0u, sel_w);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        mma_f16((ks & 1) ? s_odd[mt] : s_acc[mt], w0 & (0x00030003u << (4 * mt)), w0 & (0x000C000Cu << (4 * mt)),
                w1 & (0x00030003u << (4 * mt)), w1 & (0x000C000Cu << (4 * mt)), b0, b1);
    }
    // high plane of the promoted slots
    const uint8_t* high_thread = blob + d.key_off_high + 4 * g + 32 * c;
    const uint8_t* wh_thread = reinterpret_cast<const uint8_t*>(ps.w_high[tb]) + 8 * c + 4 * (g >> 2);
    const uint8_t* wl_thread = reinterpret_cast<const uint8_t*>(ps.w_high_lo[tb]) + 8 * c + 4 * (g >> 2);
    for (int ks = 0; ks < prom_steps; ++ks) {
      uint32_t w0 = *reinterpret_cast<const uint32_t*>(high_thread + 256 * ks);
      uint32_t w1 = *reinterpret_cast<const uint32_t*>(high_thread + 256 * ks + 128);
      w0 >>= 8 * HF; w1 >>= 8 * HF;   // HF is a run-time value: one copy of this code serves both warps of a pair
      const uint32_t b0 = prmt(*reinterpret_cast<const uint32_t*>(wh_thread + 64 * ks), 0u, sel_w);
      const uint32_t b1 = prmt(*reinterpret_cast<const uint32_t*>(wh_thread + 64 * ks + 32), 0u, sel_w);
      const uint32_t l0 = prmt(*reinterpret_cast<const uint32_t*>(wl_thread + 64 * ks), 0u, sel_w);
      const uint32_t l1 = prmt(*reinterpret_cast<const uint32_t*>(wl_thread + 64 * ks + 32), 0u, sel_w);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const uint32_t a0 = w0 & (0x00030003u << (4 * mt)), a1 = w0 & (0x000C000Cu << (4 * mt));
        const uint32_t a2 = w1 & (0x00030003u << (4 * mt)), a3 = w1 & (0x000C000Cu << (4 * mt));
        mma_f16(s_acc[mt], a0, a1, a2, a3, b0, b1);
        mma_f16(s_odd[mt], a0, a1, a2, a3, l0, l1);   // same codes against the dropped part of the weights
      }
    }
#endif
  }

  // ---- online softmax for head c over this warp's 64 tokens (this thread: 8 of them)
  const float bias = (ps.bias_part[tb][0][c] + ps.bias_part[tb][1][c]) * scale2;
  float cm[4];   // scale2 / f * 2^(24 - 2p)
  {
    const float base = scale2 * f_inv;
    cm[0] = base * 16777216.0f; cm[1] = base * 4194304.0f; cm[2] = base * 1048576.0f; cm[3] = base * 262144.0f;
  }
  float mx = -INFINITY;
  float s_sum[2][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s_sum[mt][i] = fmaf(s_acc[mt][i] + s_odd[mt][i], cm[2 * mt + (i >> 1)], bias);
    }
  if (mask_below > 0) {   // the page that holds the row's first live token: the tokens before it drop out
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (16 * g + 4 * HF + 2 * mt + (i >> 1) + 8 * (i & 1) < mask_below) s_sum[mt][i] = -INFINITY;
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = fmaxf(mx, s_sum[mt][i]);
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
  const float m_new = fmaxf(st.m_run, mx);
  const float m_ref = m_new == -INFINITY ? 0.0f : m_new;   // nothing live yet: every weight below comes out zero
  const float alpha = fast_exp2(st.m_run - m_ref);
  st.m_run = m_new;

  // value metadata of this thread's 8 tokens: token = 16g + 4HF + p + 8j', p = 2mt + (i >> 1), j' = i & 1
  const uint8_t* vmeta = blob + kOffVMeta;
  uint32_t meta_s[8], meta_z[8];   // GN == 2: (s0 | s1 << 16), (z0 | z1 << 16); GN == 1: s, z in the low half
  uint32_t smax = 0;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int tok = 16 * g + 4 * HF + 2 * mt + (i >> 1) + 8 * (i & 1);
      const int k = 4 * mt + i;
      if (GN == 2) {
        const uint2 m = *reinterpret_cast<const uint2*>(vmeta + tok * 8);
        meta_s[k] = m.x; meta_z[k] = m.y;
        smax = max(smax, max(m.x & 0xFFFFu, m.x >> 16));
      } else {
        const uint32_t m = *reinterpret_cast<const uint32_t*>(vmeta + tok * 4);
        meta_s[k] = m & 0xFFFFu; meta_z[k] = m >> 16;
        smax = max(smax, m & 0xFFFFu);
      }
    }
  // scales are positive finite 16-bit floats: their bit patterns order like the values
  smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, 4));
  smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, 8));
  smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, 16));
  float fv_page, fv_inv_page;
  pow2_normaliser(md_to_float<DT>(smax), fv_page, fv_inv_page);
  // the normaliser only ever shrinks, so accumulators are rescaled at most a handful of times per run
  const bool shrink = fv_page < st.fv_run;
  const float factor = shrink ? alpha * (fv_page * st.fv_inv_run) : alpha;
  if (shrink) { st.fv_run = fv_page; st.fv_inv_run = fv_inv_page; }
  const float fv = st.fv_run;

  float psum = 0.0f, zs0 = 0.0f, zs1 = 0.0f;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = 4 * mt + i;
      const float p = fast_exp2(s_sum[mt][i] - m_ref);
      psum += p;
      const float pf = p * fv;
      const int li = 2 * mt + (i >> 1) + 4 * (i & 1);   // local token inside this thread's 8: position + 4 j'
      uint32_t packed;
      if (GN == 2) {
        float s0, s1, z0, z1;
        md_pair_to_float<DT>(meta_s[k], s0, s1);
        md_pair_to_float<DT>(meta_z[k], z0, z1);
        zs0 = fmaf(p, z0, zs0);
        zs1 = fmaf(p, z1, zs1);
        packed = pack_f16x2(pf * s0, pf * s1);
      } else {
        const float s0 = md_to_float<DT>(meta_s[k]), z0 = md_to_float<DT>(meta_z[k]);
        zs0 = fmaf(p, z0, zs0);
        const float u = pf * s0;
        packed = pack_f16x2(u, u);
      }
      utab[g * kUStride + li * 4 + c] = packed;
    }
  st.l_run = st.l_run * alpha + psum;
  st.zs[0] = st.zs[0] * alpha + zs0;
  st.zs[1] = st.zs[1] * alpha + (GN == 2 ? zs1 : zs0);
  // the running maximum and the normaliser rarely move after the first pages
  if (__any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) st.o_acc[mt][i] *= factor;
  }
  __syncwarp();

  // ---- O[channel pair][(head, j')] += V^T U over the doubled contraction (token, j): lane row g reads the
  // code words wi = g & 3 and wi + 4 of a token row and pairs their low (g < 4) or high (g >= 4) halves, so a
  // register holds (channel 16wi + 8xy + u of group 0, the same channel + 64 of group 1).  Step ks covers the
  // eight tokens 16ks + 4HF + {0..3} and + 8.
  {
    const int wi = g & 3;
    const uint32_t sel_v = (g >> 2) ? 0x7632u : 0x5410u;
    const uint8_t* vthread = blob + kOffVCodes + 32 * (4 * HF + c) + 4 * wi;   // + 512 * ks (+256 for the second token)
    const uint32_t* uthread = utab + c * 4 + (g >> 1);                         // + kUStride * ks (+16 for the second)
#ifndef FUSED_SKIP_PV
#pragma unroll kPvUnroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t x0 = prmt(*reinterpret_cast<const uint32_t*>(vthread + 512 * ks),
                               *reinterpret_cast<const uint32_t*>(vthread + 512 * ks + 16), sel_v);
      const uint32_t x1 = prmt(*reinterpret_cast<const uint32_t*>(vthread + 512 * ks + 256),
                               *reinterpret_cast<const uint32_t*>(vthread + 512 * ks + 256 + 16), sel_v);
      const uint32_t y0 = x0 >> 10, y1 = x1 >> 10;   // codes 5, 6, 7 at positions 0, 1, 2
      const uint32_t b0 = uthread[kUStride * ks] & mask_u;
      const uint32_t b1 = uthread[kUStride * ks + 16] & mask_u;
      mma_f16(st.o_acc[0], x0 & 0x00030003u, x0 & 0x000C000Cu, x1 & 0x00030003u, x1 & 0x000C000Cu, b0, b1);
      mma_f16(st.o_acc[1], x0 & 0x00300030u, x0 & 0x00C000C0u, x1 & 0x00300030u, x1 & 0x00C000C0u, b0, b1);
      mma_f16(st.o_acc[2], x0 & 0x03000300u, y0 & 0x00030003u, x1 & 0x03000300u, y1 & 0x00030003u, b0, b1);
      mma_f16(st.o_acc[3], y0 & 0x000C000Cu, y0 & 0x00300030u, y1 & 0x000C000Cu, y1 & 0x00300030u, b0, b1);
    }
#endif
  }
}

// GN: value groups per token (1 or 2).  KP: promoted channels per page when that is a multiple of eight known to
// the host (0, 8, 16, 24, 32), else -1 (read from the descriptor).
// DT: dtype of the cache and the query; MD: dtype of the scales and zero points
template <int DT, int MD, int GN, int KP>
__global__ void __launch_bounds__(kThreads, 2) decode_fused32_kernel(dartkv_cache_desc d, FastArgs a) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  FusedPairSmem* psm_all = reinterpret_cast<FusedPairSmem*>(smem_raw);
  FusedBlockSmem& bs = *reinterpret_cast<FusedBlockSmem*>(smem_raw + sizeof(FusedPairSmem) * kPairs);
  float* warp_out = reinterpret_cast<float*>(smem_raw);   // reused after the page loop: [warp][head][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rep = a.query_heads / d.kv_heads;

  if ((int)blockIdx.x >= a.stream_blocks) {
    // dense tokens of one (batch, kv head): partial slot 0.  These short blocks come last in launch order and fill
    // the slots the stream blocks leave.
    const int bh = blockIdx.x - a.stream_blocks;
    dense_block<DT, MD>(d, a, bs, warp_out, bh);
    __syncthreads();
    block_merge(a, bs, warp_out, bh / d.kv_heads, bh % d.kv_heads, rep, 0);
    return;
  }

  // ---- stream block: an even share of all (row, four-page unit) work, possibly spanning several rows
  const int sb = blockIdx.x;
  int unit = (int)((int64_t)sb * a.units / a.stream_blocks);   // the host keeps the unit count below 2^31
  const int unit_end = (int)((int64_t)(sb + 1) * a.units / a.stream_blocks);
  const int pair = warp >> 1, hf = warp & 1;
  FusedPairSmem& ps = psm_all[pair];
  const int k_end = d.state[2], v_end = d.state[3], sink_filled = d.state[4];
  const int fast_end = fast_range_end(d.sink_tokens, d.page_size, k_end, v_end, sink_filled);
  const int total_pages = fast_end > d.sink_tokens ? (fast_end - d.sink_tokens) / 128 : 0;
  const bool issuer = hf == 0 && lane == 0;
  const int vmeta_page_bytes = 128 * 2 * d.value_groups * 2;
  const uint32_t stage_tx = d.key_page_bytes + kValueCodes + vmeta_page_bytes;
  int bh = 0;
  auto issue = [&](int pg, int stage) {
    // one lane starts the three bulk copies of a page; the barrier completes when all bytes landed
    mbar_expect_tx(&ps.bar[stage], stage_tx);
    const int64_t vrow = (int64_t)bh * d.max_value_tokens + (int64_t)pg * 128;
    bulk_copy_g2s(ps.stage[stage], d.k_pages + ((int64_t)bh * d.max_key_pages + pg) * d.key_page_bytes, d.key_page_bytes, &ps.bar[stage]);
    bulk_copy_g2s(ps.stage[stage] + kOffVCodes, d.v_codes + vrow * 32, kValueCodes, &ps.bar[stage]);
    bulk_copy_g2s(ps.stage[stage] + kOffVMeta,
                  reinterpret_cast<const uint8_t*>(d.v_meta) + vrow * (2 * d.value_groups * 2), vmeta_page_bytes, &ps.bar[stage]);
  };
  if (issuer) {
    mbar_init(&ps.bar[0], 1);
    mbar_init(&ps.bar[1], 1);
    mbar_fence_init();
  }
  __syncthreads();
  const int K = KP >= 0 ? KP : (d.key_mode == DARTKV_MIXED_PAGE ? d.promoted : 0);
  const int prom_steps = (K + 7) >> 3;
  const float scale2 = a.scale * kLog2e;
  // weight operand: column n = g is (head g >> 1, j' = g & 1); the 32-bit word read holds the fp16 weights of the
  // head pair g >> 2.  Take the head's half into half j' and zeros (from the second source) into the other.
  const uint32_t head_bytes = ((g >> 1) & 1) ? 0x32u : 0x10u;
  const uint32_t sel_w = (g & 1) ? (0x0054u | (head_bytes << 8)) : (head_bytes | 0x5400u);
  const uint32_t mask_u = (g & 1) ? 0xFFFF0000u : 0x0000FFFFu;
  uint32_t* utab = ps.u[hf];
  bool ok = true;
  int iter = 0;   // pages this pair has consumed so far: stage and barrier parity carry over from row to row

  while (unit < unit_end) {
    bh = unit / a.quads;
    const int quad_begin = unit - bh * a.quads;
    const int quad_count = min(a.quads - quad_begin, unit_end - unit);
    unit += quad_count;
    // tokens before the row's first live one get no weight: whole pages of them are not even fetched
    const int row_first = a.row_start ? max(a.row_start[bh / d.kv_heads], 0) : 0;
    const int p_begin = max(4 * quad_begin, row_first > d.sink_tokens ? (row_first - d.sink_tokens) >> 7 : 0);
    const int p_end = min(4 * (quad_begin + quad_count), total_pages);

    // the first two pages of this pair are requested before anything else, so their latency overlaps the
    // query load below
    const int pg0 = p_begin + pair;
    if (issuer) {
      if (pg0 < p_end) issue(pg0, iter & 1);
      if (pg0 + kPairs < p_end) issue(pg0 + kPairs, (iter + 1) & 1);
    }

    // query as fp32 and its largest magnitude (bounds the page weights q*s)
    {
      const int b = bh / d.kv_heads, hkv = bh % d.kv_heads;
      float amax = 0.0f;
      for (int i = tid; i < 4 * 128; i += kThreads) {
        const int r = i >> 7, ch = i & 127;
        float v = 0.0f;
        if (r < rep)
          v = md_to_float<DT>(reinterpret_cast<const uint16_t*>(a.q)[((int64_t)b * a.query_heads + hkv * rep + r) * 128 + ch]);
        bs.qf[ch][r] = v;
        amax = fmaxf(amax, fabsf(v));
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      if (lane == 0) bs.merge_m[warp][0] = amax;   // scratch use before the merge
    }
    __syncthreads();
    if (tid == 0) {
      float amax = 0.0f;
      for (int w = 0; w < kWarps; ++w) amax = fmaxf(amax, bs.merge_m[w][0]);
      bs.q_absmax = amax;
    }
    __syncthreads();
    const float q_absmax = bs.q_absmax;

    WarpState st;
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) st.o_acc[mt][i] = 0.0f;
    st.m_run = -INFINITY; st.l_run = 0.0f; st.zs[0] = st.zs[1] = 0.0f;
    st.fv_run = __uint_as_float(253u << 23); st.fv_inv_run = __uint_as_float(1u << 23);
    for (int pg = pg0; pg < p_end; pg += kPairs, ++iter) {
      const int stage = iter & 1;
      const uint32_t parity = (iter >> 1) & 1;
      ok = mbar_wait(&ps.bar[stage], parity) && ok;
      const uint8_t* blob = ps.stage[stage];

      // ---- per-page setup by the 64 threads of the pair: thread tp owns channels 2tp, 2tp+1
      float f = 1.0f, f_inv = 1.0f;
#ifndef FUSED_SKIP_SETUP
      {
        const uint32_t* kscale2 = reinterpret_cast<const uint32_t*>(blob + d.key_off_scale);
        const uint32_t* kzero2 = reinterpret_cast<const uint32_t*>(blob + d.key_off_zero);
        // largest key scale of the page (every warp computes it for itself: no exchange needed)
        const uint2 sc4 = reinterpret_cast<const uint2*>(kscale2)[lane];   // channels 4*lane .. 4*lane+3
        uint32_t smax = max(max(sc4.x & 0xFFFFu, sc4.x >> 16), max(sc4.y & 0xFFFFu, sc4.y >> 16));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, off));
        pow2_normaliser(4.0f * q_absmax * md_to_float<MD>(smax), f, f_inv);

        const int tp = 32 * hf + lane;
        float s0, s1, z0, z1;
        md_pair_to_float<MD>(kscale2[tp], s0, s1);
        md_pair_to_float<MD>(kzero2[tp], z0, z1);
        const float4 qa = *reinterpret_cast<const float4*>(bs.qf[2 * tp]);
        const float4 qb = *reinterpret_cast<const float4*>(bs.qf[2 * tp + 1]);
        const float sa = s0 * f, sb = s1 * f;
        ps.w_low[stage][2 * tp] = make_uint2(pack_f16x2(qa.x * sa, qa.y * sa), pack_f16x2(qa.z * sa, qa.w * sa));
        ps.w_low[stage][2 * tp + 1] = make_uint2(pack_f16x2(qb.x * sb, qb.y * sb), pack_f16x2(qb.z * sb, qb.w * sb));
        // sum_ch q*z per head, reduced over the warp
        float bz[4] = {fmaf(qa.x, z0, qb.x * z1), fmaf(qa.y, z0, qb.y * z1), fmaf(qa.z, z0, qb.z * z1), fmaf(qa.w, z0, qb.w * z1)};
        // four sums over 32 lanes in 6 shuffles: halve the number of sums a lane carries at the first two levels
        {
          const bool up16 = lane & 16, up8 = lane & 8;
          const float k0 = (up16 ? bz[2] : bz[0]) + __shfl_xor_sync(0xffffffffu, up16 ? bz[0] : bz[2], 16);
          const float k1 = (up16 ? bz[3] : bz[1]) + __shfl_xor_sync(0xffffffffu, up16 ? bz[1] : bz[3], 16);
          float k = (up8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, up8 ? k0 : k1, 8);   // head 2*up16 + up8
          k += __shfl_xor_sync(0xffffffffu, k, 4);
          k += __shfl_xor_sync(0xffffffffu, k, 2);
          k += __shfl_xor_sync(0xffffffffu, k, 1);
          if ((lane & 7) == 0) ps.bias_part[stage][hf][lane >> 3] = k;
        }
        // promoted slots: warp 1 of the pair, lane = slot
        if (hf == 1 && prom_steps > 0) {
          uint2 wh = make_uint2(0u, 0u), wl = make_uint2(0u, 0u);
          if (lane < K) {
            const int ch = reinterpret_cast<const int32_t*>(blob + d.key_off_index)[lane] & 127;
            const float s4 = 4.0f * f * md_to_float<MD>(reinterpret_cast<const uint16_t*>(blob + d.key_off_scale)[ch]);
            const float4 qh = *reinterpret_cast<const float4*>(bs.qf[ch]);
            const float e0 = qh.x * s4, e1 = qh.y * s4, e2 = qh.z * s4, e3 = qh.w * s4;
            wh = make_uint2(pack_f16x2(e0, e1), pack_f16x2(e2, e3));
            const float2 h01 = __half22float2(*reinterpret_cast<const __half2*>(&wh.x));
            const float2 h23 = __half22float2(*reinterpret_cast<const __half2*>(&wh.y));
            wl = make_uint2(pack_f16x2(e0 - h01.x, e1 - h01.y), pack_f16x2(e2 - h23.x, e3 - h23.y));
          }
          ps.w_high[stage][lane] = wh;
          ps.w_high_lo[stage][lane] = wl;
        }
      }
#endif
      // the only meeting point of the pair per page: the tables of this page are complete and both warps are done
      // with the page before, whose stage can take the page after this one
      pair_barrier(pair);
      if (issuer && pg != pg0 && pg + kPairs < p_end) issue(pg + kPairs, stage ^ 1);

      fused_page_half<MD, GN>(hf, stage, d, ps, blob, utab, prom_steps, scale2, f_inv, g, c, sel_w, mask_u,
                              row_first - (d.sink_tokens + 128 * pg), st);

    }

    // ---- hand the warp state to the block merge: sums over the lanes that share head c
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      st.l_run += __shfl_xor_sync(0xffffffffu, st.l_run, off);
      st.zs[0] += __shfl_xor_sync(0xffffffffu, st.zs[0], off);
      st.zs[1] += __shfl_xor_sync(0xffffffffu, st.zs[1], off);
    }
    __syncthreads();   // every warp is done with its stages: the staging memory becomes the merge buffer
    if (g == 0) { bs.merge_m[warp][c] = st.m_run; bs.merge_l[warp][c] = st.l_run; }
    {
      const int wi = g & 3, xy = g >> 2;
      const float unit = st.fv_inv_run * 16777216.0f;   // accumulators hold codes * 4^p * 2^-24 * fv
      const float pos_scale[5] = {unit, unit * 0.25f, unit * 0.0625f, unit * 0.015625f, unit * 0.00390625f};
#pragma unroll
      for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int u = 2 * mt + (i >> 1), jp = i & 1;
          const int p = u < 5 ? u : u - 5;
          const int ch = 64 * jp + 16 * wi + 8 * xy + u;
          warp_out[(warp * 4 + c) * 128 + ch] = fmaf(st.o_acc[mt][i], pos_scale[p], st.zs[jp]);
        }
    }
    __syncthreads();
    block_merge(a, bs, warp_out, bh / d.kv_heads, bh % d.kv_heads, rep,
                1 + sb - dartkv_block_of_unit((int64_t)bh * a.quads, a.stream_blocks, a.units));
    __syncthreads();   // the merge buffer is staging memory again, the query table may be overwritten
  }
  if (!ok && lane == 0) atomicExch(a.status, 1);
}

constexpr size_t kFusedSmemBytes = sizeof(FusedPairSmem) * kPairs + sizeof(FusedBlockSmem);

}  // namespace

int dartkv_decode_fused32_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads) {
  if (d->head_dim != 128 || d->page_size != 128 || d->key_group != 128 || !d->regular_pages) return 0;
  if (d->dtype != DARTKV_F16 && d->dtype != DARTKV_BF16) return 0;
  if ((d->md_dtype != DARTKV_F16 && d->md_dtype != DARTKV_BF16) || q_dtype != d->dtype) return 0;
  if (d->value_bits != 2 || (d->value_group != 64 && d->value_group != 128)) return 0;
  if (d->key_mode == DARTKV_QUANTIZED_PAGE && d->key_bits != 2) return 0;
  if (d->key_page_bytes % 16 || d->key_page_bytes > kPageBytesK) return 0;   // at most 32 promoted channels
  if (query_heads % d->kv_heads || query_heads / d->kv_heads > 4) return 0;
  if (d->max_value_tokens % 8) return 0;   // keeps every page of value metadata 16-byte aligned
  if ((uintptr_t)d->k_pages % 16 || (uintptr_t)d->v_codes % 16 || (uintptr_t)d->v_meta % 16) return 0;
  return 1;
}

// every (cache dtype, metadata dtype, value groups, promoted count) variant of the kernel; a cache whose metadata
// dtype differs from its dtype gets the promoted counts 0 and 32 specialized, the others read the count at run time
using FusedKernel = void (*)(dartkv_cache_desc, FastArgs);
template <int DT, int GN>
static FusedKernel fused_variant_kp(int kp) {
  switch (kp) {
    case 0: return decode_fused32_kernel<DT, DT, GN, 0>;
    case 8: return decode_fused32_kernel<DT, DT, GN, 8>;
    case 16: return decode_fused32_kernel<DT, DT, GN, 16>;
    case 24: return decode_fused32_kernel<DT, DT, GN, 24>;
    case 32: return decode_fused32_kernel<DT, DT, GN, 32>;
    default: return decode_fused32_kernel<DT, DT, GN, -1>;
  }
}
template <int DT, int MD, int GN>
static FusedKernel fused_mixed_kp(int kp) {
  switch (kp) {
    case 0: return decode_fused32_kernel<DT, MD, GN, 0>;
    case 32: return decode_fused32_kernel<DT, MD, GN, 32>;
    default: return decode_fused32_kernel<DT, MD, GN, -1>;
  }
}
static FusedKernel fused_variant(int dtype, int md, int value_groups, int kp) {
  if (md == dtype) {
    if (dtype == DARTKV_BF16) return value_groups == 2 ? fused_variant_kp<DARTKV_BF16, 2>(kp) : fused_variant_kp<DARTKV_BF16, 1>(kp);
    return value_groups == 2 ? fused_variant_kp<DARTKV_F16, 2>(kp) : fused_variant_kp<DARTKV_F16, 1>(kp);
  }
  if (dtype == DARTKV_BF16)
    return value_groups == 2 ? fused_mixed_kp<DARTKV_BF16, DARTKV_F16, 2>(kp) : fused_mixed_kp<DARTKV_BF16, DARTKV_F16, 1>(kp);
  return value_groups == 2 ? fused_mixed_kp<DARTKV_F16, DARTKV_BF16, 2>(kp) : fused_mixed_kp<DARTKV_F16, DARTKV_BF16, 1>(kp);
}

int dartkv_decode_fused32_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
                                 int flavour, int quads, int stream_blocks, long long units, int total_splits,
                                 float* part_m, float* part_l, float* part_acc, int* status, const int32_t* row_start,
                                 cudaStream_t stream) {
  (void)q_dtype;
  FastArgs a{query, query_heads, scale, flavour, quads, stream_blocks, units, total_splits, part_m, part_l, part_acc, status,
             row_start};
  dim3 grid(stream_blocks + d->batch * d->kv_heads);
  {
    // the shared-memory opt-in is per device and per kernel: ask once per device (the flags are atomic; two threads
    // that race on a device's first call both set the attribute, which is harmless)
    static std::atomic<bool> ready[64];
    int device = 0;
    DARTKV_CUDA_OK(cudaGetDevice(&device));
    if (device < 0 || device >= 64 || !ready[device].load(std::memory_order_acquire)) {
      for (int dt : {DARTKV_BF16, DARTKV_F16})
        for (int md : {DARTKV_BF16, DARTKV_F16})
          for (int gn : {1, 2})
            for (int kp : {-1, 0, 8, 16, 24, 32})
              DARTKV_CUDA_OK(cudaFuncSetAttribute(fused_variant(dt, md, gn, kp), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)kFusedSmemBytes));
      if (device >= 0 && device < 64) ready[device].store(true, std::memory_order_release);
    }
  }
  const int promoted = d->key_mode == DARTKV_MIXED_PAGE ? d->promoted : 0;
  const int kp = (promoted % 8 == 0 && promoted <= 32) ? promoted : -1;
  fused_variant(d->dtype, d->md_dtype, d->value_groups, kp)<<<grid, kThreads, kFusedSmemBytes, stream>>>(*d, a);
  DARTKV_LAUNCH_OK("decode_fused32_kernel");
  return DARTKV_OK;
}
