// Tensor-core fused decode attention for the common page geometry: head_dim 128, 128-token pages,
// one 128-token key group, 2-bit values with 64/128-channel groups, 2-bit keys (uniform or with up to
// 32 promoted 2+2-bit channels), 16-bit data whose metadata has the same dtype, up to 4 query heads
// per KV head.  Everything else takes the generic kernel in decode_attention.cu.
//
// Work split: one unit = four consecutive pages of a (batch, kv head) row.  The units of all rows are dealt out
// evenly to the stream blocks (aligned to rows, or one block per resident slot whose share may run from one
// row into the next; the host chooses).  A block of 8 warps (4 warp pairs) hands page p of its run to pair
// p % 4.  A pair streams its pages through a two-stage shared-memory ring filled by 1-D bulk async copies
// (one key blob of up to 5760 bytes, 4096 bytes of value codes and up to 1024 bytes of value metadata per
// page, completion on an mbarrier).  For the logits the two warps of a pair split the CONTRACTION (alternate
// steps of eight channels each, whole 32-bit code words per thread) and swap half of their partial sums through
// shared memory; for the softmax and P.V they split the page's TOKENS (codes 0-3 / 4-7 of every packed 16-bit
// half, i.e. 64 tokens each) and keep private online-softmax states.  They meet at two named barriers per page;
// the block merges all eight states when it leaves a row and writes one partial per row it touched.  One more short block per row, launched after the stream blocks, handles the
// dense tokens: the sink prefix and everything after the last page that is packed on both the key and the
// value side.
//
// Per page a warp never materializes K or V: packed 2-bit codes are turned into exactly rounded
// 16-bit operands with one logic op and two packed fma/add per pair (mma_utils.cuh) and fed straight
// into m16n8k16 MMAs.  Keys: a register of the operand pairs two tokens of one channel (they share the
// channel's scale and zero point), which is the MMA's non-contraction direction, so the contraction index is
// doubled, k = (channel, j), against a block-diagonal query operand whose columns are (query head, j).
// Values: the code words of two tokens are byte-interleaved so that a register pairs two TOKENS of one
// channel, the contraction direction itself; each half of the packed arithmetic carries its own token's scale
// and zero point, the probability operand is plain (p[a], p[b]), and its eight columns hold the high and the
// low 16-bit parts of the four heads' probabilities, so one MMA accumulates both.
// Algorithmic HBM bytes per page and (batch, kv head): 10880.

#include <atomic>

#include "decode_fast_common.cuh"

namespace {

// timing experiments only (a library built with these computes garbage)
#if defined(PEROP_SKIP_MMA)
#define PEROP_MMA(acc, a0, a1, a2, a3, b0, b1) ((acc)[0] += __uint_as_float((a0) ^ (a1) ^ (a2) ^ (a3) ^ (b0) ^ (b1)))
#else
#define PEROP_MMA(acc, a0, a1, a2, a3, b0, b1) HO::mma(acc, a0, a1, a2, a3, b0, b1)
#endif

#ifndef PEROP_QK_UNROLL
#define PEROP_QK_UNROLL 8
#endif
#ifndef PEROP_PV_UNROLL
#define PEROP_PV_UNROLL 4
#endif
constexpr int kQkUnroll = PEROP_QK_UNROLL, kPvUnroll = PEROP_PV_UNROLL;

struct PairSmem {
  uint8_t stage[2][kStageBytes];
  uint4 kpar_a[128];      // by contraction position: (s,s) (z,z) -magic0*s -magic1*s of that position's channel
  uint2 kpar_b[128];      // by contraction position: -magic2*s, byte offset of the channel's row (32 * channel)
  uint16_t prob[2][2 * 4 * kPStride];  // per warp of the pair: [hi/lo][head][local token]
  uint8_t order[2][128];  // per warp: contraction order of the channels, promoted slots first
  uint8_t is_promoted[2][128];
  uint64_t bar[2];
};

struct BlockSmem {
  uint32_t q32[128][8];      // [channel][2*head + j']: query pre-shifted into the low (j'=0) or high (j'=1) half
  float merge_m[kWarps][4];
  float merge_l[kWarps][4];
  int slot_map[128];
};

// the dequantized registers of a code word, from the metadata dtype to the cache dtype (nothing when they agree)
template <int DT, int OUT>
__device__ __forceinline__ void cast_registers(uint32_t (&r)[8]) {
  if (DT != OUT) {
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = cast16<DT, OUT>(r[i]);
  }
}

// One warp's share of a staged page: QK over its 64 tokens, online softmax, PV over the same tokens.
// DT = metadata dtype (the arithmetic of the dequantization), OUT = cache dtype (the MMA operands): when they differ
// every dequantized register is cast, as the reference casts its dequantized pages (src/dart/quantization.py:103-106).
// GN = value groups per token (1 or 2).
template <int DT, int OUT, int GN, int KP>
__device__ __forceinline__ void page_half(const int HF, const int pair, const int lane, const dartkv_cache_desc& d, PairSmem& ps,
                                          const uint8_t* blob, uint16_t* prob, uint16_t* partner_prob, const uint8_t* q_thread, const CodeConsts<DT>& cc, int K, int prom_steps,
                                          float scale2, int g, int c, int jp, int hq, int gv, int mask_below,
                                          float (&o_acc)[8][4],
                                          float& m_run, float& l_run) {
  using H = Half2Ops<DT>;
  using HO = Half2Ops<OUT>;
  const uint8_t* low_thread = blob + 4 * g;   // + 32 * channel = this thread's word of the channel row
  const uint32_t* high = reinterpret_cast<const uint32_t*>(blob + d.key_off_high);

  // ---- logits.  The two warps of a pair split the CONTRACTION: warp HF takes the steps of eight positions
  // 2i + HF, i = 0..7 (the promoted slots come first in the order, so both warps get their share of them), and
  // computes partial logits of all 128 tokens: S[token pair][(head, j')] over the doubled contraction
  // (channel, j).  A thread reads the whole 32-bit word g of a channel row (tokens 16g .. 16g+15): register u
  // pairs tokens 16g+u and 16g+u+8, m-tile mt takes registers 2mt (row g) and 2mt+1 (row g+8).
  float s_acc[4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s_acc[mt][i] = 0.0f;
#if !defined(PEROP_SKIP_QK)
  const int my_prom_steps = (prom_steps + 1 - HF) >> 1;   // promoted steps with the parity of this warp
  for (int i = 0; i < my_prom_steps; ++i) {
    const int s0 = 8 * (2 * i + HF) + c, s1 = s0 + 4;
    const uint4 a0 = ps.kpar_a[s0], a1 = ps.kpar_a[s1];
    const uint2 o0 = ps.kpar_b[s0], o1 = ps.kpar_b[s1];
    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(low_thread + o0.y);
    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(low_thread + o1.y);
    // with a promoted count that is a multiple of eight every position of a promoted step is a promoted slot
    const uint32_t h0 = (KP >= 0 || s0 < K) ? high[s0 * 8 + g] : 0u;
    const uint32_t h1 = (KP >= 0 || s1 < K) ? high[s1 * 8 + g] : 0u;
    uint32_t r0[8], r1[8];
    dequant_word4<DT>(cc, w0, h0, a0.x, a0.y, a0.z, a0.w, r0);
    dequant_word4<DT>(cc, w1, h1, a1.x, a1.y, a1.z, a1.w, r1);
    cast_registers<DT, OUT>(r0);
    cast_registers<DT, OUT>(r1);
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(q_thread + o0.y);
    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(q_thread + o1.y);
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) PEROP_MMA(s_acc[mt], r0[2 * mt], r0[2 * mt + 1], r1[2 * mt], r1[2 * mt + 1], b0, b1);
  }
#pragma unroll kQkUnroll
  for (int i = my_prom_steps; i < 8; ++i) {
    const int s0 = 8 * (2 * i + HF) + c, s1 = s0 + 4;
#if defined(PEROP_SKIP_KPAR)
    const uint4 a0 = make_uint4(cc.mask[0], cc.mask[1], cc.magic[0], cc.magic[1]), a1 = a0;
    const uint2 o0 = make_uint2(cc.magic[2], 32u * s0), o1 = make_uint2(cc.magic[2], 32u * s1);
#else
    const uint4 a0 = ps.kpar_a[s0], a1 = ps.kpar_a[s1];
    const uint2 o0 = ps.kpar_b[s0], o1 = ps.kpar_b[s1];
#endif
    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(low_thread + o0.y);
    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(low_thread + o1.y);
    uint32_t r0[8], r1[8];
    dequant_word2<DT>(cc, w0, a0.x, a0.y, a0.z, a0.w, o0.x, r0);
    dequant_word2<DT>(cc, w1, a1.x, a1.y, a1.z, a1.w, o1.x, r1);
    cast_registers<DT, OUT>(r0);
    cast_registers<DT, OUT>(r1);
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(q_thread + o0.y);
    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(q_thread + o1.y);
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) PEROP_MMA(s_acc[mt], r0[2 * mt], r0[2 * mt + 1], r1[2 * mt], r1[2 * mt + 1], b0, b1);
  }
#endif   // PEROP_SKIP_QK

  // ---- exchange: this warp goes on with the tokens of m-tiles 2HF and 2HF+1 (codes 4HF .. 4HF+3 of every packed
  // half-word), so it hands its partial logits of the other two m-tiles to its partner and takes the partner's
  // partials of its own.  The message travels through the receiver's probability table, which is idle here: both
  // warps left the previous page's P.V behind at the barrier that ended that page.
  float s_sum[2][4];
  {
    float4* to_partner = reinterpret_cast<float4*>(partner_prob);
    const float4* from_partner = reinterpret_cast<const float4*>(prob);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      float4 v;
      v.x = HF ? s_acc[mt][0] : s_acc[2 + mt][0]; v.y = HF ? s_acc[mt][1] : s_acc[2 + mt][1];
      v.z = HF ? s_acc[mt][2] : s_acc[2 + mt][2]; v.w = HF ? s_acc[mt][3] : s_acc[2 + mt][3];
      to_partner[mt * 32 + lane] = v;
    }
    pair_barrier(pair);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const float4 v = from_partner[mt * 32 + lane];
      s_sum[mt][0] = ((HF ? s_acc[2 + mt][0] : s_acc[mt][0]) + v.x) * scale2;
      s_sum[mt][1] = ((HF ? s_acc[2 + mt][1] : s_acc[mt][1]) + v.y) * scale2;
      s_sum[mt][2] = ((HF ? s_acc[2 + mt][2] : s_acc[mt][2]) + v.z) * scale2;
      s_sum[mt][3] = ((HF ? s_acc[2 + mt][3] : s_acc[mt][3]) + v.w) * scale2;
    }
    __syncwarp();   // every lane has read its message before any lane writes probabilities over it
  }
  if (mask_below > 0) {   // the page that holds the row's first live token: the tokens before it drop out
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (16 * g + 4 * HF + 2 * mt + (i >> 1) + 8 * (i & 1) < mask_below) s_sum[mt][i] = -INFINITY;
  }

  // ---- online softmax for head c over this warp's 64 tokens (this thread: 8 of them)
  float mx = -INFINITY;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = fmaxf(mx, s_sum[mt][i]);
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
  const float m_new = fmaxf(m_run, mx);
  const float m_ref = m_new == -INFINITY ? 0.0f : m_new;   // nothing live yet: every weight below comes out zero
  const float alpha = fast_exp2(m_run - m_ref);
  m_run = m_new;
  float psum = 0.0f;
  uint16_t phi[8], plo[8];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p = fast_exp2(s_sum[mt][i] - m_ref);
      psum += p;
      const int li = 4 * mt + i;   // table order inside this thread's 8 tokens: token offset (li >> 1) + 8 * (li & 1)
      const uint16_t hi = HO::from_float(p);
      phi[li] = hi;
      plo[li] = HO::from_float(p - HO::to_float(hi));
    }
  l_run = l_run * alpha + psum;
  // the running maximum rarely moves after the first pages: skip the rescale when no lane needs it.  This thread's
  // accumulator columns belong to heads 2(c&1) and 2(c&1)+1, whose factors live in the lanes c' = head of its quad.
  if (__any_sync(0xffffffffu, alpha != 1.0f)) {
    const float alpha_even = __shfl_sync(0xffffffffu, alpha, (lane & ~3) | (2 * (c & 1)));
    const float alpha_odd = __shfl_sync(0xffffffffu, alpha, (lane & ~3) | (2 * (c & 1) + 1));
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      o_acc[mt][0] *= alpha_even; o_acc[mt][1] *= alpha_odd;
      o_acc[mt][2] *= alpha_even; o_acc[mt][3] *= alpha_odd;
    }
  }
  {
    uint4 hv, lv;
    hv.x = (uint32_t)phi[0] | ((uint32_t)phi[1] << 16); hv.y = (uint32_t)phi[2] | ((uint32_t)phi[3] << 16);
    hv.z = (uint32_t)phi[4] | ((uint32_t)phi[5] << 16); hv.w = (uint32_t)phi[6] | ((uint32_t)phi[7] << 16);
    lv.x = (uint32_t)plo[0] | ((uint32_t)plo[1] << 16); lv.y = (uint32_t)plo[2] | ((uint32_t)plo[3] << 16);
    lv.z = (uint32_t)plo[4] | ((uint32_t)plo[5] << 16); lv.w = (uint32_t)plo[6] | ((uint32_t)plo[7] << 16);
    *reinterpret_cast<uint4*>(&prob[(0 * 4 + c) * kPStride + 8 * g]) = hv;
    *reinterpret_cast<uint4*>(&prob[(1 * 4 + c) * kPStride + 8 * g]) = lv;
  }
  __syncwarp();

  // ---- O[channel][(part, head)] += V^T P over this warp's 64 tokens, 16 per step.  A register of the value
  // operand pairs two TOKENS of one channel (the contraction direction): the code words of the two tokens are
  // byte-interleaved first (low halves together: channels 0..7 of both tokens; high halves: channels 8..15), so that
  // the packed dequantization sees token a in the low half and token b in the high half, each with its own scale
  // and zero point.  The probability operand then is just (p[a], p[b]), and its eight columns carry the high and
  // the low parts of the four heads side by side, so one MMA does both.  Local token L of this warp (the order of
  // the probability table) is page token 16*(L>>3) + 4*HF + ((L&7)>>1) + 8*(L&1); m-tile mt, row g is channel
  // 16g + mt, row g+8 channel 16g + 8 + mt.
  const uint32_t* vcodes = reinterpret_cast<const uint32_t*>(blob + kOffVCodes) + g;   // word g of a token row: + 8 * token
  const uint8_t* vmeta = blob + kOffVMeta;
  const uint32_t* pb = reinterpret_cast<const uint32_t*>(&prob[((g >> 2) * 4 + (g & 3)) * kPStride]) + c;   // column n = g
  const int tok_a = 4 * HF + c;   // page token of local token 2c; local token 2c + 1 is page token tok_a + 8
  // byte selectors that bring the scale (zero point) of this thread's value group of tokens a and b together
  const uint32_t sel_s = GN == 2 ? (gv ? 0x7632u : 0x5410u) : 0x5410u;
  const uint32_t sel_z = GN == 2 ? (gv ? 0x7632u : 0x5410u) : 0x7632u;
  auto token_pair = [&](int ta, uint32_t (&r_lo)[8], uint32_t (&r_hi)[8]) {
    const uint32_t wa = vcodes[ta * 8], wb = vcodes[ta * 8 + 64];
    uint32_t ss, zz;
    if (GN == 2) {
      const uint2 ma = *reinterpret_cast<const uint2*>(vmeta + ta * 8);        // {s0,s1} {z0,z1}
      const uint2 mb = *reinterpret_cast<const uint2*>(vmeta + ta * 8 + 64);
      ss = prmt(ma.x, mb.x, sel_s);
      zz = prmt(ma.y, mb.y, sel_z);
    } else {
      const uint32_t ma = *reinterpret_cast<const uint32_t*>(vmeta + ta * 4);   // {s0, z0}
      const uint32_t mb = *reinterpret_cast<const uint32_t*>(vmeta + ta * 4 + 32);
      ss = prmt(ma, mb, sel_s);
      zz = prmt(ma, mb, sel_z);
    }
    const uint32_t ms0 = H::mul(ss, H::neg_magic(0)), ms1 = H::mul(ss, H::neg_magic(1)), ms2 = H::mul(ss, H::neg_magic(2));
    dequant_word2<DT>(cc, prmt(wa, wb, 0x5410u), ss, zz, ms0, ms1, ms2, r_lo);
    dequant_word2<DT>(cc, prmt(wa, wb, 0x7632u), ss, zz, ms0, ms1, ms2, r_hi);
    cast_registers<DT, OUT>(r_lo);
    cast_registers<DT, OUT>(r_hi);
  };
#if !defined(PEROP_SKIP_PV)
#pragma unroll kPvUnroll
  for (int s = 0; s < 4; ++s) {
    uint32_t r0_lo[8], r0_hi[8], r1_lo[8], r1_hi[8];
    token_pair(32 * s + tok_a, r0_lo, r0_hi);          // local tokens 16s + 2c, 16s + 2c + 1: page tokens a, a + 8
    token_pair(32 * s + tok_a + 16, r1_lo, r1_hi);     // local tokens 16s + 2c + 8, 16s + 2c + 9: a + 16, a + 24
    const uint32_t b0 = pb[8 * s], b1 = pb[8 * s + 4];
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) PEROP_MMA(o_acc[mt], r0_lo[mt], r0_hi[mt], r1_lo[mt], r1_hi[mt], b0, b1);
  }
#endif   // PEROP_SKIP_PV
}

// GN: value groups per token (1 or 2).  KP: promoted channels per page when that is a multiple of eight known to
// the host (0, 8, 16, 24, 32), else -1 (read from the descriptor): with the count fixed the logits loops have
// constant trip counts and no per-position "is this slot promoted" test.
template <int DT, int OUT, int GN, int KP>
__global__ void __launch_bounds__(kThreads, 2) decode_fast_kernel(dartkv_cache_desc d, FastArgs a) {
  using H = Half2Ops<DT>;
  using HO = Half2Ops<OUT>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  PairSmem* psm_all = reinterpret_cast<PairSmem*>(smem_raw);
  BlockSmem& bs = *reinterpret_cast<BlockSmem*>(smem_raw + sizeof(PairSmem) * kPairs);
  float* warp_out = reinterpret_cast<float*>(smem_raw);   // reused after the page loop: [warp][head][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rep = a.query_heads / d.kv_heads;

  if ((int)blockIdx.x >= a.stream_blocks) {
    // dense tokens of one (batch, kv head): partial slot 0.  These short blocks come last in launch order and fill
    // the slots the stream blocks leave.
    const int bh = blockIdx.x - a.stream_blocks;
    dense_block<OUT, DT>(d, a, bs, warp_out, bh);
    __syncthreads();
    block_merge(a, bs, warp_out, bh / d.kv_heads, bh % d.kv_heads, rep, 0);
    return;
  }

  // ---- stream block: an even share of all (row, four-page unit) work, possibly spanning several rows
  const int sb = blockIdx.x;
  int unit = (int)((int64_t)sb * a.units / a.stream_blocks);   // the host keeps the unit count below 2^31
  const int unit_end = (int)((int64_t)(sb + 1) * a.units / a.stream_blocks);
  const int pair = warp >> 1, hf = warp & 1;
  PairSmem& ps = psm_all[pair];
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
  const int jp = g & 1, hq = g >> 1;
  const uint8_t* q_thread = reinterpret_cast<const uint8_t*>(&bs.q32[0][g]);   // + 32 * channel
  const float scale2 = a.scale * kLog2e;
  const int gv = (16 * g) / d.value_group;
  bool ok = true;
  CodeConsts<DT> cc;
  cc.init();
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

    // query, pre-shifted for the block-diagonal operand
    const int b = bh / d.kv_heads, hkv = bh % d.kv_heads;
    for (int i = tid; i < 4 * 128; i += kThreads) {
      const int r = i >> 7, ch = i & 127;
      uint32_t v = 0;
      if (r < rep) v = reinterpret_cast<const uint16_t*>(a.q)[((int64_t)b * a.query_heads + hkv * rep + r) * 128 + ch];
      bs.q32[ch][2 * r] = v;
      bs.q32[ch][2 * r + 1] = v << 16;
    }
    __syncthreads();

    float o_acc[8][4];   // [m-tile][c-reg]: channel 16g + mt + 8(i>>1), head 2(c&1) + (i&1), high (c<2) or low part of P
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) o_acc[mt][i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;   // head c, log2 domain
    for (int pg = pg0; pg < p_end; pg += kPairs, ++iter) {
      const int stage = iter & 1;
      const uint32_t parity = (iter >> 1) & 1;
      ok = mbar_wait(&ps.bar[stage], parity) && ok;
      const uint8_t* blob = ps.stage[stage];
      const uint16_t* kscale = reinterpret_cast<const uint16_t*>(blob + d.key_off_scale);
      const uint16_t* kzero = reinterpret_cast<const uint16_t*>(blob + d.key_off_zero);

      // ---- per-page setup: each warp orders the channels (promoted slots first) into its own copy, then
      // fills the per-position constants of the contraction steps it owns (steps 2i + hf); nothing of this is
      // shared with the other warp of the pair
#if !defined(PEROP_SKIP_SETUP)
      {
        uint8_t* order = ps.order[hf];
        uint8_t* flag = ps.is_promoted[hf];
        reinterpret_cast<uint32_t*>(flag)[lane] = 0;
        __syncwarp();
        if (K > 0) {
          const int32_t* idx = reinterpret_cast<const int32_t*>(blob + d.key_off_index);
          for (int k = lane; k < K; k += 32) {
            const int ch = idx[k] & 127;
            flag[ch] = 1;
            order[k] = (uint8_t)ch;
          }
        }
        __syncwarp();
        const uint32_t flags = reinterpret_cast<const uint32_t*>(flag)[lane];   // channels 4*lane .. +3
        const int mine = 4 - __popc(flags & 0x01010101u);
        int before = mine;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          int up = __shfl_up_sync(0xffffffffu, before, off);
          if (lane >= off) before += up;
        }
        int pos = K + before - mine;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (!((flags >> (8 * i)) & 1u)) order[pos++] = (uint8_t)(4 * lane + i);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int f = lane + 32 * i;                        // 64 positions of this warp
          const int p = 8 * (2 * (f >> 3) + hf) + (f & 7);
          const int ch = order[p];
          const uint32_t ss = (uint32_t)kscale[ch] * 0x00010001u;
          const uint32_t zz = (uint32_t)kzero[ch] * 0x00010001u;
          ps.kpar_a[p] = make_uint4(ss, zz, H::mul(ss, H::neg_magic(0)), H::mul(ss, H::neg_magic(1)));
          ps.kpar_b[p] = make_uint2(H::mul(ss, H::neg_magic(2)), 32u * ch);
        }
      }
#endif
      __syncwarp();

      page_half<DT, OUT, GN, KP>(hf, pair, lane, d, ps, blob, ps.prob[hf], ps.prob[hf ^ 1], q_thread, cc, K, prom_steps, scale2, g, c, jp,
                            hq, gv, row_first - (d.sink_tokens + 128 * pg), o_acc, m_run, l_run);

      pair_barrier(pair);
      // the stage is free again: prefetch the page two iterations ahead
      if (issuer && pg + 2 * kPairs < p_end) issue(pg + 2 * kPairs, stage);
    }

    // ---- hand the warp state to the block merge
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
    __syncthreads();   // every warp is done with its stages: the staging memory becomes the merge buffer
    if (g == 0) { bs.merge_m[warp][c] = m_run; bs.merge_l[warp][c] = l_run; }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // lanes c and c ^ 2 hold what the high and the low parts of the probabilities contributed
        const float v = o_acc[mt][i] + __shfl_xor_sync(0xffffffffu, o_acc[mt][i], 2);
        if (c < 2) warp_out[(warp * 4 + 2 * c + (i & 1)) * 128 + 16 * g + mt + 8 * (i >> 1)] = v;
      }
    __syncthreads();
    block_merge(a, bs, warp_out, bh / d.kv_heads, bh % d.kv_heads, rep,
                1 + sb - dartkv_block_of_unit((int64_t)bh * a.quads, a.stream_blocks, a.units));
    __syncthreads();   // the merge buffer is staging memory again, the query table may be overwritten
  }
  if (!ok && lane == 0) atomicExch(a.status, 1);
}

constexpr size_t kSmemBytes = sizeof(PairSmem) * kPairs + sizeof(BlockSmem);

}  // namespace

int dartkv_decode_fast_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads) {
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

// every (metadata dtype, cache dtype, value groups, promoted count) variant of the kernel; a cache whose metadata
// dtype differs from its dtype gets the promoted counts 0 and 32 specialized, the others read the count at run time
using FastKernel = void (*)(dartkv_cache_desc, FastArgs);
template <int DT, int GN>
static FastKernel fast_variant_kp(int kp) {
  switch (kp) {
    case 0: return decode_fast_kernel<DT, DT, GN, 0>;
    case 8: return decode_fast_kernel<DT, DT, GN, 8>;
    case 16: return decode_fast_kernel<DT, DT, GN, 16>;
    case 24: return decode_fast_kernel<DT, DT, GN, 24>;
    case 32: return decode_fast_kernel<DT, DT, GN, 32>;
    default: return decode_fast_kernel<DT, DT, GN, -1>;
  }
}
template <int DT, int OUT, int GN>
static FastKernel mixed_variant_kp(int kp) {
  switch (kp) {
    case 0: return decode_fast_kernel<DT, OUT, GN, 0>;
    case 32: return decode_fast_kernel<DT, OUT, GN, 32>;
    default: return decode_fast_kernel<DT, OUT, GN, -1>;
  }
}
static FastKernel fast_variant(int md, int dtype, int value_groups, int kp) {
  if (md == dtype) {
    if (dtype == DARTKV_BF16) return value_groups == 2 ? fast_variant_kp<DARTKV_BF16, 2>(kp) : fast_variant_kp<DARTKV_BF16, 1>(kp);
    return value_groups == 2 ? fast_variant_kp<DARTKV_F16, 2>(kp) : fast_variant_kp<DARTKV_F16, 1>(kp);
  }
  if (md == DARTKV_F16)
    return value_groups == 2 ? mixed_variant_kp<DARTKV_F16, DARTKV_BF16, 2>(kp) : mixed_variant_kp<DARTKV_F16, DARTKV_BF16, 1>(kp);
  return value_groups == 2 ? mixed_variant_kp<DARTKV_BF16, DARTKV_F16, 2>(kp) : mixed_variant_kp<DARTKV_BF16, DARTKV_F16, 1>(kp);
}
static void launch_variant(int md, int dtype, int value_groups, int kp, dim3 grid, cudaStream_t stream,
                           const dartkv_cache_desc& d, const FastArgs& a) {
  fast_variant(md, dtype, value_groups, kp)<<<grid, kThreads, kSmemBytes, stream>>>(d, a);
}

int dartkv_decode_fast_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
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
      for (int md : {DARTKV_BF16, DARTKV_F16})
        for (int dt : {DARTKV_BF16, DARTKV_F16})
          for (int gn : {1, 2})
            for (int kp : {-1, 0, 8, 16, 24, 32})
              DARTKV_CUDA_OK(cudaFuncSetAttribute(fast_variant(md, dt, gn, kp), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)kSmemBytes));
      if (device >= 0 && device < 64) ready[device].store(true, std::memory_order_release);
    }
  }
  const int promoted = d->key_mode == DARTKV_MIXED_PAGE ? d->promoted : 0;
  const int kp = (promoted % 8 == 0 && promoted <= 32) ? promoted : -1;
  launch_variant(d->md_dtype, d->dtype, d->value_groups, kp, grid, stream, *d, a);
  DARTKV_LAUNCH_OK("decode_fast_kernel");
  return DARTKV_OK;
}
