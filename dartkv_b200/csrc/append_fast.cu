// Page-shaped quantize+pack kernels for the common geometry: head_dim 128, 16-bit data,
// full 128-token key pages with one 128-token key group, value groups of 32/64/128 channels.
//
// Keys (one block of 64 threads per (batch*head, page)): the page is staged in shared memory
// with 16-byte async copies; thread p owns the channel pair (2p, 2p+1), which moves through both
// passes as one packed 16-bit pair: a pass for min / max / sum|k|, a block-wide rank for the
// promoted channels, a pass that emits the codes and packs them in registers, then 16-byte row
// stores.  Values: eight lanes per token row (16 channels per lane), group min/max by
// xor-shuffles, packed bytes and metadata written coalesced.
// HBM traffic per page: 64 KiB read (K and V rows), 10.6 KiB written (2-bit, 32 promoted).
// The arithmetic is the reference's per-op rounding in the data dtype
// (src/dart/quantization.py:178-186, src/dart/mixed.py:200-209).

#include "common.cuh"

namespace {

constexpr int kD = 128;
constexpr int kP = 128;

struct RowSource {
  const void* chunk;
  const void* ring;
  int64_t sb, sh, st;
  int chunk_start, ring_tokens, kv_heads;
  // base pointers for one (batch, head): chunk rows then ring rows
  __device__ __forceinline__ void bases(int bh, const uint16_t*& chunk_base, const uint16_t*& ring_base) const {
    int b = bh / kv_heads, h = bh % kv_heads;
    chunk_base = reinterpret_cast<const uint16_t*>(chunk) + (int64_t)b * sb + (int64_t)h * sh;
    ring_base = reinterpret_cast<const uint16_t*>(ring) + (int64_t)bh * ring_tokens * kD;
  }
  __device__ __forceinline__ const uint16_t* row_from(const uint16_t* chunk_base, const uint16_t* ring_base, int t) const {
    if (t >= chunk_start) return chunk_base + (int64_t)(t - chunk_start) * st;
    return ring_base + (t % ring_tokens) * kD;
  }
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

// range / qmax rounded to the data dtype.  For bf16 the quotient of two 8-bit significands is never within
// 2^-17 of a rounding boundary (see below), so a multiply by the fp32 reciprocal rounds to the same bf16.
template <int DT>
__device__ __forceinline__ float scale_of(float mn, float mx, float qmax) {
  float range = rnd<DT>(__fsub_rn(mx, mn));
  range = fmaxf(range, rnd<DT>(1e-4f));
  // qmax is one of 3, 15, 255: correctly rounded fp32 reciprocals as constants
  const float inv_qmax = qmax == 3.0f ? 0.3333333432674408f : (qmax == 15.0f ? 0.06666667014360428f : 0.003921568859368563f);
  if (DT == DARTKV_BF16) return rnd<DT>(__fmul_rn(range, inv_qmax));
  return rnd<DT>(__fdiv_rn(range, qmax));
}
// 1 / scale for the reciprocal-multiply quotient (bf16 only): the approximate reciprocal is within 2^-22
template <int DT>
__device__ __forceinline__ float inverse_scale(float scale) {
  if (DT != DARTKV_BF16) return 0.0f;   // fp16 takes the true division
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(scale));
  return r;
}

// ---- packed code computation -------------------------------------------------------------------
// Two elements that share (min, scale) travel as one 16-bit pair.  The reference computes
//   code = clamp(rint(r16(r16(x - min) / scale)), 0, qmax)        (r16 = round to the data dtype)
// which is evaluated here as
//   a2   = x2 - min2                      packed subtract, one rounding (exact for the 16-bit formats)
//   q    = a * (1/scale)  (bf16)          the quotient of two 8-bit significands is never within 2^-17
//          a / scale      (fp16)          of a bf16 rounding boundary and never on one, so a reciprocal
//                                         multiply rounds to the same bf16 as the IEEE quotient; fp16
//                                         significands are too long for that and take the true division
//   r2   = r16(q) packed
//   m2   = r2 + magic                     magic = 128 (bf16) / 1024 (fp16): the sum has unit ulp, so the
//                                         packed add rounds half-to-even to an integer = rint
// leaving the codes in the low mantissa bits of each half.  bf16 cannot hold 128 + code for 8-bit
// codes; that combination uses scalar rint.
template <int DT> struct Pack16;
template <> struct Pack16<DARTKV_BF16> {
  static constexpr uint32_t kMagic = 0x43004300u;   // 128.0 | 128.0
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    uint32_t d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) {
    uint32_t d; asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t d; asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
  static __device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
  static __device__ __forceinline__ uint32_t pack(float hi_v, float lo_v) {
    uint32_t d; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_v), "f"(lo_v)); return d;
  }
  static __device__ __forceinline__ float quotient(float a, float s, float inv) { (void)s; return __fmul_rn(a, inv); }
  static __device__ __forceinline__ uint16_t bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
  // |x| as a double, from the 15 magnitude bits (subnormal inputs count as zero)
  static __device__ __forceinline__ double abs_double(uint32_t b) {
    const uint32_t mag = b & 0x7FFFu;
    return __hiloint2double(mag >= 0x80u ? (int)(mag * 8192u + 0x38000000u) : 0, 0);
  }
};
template <> struct Pack16<DARTKV_F16> {
  static constexpr uint32_t kMagic = 0x64006400u;   // 1024.0 | 1024.0
  static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
    uint32_t d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) {
    uint32_t d; asm("min.NaN.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t d; asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ float lo(uint32_t v) { return __half2float(__ushort_as_half((uint16_t)(v & 0xFFFFu))); }
  static __device__ __forceinline__ float hi(uint32_t v) { return __half2float(__ushort_as_half((uint16_t)(v >> 16))); }
  static __device__ __forceinline__ uint32_t pack(float hi_v, float lo_v) {
    uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_v), "f"(lo_v)); return d;
  }
  static __device__ __forceinline__ float quotient(float a, float s, float inv) { (void)inv; return __fdiv_rn(a, s); }
  static __device__ __forceinline__ uint16_t bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
  static __device__ __forceinline__ double abs_double(uint32_t b) {
    const uint32_t mag = b & 0x7FFFu;
    if (mag < 0x400u) return (double)__half2float(__ushort_as_half((uint16_t)mag));   // zero / subnormal
    return __hiloint2double((int)(mag * 1024u + 0x3F000000u), 0);
  }
};

// codes of a pair in bits [7:0] (low element) and [23:16] (high element)
template <int DT, int BITS>
__device__ __forceinline__ uint32_t pair_codes(uint32_t x2, uint32_t mn2, float s, float inv, uint32_t cap2) {
  using P = Pack16<DT>;
  const uint32_t a2 = P::sub(x2, mn2);
  const float q_lo = P::quotient(P::lo(a2), s, inv), q_hi = P::quotient(P::hi(a2), s, inv);
  if (DT == DARTKV_BF16 && BITS == 8) {
    const uint32_t r2 = P::pack(q_hi, q_lo);
    const uint32_t c_lo = (uint32_t)fminf(rintf(P::lo(r2)), 255.0f), c_hi = (uint32_t)fminf(rintf(P::hi(r2)), 255.0f);
    return c_lo | (c_hi << 16);
  }
  const uint32_t m2 = P::min2(P::add(P::pack(q_hi, q_lo), P::kMagic), cap2);   // magic + code, capped at magic + qmax
  return m2 & (DT == DARTKV_BF16 ? 0x007F007Fu : 0x03FF03FFu);
}

template <int DT>
__device__ __forceinline__ uint32_t cap_pair(float qmax) {
  const uint32_t one = Pack16<DT>::bits((DT == DARTKV_BF16 ? 128.0f : 1024.0f) + qmax);
  return one * 0x00010001u;
}

__device__ __forceinline__ uint32_t umin16x2(uint32_t a, uint32_t b) {
  uint32_t d; asm("min.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}

// |x| of a normal 16-bit float, from its 15 magnitude bits, as the high word of a double (low word 0)
template <int DT>
__device__ __forceinline__ double normal_abs_as_double(uint32_t magnitude) {
  constexpr uint32_t kShift = DT == DARTKV_BF16 ? 8192u : 1024u;
  constexpr uint32_t kBias = DT == DARTKV_BF16 ? 0x38000000u : 0x3F000000u;
  return __hiloint2double((int)(magnitude * kShift + kBias), 0);
}
// any magnitude, zero and subnormals included
template <int DT>
__device__ __forceinline__ double any_abs_as_double(uint32_t magnitude) {
  constexpr uint32_t kMinNormal = DT == DARTKV_BF16 ? 0x80u : 0x400u;
  constexpr double kUnit = DT == DARTKV_BF16 ? 9.183549615799121e-41 : 5.9604644775390625e-08;   // 2^-133, 2^-24
  return magnitude >= kMinNormal ? normal_abs_as_double<DT>(magnitude) : (double)(int)magnitude * kUnit;
}

// KBITS: 0 = mixed 2+2-bit keys, else uniform keys with KBITS bits.
// One block of 64 * TQ threads per (batch*head, page); thread (tq, p) owns the adjacent channels 2p, 2p+1, which
// travel together as one packed pair through both passes, for the tokens of quarter tq (TQ = 1, 2 or 4 splits
// of the page's 128 tokens).  The splits meet twice in shared memory: for the channel statistics after pass 1
// and for the ranks of the promoted channels.  More threads per page mean more resident warps per SM (the page
// staging, 32 KiB, is what limits the pages per SM) and a shorter critical path when a step brings few pages.
template <int DT, int KBITS, int TQ>
__global__ void __launch_bounds__(64 * TQ) fast_key_pages_kernel(dartkv_cache_desc d, RowSource src, int first_slot,
                                                                 int num_pages, int page_token_start,
                                                                 const int32_t* __restrict__ indices, int32_t* nonfinite,
                                                                 const dartkv_append_plan* device_plan) {
  using P = Pack16<DT>;
  constexpr int TOK = kP / TQ;   // tokens per thread and pass
  if (device_plan) {
    // the step was planned on the device (the grid is the most pages such a step can bring): take the step's
    // numbers from there; blocks beyond its pages have nothing to do
    first_slot = device_plan->first_page;
    num_pages = device_plan->num_pages;
    page_token_start = device_plan->page_token_start;
    src.chunk_start = device_plan->chunk_start;
    if ((int)blockIdx.y >= num_pages) return;
  }
  __shared__ __align__(16) uint32_t s_page[kP * 64];   // [token][channel pair]
  __shared__ __align__(16) uint32_t s_key[kD];
  __shared__ uint32_t s_part[TQ > 1 ? 3 * TQ * 64 : 1];      // [min | max | smallest magnitude][split][pair]
  __shared__ double s_sum[TQ > 1 ? 2 * TQ * 64 : 1];         // [low | high channel][split][pair]
  __shared__ int s_rank[TQ > 1 ? TQ * kD : 1];               // [split][channel]
  const int bh = blockIdx.x, pg = blockIdx.y, p = threadIdx.x & 63, tq = threadIdx.x >> 6;
  const int t0 = page_token_start + pg * kP;
  const uint16_t *chunk_base, *ring_base;
  src.bases(bh, chunk_base, ring_base);
  // stage the page: 2048 16-byte pieces (thread: piece tid%16 of rows tid/16, tid/16 + 4*TQ, ...)
  {
    const int piece = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    char* dst = reinterpret_cast<char*>(s_page) + r0 * 256 + piece * 16;
    if (t0 >= src.chunk_start) {
      const char* from = reinterpret_cast<const char*>(chunk_base + (int64_t)(t0 - src.chunk_start + r0) * src.st) + piece * 16;
      const int64_t step = src.st * (8 * TQ);   // 4 * TQ rows, in bytes
#pragma unroll 8
      for (int k = 0; k < kP / (4 * TQ); ++k) cp_async16(dst + k * (1024 * TQ), from + k * step);
    } else {
      for (int k = 0; k < kP / (4 * TQ); ++k)
        cp_async16(dst + k * (1024 * TQ),
                   reinterpret_cast<const char*>(src.row_from(chunk_base, ring_base, t0 + r0 + 4 * TQ * k)) + piece * 16);
    }
  }
  cp_async_wait_all();
  __syncthreads();

  uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + first_slot + pg) * d.key_page_bytes;
  const uint32_t* col = s_page + p;
  // pass 1: packed min / max (NaN-propagating, so Inf/NaN inputs surface in them) and, for mixed pages,
  // sum |k| per channel in double (exact for 16-bit inputs).  The loop takes every magnitude for a normal
  // number; the smallest magnitude seen says whether a channel has to be summed again with care.
  uint32_t mn2 = col[tq * TOK * 64], mx2 = mn2, min_mag2 = 0xFFFFFFFFu;
  constexpr uint32_t kMinNormal = DT == DARTKV_BF16 ? 0x80u : 0x400u;
  double sum_lo = 0.0, sum_hi = 0.0;
#pragma unroll 8
  for (int t = tq * TOK; t < (tq + 1) * TOK; ++t) {
    const uint32_t x2 = col[t * 64];
    mn2 = P::min2(mn2, x2);
    mx2 = P::max2(mx2, x2);
    if (KBITS == 0) {
      const uint32_t mag2 = x2 & 0x7FFF7FFFu;
      min_mag2 = umin16x2(min_mag2, mag2);
      sum_lo += normal_abs_as_double<DT>(mag2 & 0xFFFFu);
      sum_hi += normal_abs_as_double<DT>(mag2 >> 16);
    }
  }
  if (TQ > 1) {
    // the splits of a channel pair exchange their partial statistics; every split then holds the page's values
    s_part[(0 * TQ + tq) * 64 + p] = mn2;
    s_part[(1 * TQ + tq) * 64 + p] = mx2;
    if (KBITS == 0) {
      s_part[(2 * TQ + tq) * 64 + p] = min_mag2;
      s_sum[(0 * TQ + tq) * 64 + p] = sum_lo;
      s_sum[(1 * TQ + tq) * 64 + p] = sum_hi;
    }
    __syncthreads();
    mn2 = s_part[(0 * TQ) * 64 + p];
    mx2 = s_part[(1 * TQ) * 64 + p];
    if (KBITS == 0) { min_mag2 = s_part[(2 * TQ) * 64 + p]; sum_lo = s_sum[p]; sum_hi = s_sum[TQ * 64 + p]; }
#pragma unroll
    for (int o = 1; o < TQ; ++o) {
      mn2 = P::min2(mn2, s_part[(0 * TQ + o) * 64 + p]);
      mx2 = P::max2(mx2, s_part[(1 * TQ + o) * 64 + p]);
      if (KBITS == 0) {
        min_mag2 = umin16x2(min_mag2, s_part[(2 * TQ + o) * 64 + p]);
        sum_lo += s_sum[(0 * TQ + o) * 64 + p];     // sums of 16-bit magnitudes are exact in double: any order
        sum_hi += s_sum[(1 * TQ + o) * 64 + p];
      }
    }
  }
  const float mn_lo = P::lo(mn2), mn_hi = P::hi(mn2), mx_lo = P::lo(mx2), mx_hi = P::hi(mx2);
  const bool bad = !(isfinite(mn_lo) && isfinite(mn_hi) && isfinite(mx_lo) && isfinite(mx_hi));
  int slot_lo = -1, slot_hi = -1;
  float qmax_lo, qmax_hi;
  if (KBITS == 0) {
    const int K = d.promoted;
    int32_t* idx_field = reinterpret_cast<int32_t*>(page + d.key_off_index);
    const int c_lo = 2 * p, c_hi = 2 * p + 1;
    if (indices != nullptr) {
      const int32_t* mine = indices + ((int64_t)bh * num_pages + pg) * K;
      for (int k = 0; k < K; ++k) {
        const int ch = mine[k];
        if (ch == c_lo) slot_lo = k;
        if (ch == c_hi) slot_hi = k;
      }
      for (int k = threadIdx.x; k < K; k += 64 * TQ) idx_field[k] = mine[k];
    } else if (K == kD) {
      slot_lo = c_lo; slot_hi = c_hi;
      if (tq == 0) { idx_field[c_lo] = c_lo; idx_field[c_hi] = c_hi; }
    } else if (K > 0) {
      if ((min_mag2 & 0xFFFFu) < kMinNormal || (min_mag2 >> 16) < kMinNormal) {   // zeros or subnormals: sum again
        sum_lo = 0.0; sum_hi = 0.0;
        for (int t = 0; t < kP; ++t) {
          const uint32_t mag2 = col[t * 64] & 0x7FFF7FFFu;
          sum_lo += any_abs_as_double<DT>(mag2 & 0xFFFFu);
          sum_hi += any_abs_as_double<DT>(mag2 >> 16);
        }
      }
      // rank by (score descending, channel ascending): scores are non-negative 16-bit floats, so their bit
      // patterns order like integers and one unsigned key carries both criteria
      const uint32_t key_lo = ((uint32_t)P::bits(__fdiv_rn((float)sum_lo, (float)kP)) << 7) | (uint32_t)(kD - 1 - c_lo);
      const uint32_t key_hi = ((uint32_t)P::bits(__fdiv_rn((float)sum_hi, (float)kP)) << 7) | (uint32_t)(kD - 1 - c_hi);
      if (tq == 0) {
        s_key[c_lo] = key_lo;
        s_key[c_hi] = key_hi;
      }
      __syncthreads();
      // every split counts the larger keys among its share of the 128 channels
      int rank_lo = 0, rank_hi = 0;
#pragma unroll 4
      for (int o = tq * (kD / 4 / TQ); o < (tq + 1) * (kD / 4 / TQ); ++o) {
        const uint4 k4 = reinterpret_cast<const uint4*>(s_key)[o];
        rank_lo += (k4.x > key_lo) + (k4.y > key_lo) + (k4.z > key_lo) + (k4.w > key_lo);
        rank_hi += (k4.x > key_hi) + (k4.y > key_hi) + (k4.z > key_hi) + (k4.w > key_hi);
      }
      if (TQ > 1) {
        s_rank[tq * kD + c_lo] = rank_lo;
        s_rank[tq * kD + c_hi] = rank_hi;
        __syncthreads();
        rank_lo = 0; rank_hi = 0;
#pragma unroll
        for (int o = 0; o < TQ; ++o) { rank_lo += s_rank[o * kD + c_lo]; rank_hi += s_rank[o * kD + c_hi]; }
      }
      if (rank_lo < K) { slot_lo = rank_lo; if (tq == 0) idx_field[rank_lo] = c_lo; }
      if (rank_hi < K) { slot_hi = rank_hi; if (tq == 0) idx_field[rank_hi] = c_hi; }
    }
    qmax_lo = slot_lo >= 0 ? 15.0f : 3.0f;
    qmax_hi = slot_hi >= 0 ? 15.0f : 3.0f;
  } else {
    qmax_lo = qmax_hi = (float)((1 << KBITS) - 1);
  }
  const float scale_lo = scale_of<DT>(mn_lo, mx_lo, qmax_lo), scale_hi = scale_of<DT>(mn_hi, mx_hi, qmax_hi);
  if (tq == 0) {
    store_f(page + d.key_off_scale, d.md_dtype, 2 * p, scale_lo);
    store_f(page + d.key_off_scale, d.md_dtype, 2 * p + 1, scale_hi);
    store_f(page + d.key_off_zero, d.md_dtype, 2 * p, mn_lo);
    store_f(page + d.key_off_zero, d.md_dtype, 2 * p + 1, mn_hi);
  }
  const float inv_lo = inverse_scale<DT>(scale_lo), inv_hi = inverse_scale<DT>(scale_hi);
  const uint32_t cap2 = (uint32_t)P::bits((DT == DARTKV_BF16 ? 128.0f : 1024.0f) + qmax_lo) |
                        ((uint32_t)P::bits((DT == DARTKV_BF16 ? 128.0f : 1024.0f) + qmax_hi) << 16);

  // pass 2: codes of (channel 2p, channel 2p+1) for one token per step.  A plane's fields of both channels
  // gather in one register (channel 2p in the low half, 2p+1 in the high half, 16/BITS tokens each); two such
  // registers split into one 32-bit word per channel.  Split tq produces words [tq, tq+1) * WORDS / TQ.
  constexpr int BITS = KBITS == 0 ? 2 : KBITS;      // bits per stored plane
  constexpr int CODE_BITS = KBITS == 0 ? 4 : KBITS; // bits the quantizer produces
  constexpr int PER_HALF = 16 / BITS;               // tokens per 16-bit half of a plane word
  constexpr int WORDS = kP / (2 * PER_HALF);        // 32-bit words per channel and plane
  constexpr int MY_WORDS = WORDS / TQ;              // words of this split
  constexpr int CHUNK = MY_WORDS < 4 ? MY_WORDS : 4;   // words per store
  static_assert(MY_WORDS >= 2 && MY_WORDS % CHUNK == 0, "page words do not split this way");
  constexpr uint32_t FIELD2 = ((1u << BITS) - 1u) * 0x00010001u;
  uint32_t* low_lo = reinterpret_cast<uint32_t*>(page + (2 * p) * (WORDS * 4));
  uint32_t* low_hi = low_lo + WORDS;
  uint32_t* high_lo = (KBITS == 0 && slot_lo >= 0) ? reinterpret_cast<uint32_t*>(page + d.key_off_high + slot_lo * (WORDS * 4)) : nullptr;
  uint32_t* high_hi = (KBITS == 0 && slot_hi >= 0) ? reinterpret_cast<uint32_t*>(page + d.key_off_high + slot_hi * (WORDS * 4)) : nullptr;
#pragma unroll 1
  for (int w4 = tq * MY_WORDS; w4 < (tq + 1) * MY_WORDS; w4 += CHUNK) {
    uint32_t a_lo[CHUNK], a_hi[CHUNK], b_lo[CHUNK], b_hi[CHUNK];   // a: low plane, b: high plane
#pragma unroll
    for (int q = 0; q < CHUNK; ++q) {
      uint32_t acc_a[2], acc_b[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t fa = 0, fb = 0;
        const int base = ((w4 + q) * 2 + half) * PER_HALF;
#pragma unroll
        for (int u = 0; u < PER_HALF; ++u) {
          const uint32_t x2 = col[(base + u) * 64];
          const uint32_t a2 = P::sub(x2, mn2);
          const float q_l = P::quotient(P::lo(a2), scale_lo, inv_lo), q_h = P::quotient(P::hi(a2), scale_hi, inv_hi);
          uint32_t codes;
          if (DT == DARTKV_BF16 && CODE_BITS == 8) {
            const uint32_t r2 = P::pack(q_h, q_l);
            codes = (uint32_t)fminf(rintf(P::lo(r2)), 255.0f) | ((uint32_t)fminf(rintf(P::hi(r2)), 255.0f) << 16);
          } else {
            codes = P::min2(P::add(P::pack(q_h, q_l), P::kMagic), cap2);
          }
          fa += (codes & FIELD2) << (BITS * u);
          if (KBITS == 0) fb += ((codes >> 2) & FIELD2) << (BITS * u);
        }
        acc_a[half] = fa;
        acc_b[half] = fb;
      }
      a_lo[q] = __byte_perm(acc_a[0], acc_a[1], 0x5410);
      a_hi[q] = __byte_perm(acc_a[0], acc_a[1], 0x7632);
      if (KBITS == 0) {
        b_lo[q] = __byte_perm(acc_b[0], acc_b[1], 0x5410);
        b_hi[q] = __byte_perm(acc_b[0], acc_b[1], 0x7632);
      }
    }
    if (CHUNK == 4) {
      reinterpret_cast<uint4*>(low_lo)[w4 / 4] = make_uint4(a_lo[0], a_lo[1], a_lo[2], a_lo[3]);
      reinterpret_cast<uint4*>(low_hi)[w4 / 4] = make_uint4(a_hi[0], a_hi[1], a_hi[2], a_hi[3]);
      if (KBITS == 0) {
        if (high_lo) reinterpret_cast<uint4*>(high_lo)[w4 / 4] = make_uint4(b_lo[0], b_lo[1], b_lo[2], b_lo[3]);
        if (high_hi) reinterpret_cast<uint4*>(high_hi)[w4 / 4] = make_uint4(b_hi[0], b_hi[1], b_hi[2], b_hi[3]);
      }
    } else {
      reinterpret_cast<uint2*>(low_lo)[w4 / 2] = make_uint2(a_lo[0], a_lo[CHUNK - 1]);
      reinterpret_cast<uint2*>(low_hi)[w4 / 2] = make_uint2(a_hi[0], a_hi[CHUNK - 1]);
      if (KBITS == 0) {
        if (high_lo) reinterpret_cast<uint2*>(high_lo)[w4 / 2] = make_uint2(b_lo[0], b_lo[CHUNK - 1]);
        if (high_hi) reinterpret_cast<uint2*>(high_hi)[w4 / 2] = make_uint2(b_hi[0], b_hi[CHUNK - 1]);
      }
    }
  }
  if (bad && nonfinite) *nonfinite = 1;
}

// Values: eight lanes per token row (16 channels per lane), four rows per warp per step, two steps in
// flight; grid (64-row blocks of one (batch, head), batch*head).  VBITS in {2,4,8}; lanes_per_group =
// value_group / 16.
template <int DT, int VBITS>
__global__ void __launch_bounds__(256) fast_value_rows_kernel(dartkv_cache_desc d, RowSource src, int value_begin,
                                                              int count, int lanes_per_group, int32_t* nonfinite,
                                                              const dartkv_append_plan* device_plan) {
  using P = Pack16<DT>;
  constexpr int STEPS = 2;
  if (device_plan) {   // planned on the device: the grid covers the most rows such a step can pack
    value_begin = device_plan->value_begin;
    count = device_plan->value_end - device_plan->value_begin;
    src.chunk_start = device_plan->chunk_start;
  }
  const int bh = blockIdx.y, lane = threadIdx.x & 31;
  const int sub = lane >> 3, part = lane & 7;   // row within the step, 16-channel slice of the row
  const int first = (blockIdx.x * 8 + (threadIdx.x >> 5)) * (4 * STEPS);
  if (first >= count) return;
  const uint16_t *chunk_base, *ring_base;
  src.bases(bh, chunk_base, ring_base);
  uint4 raw[STEPS][2];
  int t_of[STEPS];
  bool live[STEPS];
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const int row = first + 4 * s + sub;
    live[s] = row < count;
    t_of[s] = value_begin + (live[s] ? row : count - 1);
    const uint4* ptr = reinterpret_cast<const uint4*>(src.row_from(chunk_base, ring_base, t_of[s]) + part * 16);
    raw[s][0] = ptr[0];
    raw[s][1] = ptr[1];
  }
  constexpr float qmax = (float)((1 << VBITS) - 1);
  const uint32_t cap2 = cap_pair<DT>(qmax);
  bool bad = false;
#pragma unroll
  for (int s = 0; s < STEPS; ++s) {
    const uint32_t x[8] = {raw[s][0].x, raw[s][0].y, raw[s][0].z, raw[s][0].w, raw[s][1].x, raw[s][1].y, raw[s][1].z, raw[s][1].w};
    uint32_t mn2 = x[0], mx2 = x[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) {
      mn2 = P::min2(mn2, x[i]);
      mx2 = P::max2(mx2, x[i]);
    }
    for (int off = 1; off < lanes_per_group; off <<= 1) {
      mn2 = P::min2(mn2, __shfl_xor_sync(0xffffffffu, mn2, off));
      mx2 = P::max2(mx2, __shfl_xor_sync(0xffffffffu, mx2, off));
    }
    // NaN-propagating min / max: any Inf or NaN of the group ends up in mn or mx
    const uint32_t mn1 = P::min2(mn2, mn2 >> 16), mx1 = P::max2(mx2, mx2 >> 16);
    const float mn = P::lo(mn1), mx = P::lo(mx1);
    bad |= live[s] && !(isfinite(mn) && isfinite(mx));
    const float scale = scale_of<DT>(mn, mx, qmax);
    const float inv = inverse_scale<DT>(scale);
    const uint32_t mnp = (mn1 & 0xFFFFu) * 0x00010001u;
    // codes of 16/(2*VBITS) pairs gather in one register (even channels in the low half, odd in the high half)
    constexpr int PAIRS = 8 / VBITS;                      // pairs per gather register
    constexpr int GATHERS = 8 / PAIRS;
    constexpr uint32_t LOMASK = VBITS == 2 ? 0x3333u : VBITS == 4 ? 0x0F0Fu : 0x00FFu;
    uint32_t half_word[GATHERS];
#pragma unroll
    for (int g = 0; g < GATHERS; ++g) {
      uint32_t acc = 0;
#pragma unroll
      for (int i = 0; i < PAIRS; ++i) acc += pair_codes<DT, VBITS>(x[g * PAIRS + i], mnp, scale, inv, cap2) << (2 * VBITS * i);
      half_word[g] = (acc & LOMASK) | ((acc >> (16 - VBITS)) & (LOMASK << VBITS));
    }
    if (!live[s]) continue;
    const int64_t out_row = (int64_t)bh * d.max_value_tokens + (t_of[s] - d.sink_tokens);
    uint8_t* codes = d.v_codes + out_row * d.value_row_bytes;
    if (VBITS == 2) {
      reinterpret_cast<uint32_t*>(codes)[part] = half_word[0] | (half_word[1] << 16);
    } else if (VBITS == 4) {
      reinterpret_cast<uint2*>(codes)[part] = make_uint2(half_word[0] | (half_word[1] << 16), half_word[2] | (half_word[3] << 16));
    } else {
      reinterpret_cast<uint4*>(codes)[part] = make_uint4(half_word[0] | (half_word[1] << 16), half_word[2] | (half_word[3] << 16),
                                                         half_word[4] | (half_word[5] << 16), half_word[6] | (half_word[7] << 16));
    }
    if ((part % lanes_per_group) == 0) {
      const int g = part / lanes_per_group;
      store_f(d.v_meta, d.md_dtype, (out_row * 2 + 0) * d.value_groups + g, scale);
      store_f(d.v_meta, d.md_dtype, (out_row * 2 + 1) * d.value_groups + g, mn);
    }
  }
  if (bad && nonfinite) *nonfinite = 1;
}

bool fast_common(const dartkv_cache_desc* d, int64_t sb, int64_t sh, int64_t st) {
  return (d->dtype == DARTKV_F16 || d->dtype == DARTKV_BF16) && d->head_dim == kD && st % 8 == 0 && sb % 8 == 0 &&
         sh % 8 == 0;
}

}  // namespace

// bit 0: keys can take the fast kernel; bit 1: values can
int dartkv_append_fast_supported(const dartkv_cache_desc* d, const dartkv_append_plan* p, int64_t st) {
  if (!fast_common(d, 0, 0, st)) return 0;
  int ok = 0;
  if (d->page_size == kP && d->key_group == kP && (p->num_pages == 0 || p->last_page_tokens == kP) &&
      (d->key_mode == DARTKV_QUANTIZED_PAGE || d->promoted <= kD))
    ok |= 1;
  if (d->value_group == 16 || d->value_group == 32 || d->value_group == 64 || d->value_group == 128) ok |= 2;
  return ok;
}

#ifndef APPEND_KEY_SPLITS
#define APPEND_KEY_SPLITS 4
#endif

template <int DT, int TQ>
static int launch_keys_split(const dartkv_cache_desc& d, const dartkv_append_plan& p, const RowSource& src,
                             const int32_t* indices, int32_t* nonfinite, cudaStream_t stream,
                             const dartkv_append_plan* device_plan) {
  dim3 grid(d.batch * d.kv_heads, p.num_pages);
  if (d.key_mode == DARTKV_MIXED_PAGE)
    fast_key_pages_kernel<DT, 0, TQ><<<grid, 64 * TQ, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite, device_plan);
  else if (d.key_bits == 2)
    fast_key_pages_kernel<DT, 2, TQ><<<grid, 64 * TQ, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite, device_plan);
  else if (d.key_bits == 4)
    fast_key_pages_kernel<DT, 4, TQ><<<grid, 64 * TQ, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite, device_plan);
  else
    fast_key_pages_kernel<DT, 8, TQ><<<grid, 64 * TQ, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite, device_plan);
  DARTKV_LAUNCH_OK("fast_key_pages_kernel");
  return DARTKV_OK;
}

template <int DT>
static int launch_keys(const dartkv_cache_desc& d, const dartkv_append_plan& p, const RowSource& src,
                       const int32_t* indices, int32_t* nonfinite, cudaStream_t stream,
                       const dartkv_append_plan* device_plan) {
#ifdef APPEND_KEY_SPLITS_FIXED
  return launch_keys_split<DT, APPEND_KEY_SPLITS>(d, p, src, indices, nonfinite, stream, device_plan);
#else
  // Four token splits per page give a step of few pages more warps and a shorter critical path; with thousands of
  // pages in flight the splits' extra combine work costs more than it hides: two splits (measured on bulk appends
  // of bf16 [16,8,4096,128]: 123 us against 132 us; a 128-token step replayed from a graph: 10.1 against 9.9 us).
  if ((long long)d.batch * d.kv_heads * p.num_pages >= 2048)
    return launch_keys_split<DT, 2>(d, p, src, indices, nonfinite, stream, device_plan);
  return launch_keys_split<DT, APPEND_KEY_SPLITS>(d, p, src, indices, nonfinite, stream, device_plan);
#endif
}

template <int DT>
static int launch_values(const dartkv_cache_desc& d, const dartkv_append_plan& p, const RowSource& src,
                         int32_t* nonfinite, cudaStream_t stream, const dartkv_append_plan* device_plan) {
  const int count = p.value_end - p.value_begin;
  DARTKV_REQUIRE(d.batch * d.kv_heads <= 65535, "batch * kv_heads above 65535");
  const dim3 blocks((unsigned)((count + 63) / 64), d.batch * d.kv_heads);   // 8 warps per block, 8 rows per warp
  const int lpg = d.value_group / 16;
  if (d.value_bits == 2)
    fast_value_rows_kernel<DT, 2><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite, device_plan);
  else if (d.value_bits == 4)
    fast_value_rows_kernel<DT, 4><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite, device_plan);
  else
    fast_value_rows_kernel<DT, 8><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite, device_plan);
  DARTKV_LAUNCH_OK("fast_value_rows_kernel");
  return DARTKV_OK;
}

// device_plan (optional): the step's plan in device memory, written by a kernel earlier on the stream; *p then
// only sizes the grids (the most pages / rows the step can bring)
int dartkv_append_fast_keys(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* keys, int64_t sb,
                            int64_t sh, int64_t st, const int32_t* indices, int32_t* nonfinite, cudaStream_t stream,
                            const dartkv_append_plan* device_plan) {
  if (p->num_pages == 0) return DARTKV_OK;
  DARTKV_REQUIRE(p->num_pages <= 65535, "too many pages in one append (limit 65535)");
  RowSource src{keys, d->k_ring, sb, sh, st, p->chunk_start, d->ring_tokens, d->kv_heads};
  return d->dtype == DARTKV_F16 ? launch_keys<DARTKV_F16>(*d, *p, src, indices, nonfinite, stream, device_plan)
                                : launch_keys<DARTKV_BF16>(*d, *p, src, indices, nonfinite, stream, device_plan);
}

int dartkv_append_fast_values(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* values, int64_t sb,
                              int64_t sh, int64_t st, int32_t* nonfinite, cudaStream_t stream,
                              const dartkv_append_plan* device_plan) {
  if (p->value_end <= p->value_begin) return DARTKV_OK;
  RowSource src{values, d->v_ring, sb, sh, st, p->chunk_start, d->ring_tokens, d->kv_heads};
  return d->dtype == DARTKV_F16 ? launch_values<DARTKV_F16>(*d, *p, src, nonfinite, stream, device_plan)
                                : launch_values<DARTKV_BF16>(*d, *p, src, nonfinite, stream, device_plan);
}
