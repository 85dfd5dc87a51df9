// Page-shaped quantize+pack kernels for the common geometry: head_dim 128, 16-bit data,
// full 128-token key pages with one 128-token key group, value groups of 32/64/128 channels.
//
// Keys (one block of 128 threads per (batch*head, page)): the page is staged in shared memory
// with 16-byte async copies; thread c owns channel c: one pass for min / max / sum|k|, a
// block-wide rank for the promoted channels, one pass that emits the codes and packs them in
// registers, then 32-byte row stores.  Values (one warp per token row): four channels per lane,
// group min/max by xor-shuffles, packed bytes and metadata written coalesced.
// HBM traffic per page: 64 KiB read (K and V rows), 10.6 KiB written (2-bit, 32 promoted).
// The arithmetic is the reference's per-op rounding in the data dtype
// (src/dart/quantization.py:178-186, src/dart/mixed.py:200-209).

#include "common.cuh"

namespace {

constexpr int kD = 128;
constexpr int kP = 128;

template <int DT> struct Elem;
template <> struct Elem<DARTKV_F16> {
  using type = __half;
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
};
template <> struct Elem<DARTKV_BF16> {
  using type = __nv_bfloat16;
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
};

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
  // 16-bit elements; rows are head_dim contiguous elements
  __device__ __forceinline__ const uint16_t* row(int bh, int t) const {
    if (t >= chunk_start) {
      int b = bh / kv_heads, h = bh % kv_heads;
      return reinterpret_cast<const uint16_t*>(chunk) + (int64_t)b * sb + (int64_t)h * sh + (int64_t)(t - chunk_start) * st;
    }
    return reinterpret_cast<const uint16_t*>(ring) + ((int64_t)bh * ring_tokens + (t % ring_tokens)) * kD;
  }
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

template <int DT>
__device__ __forceinline__ float scale_of(float mn, float mx, float qmax) {
  float range = rnd<DT>(__fsub_rn(mx, mn));
  range = fmaxf(range, rnd<DT>(1e-4f));
  return rnd<DT>(__fdiv_rn(range, qmax));
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
    uint32_t d; asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t d; asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
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
    uint32_t d; asm("min.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
  }
  static __device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    uint32_t d; asm("max.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
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

// KBITS: 0 = mixed 2+2-bit keys, else uniform keys with KBITS bits
template <int DT, int KBITS>
__global__ void __launch_bounds__(128) fast_key_pages_kernel(dartkv_cache_desc d, RowSource src, int first_slot,
                                                             int num_pages, int page_token_start,
                                                             const int32_t* __restrict__ indices, int32_t* nonfinite) {
  using P = Pack16<DT>;
  __shared__ __align__(16) uint16_t s_page[kP * kD];
  __shared__ float s_score[kD];
  const int bh = blockIdx.x, pg = blockIdx.y, c = threadIdx.x;
  const int t0 = page_token_start + pg * kP;
  // stage the page: 2048 16-byte pieces, 16 per thread
  const uint16_t *chunk_base, *ring_base;
  src.bases(bh, chunk_base, ring_base);
  for (int i = c; i < kP * 16; i += 128) {
    int r = i >> 4, piece = i & 15;
    cp_async16(reinterpret_cast<char*>(s_page) + r * 256 + piece * 16,
               reinterpret_cast<const char*>(src.row_from(chunk_base, ring_base, t0 + r)) + piece * 16);
  }
  cp_async_wait_all();
  __syncthreads();

  uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + first_slot + pg) * d.key_page_bytes;
  const uint16_t* col = s_page + c;
  // pass 1: min / max on packed pairs, sum |k| in double (order independent for 16-bit data)
  uint32_t mn2 = (uint32_t)col[0] * 0x00010001u, mx2 = mn2;
  uint32_t exp_or = 0;   // bit 15 / 31 end up set iff some magnitude has an all-ones exponent (Inf or NaN)
  constexpr uint32_t kExpCarry = DT == DARTKV_BF16 ? 0x00800080u : 0x04000400u;
  double asum = 0.0;
#pragma unroll 4
  for (int t = 0; t < kP; t += 2) {
    const uint32_t lo = col[t * kD], hi = col[(t + 1) * kD];
    const uint32_t x2 = lo | (hi << 16);
    mn2 = P::min2(mn2, x2);
    mx2 = P::max2(mx2, x2);
    exp_or |= (x2 & 0x7FFF7FFFu) + kExpCarry;
    if (KBITS == 0) asum += P::abs_double(lo) + P::abs_double(hi);
  }
  const bool bad = (exp_or & 0x80008000u) != 0;
  const float mn = fminf(P::lo(mn2), P::hi(mn2)), mx = fmaxf(P::lo(mx2), P::hi(mx2));
  int slot = -1;
  float qmax;
  if (KBITS == 0) {
    const int K = d.promoted;
    int32_t* idx_field = reinterpret_cast<int32_t*>(page + d.key_off_index);
    if (indices != nullptr) {
      const int32_t* mine = indices + ((int64_t)bh * num_pages + pg) * K;
      for (int k = 0; k < K; ++k)
        if (mine[k] == c) slot = k;
      if (c < K) idx_field[c] = mine[c];
    } else if (K == kD) {
      slot = c;
      idx_field[c] = c;
    } else if (K > 0) {
      const float score = rnd<DT>(__fdiv_rn((float)asum, (float)kP));
      s_score[c] = score;
      __syncthreads();
      int rank = 0;
#pragma unroll 8
      for (int o = 0; o < kD; ++o) {
        const float other = s_score[o];
        rank += (other > score) || (other == score && o < c);
      }
      if (rank < K) { slot = rank; idx_field[rank] = c; }
    }
    qmax = slot >= 0 ? 15.0f : 3.0f;
  } else {
    qmax = (float)((1 << KBITS) - 1);
  }
  const float scale = scale_of<DT>(mn, mx, qmax);
  store_f(page + d.key_off_scale, d.md_dtype, c, scale);
  store_f(page + d.key_off_zero, d.md_dtype, c, mn);
  const float inv = __frcp_rn(scale);
  const uint32_t mnp = (uint32_t)P::bits(mn) * 0x00010001u;
  const uint32_t cap2 = cap_pair<DT>(qmax);

  // pass 2: a pair is (token i, token i + step) of a 32-bit output word, so both codes fall 16 bits apart
  constexpr int BITS = KBITS == 0 ? 2 : KBITS;      // bits per stored plane
  constexpr int CODE_BITS = KBITS == 0 ? 4 : KBITS; // bits the quantizer produces
  constexpr int PER_WORD = 32 / BITS;               // tokens per 32-bit word of a plane
  constexpr int STEP = PER_WORD / 2;
  constexpr int WORDS = kP / PER_WORD;
  constexpr uint32_t FIELD = ((1u << BITS) - 1u) * 0x00010001u;
  uint32_t* low_row = reinterpret_cast<uint32_t*>(page + c * (WORDS * 4));
  uint32_t* high_row = (KBITS == 0 && slot >= 0) ? reinterpret_cast<uint32_t*>(page + d.key_off_high + slot * (WORDS * 4)) : nullptr;
#pragma unroll 1
  for (int w4 = 0; w4 < WORDS; w4 += 4) {
    uint32_t lo_words[4], hi_words[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t lacc = 0, hacc = 0;
      const int base = (w4 + q) * PER_WORD;
#pragma unroll
      for (int u = 0; u < STEP; ++u) {
        const uint32_t x2 = (uint32_t)col[(base + u) * kD] | ((uint32_t)col[(base + u + STEP) * kD] << 16);
        const uint32_t codes = pair_codes<DT, CODE_BITS>(x2, mnp, scale, inv, cap2);
        lacc |= (codes & FIELD) << (BITS * u);
        if (KBITS == 0) hacc |= ((codes >> 2) & FIELD) << (BITS * u);
      }
      lo_words[q] = lacc;
      hi_words[q] = hacc;
    }
    reinterpret_cast<uint4*>(low_row)[w4 / 4] = make_uint4(lo_words[0], lo_words[1], lo_words[2], lo_words[3]);
    if (KBITS == 0 && high_row) reinterpret_cast<uint4*>(high_row)[w4 / 4] = make_uint4(hi_words[0], hi_words[1], hi_words[2], hi_words[3]);
  }
  if (bad && nonfinite) *nonfinite = 1;
}

// one warp per four token rows (loads issued together); VBITS in {2,4,8}; LPG = lanes per group
template <int DT, int VBITS>
__global__ void __launch_bounds__(256) fast_value_rows_kernel(dartkv_cache_desc d, RowSource src, int value_begin,
                                                              int count, int lanes_per_group, int32_t* nonfinite) {
  using P = Pack16<DT>;
  constexpr int ROWS = 4;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const uint32_t total = (uint32_t)d.batch * d.kv_heads * count;   // checked on the host to fit 32 bits
  const uint32_t first = (uint32_t)warp * ROWS;
  if (first >= total) return;
  uint2 raw[ROWS];
  int bh_of[ROWS], t_of[ROWS];
  {
    int bh = (int)(first / (uint32_t)count), j = (int)(first % (uint32_t)count);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      bh_of[r] = bh;
      t_of[r] = value_begin + j;
      raw[r] = *reinterpret_cast<const uint2*>(src.row(bh, t_of[r]) + lane * 4);
      if (first + r + 1 < total && ++j == count) { j = 0; ++bh; }
    }
  }
  constexpr float qmax = (float)((1 << VBITS) - 1);
  const uint32_t cap2 = cap_pair<DT>(qmax);
  bool bad = false;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (first + r >= total) break;
    const uint32_t x01 = raw[r].x, x23 = raw[r].y;
    constexpr uint32_t kExpCarry = DT == DARTKV_BF16 ? 0x00800080u : 0x04000400u;
    bad |= ((((x01 & 0x7FFF7FFFu) + kExpCarry) | ((x23 & 0x7FFF7FFFu) + kExpCarry)) & 0x80008000u) != 0;
    uint32_t mn2 = P::min2(x01, x23), mx2 = P::max2(x01, x23);
    for (int off = 1; off < lanes_per_group; off <<= 1) {
      mn2 = P::min2(mn2, __shfl_xor_sync(0xffffffffu, mn2, off));
      mx2 = P::max2(mx2, __shfl_xor_sync(0xffffffffu, mx2, off));
    }
    const float mn = fminf(P::lo(mn2), P::hi(mn2)), mx = fmaxf(P::lo(mx2), P::hi(mx2));
    const float scale = scale_of<DT>(mn, mx, qmax);
    const float inv = __frcp_rn(scale);
    const uint32_t mnp = (uint32_t)P::bits(mn) * 0x00010001u;
    const uint32_t c01 = pair_codes<DT, VBITS>(x01, mnp, scale, inv, cap2);
    const uint32_t c23 = pair_codes<DT, VBITS>(x23, mnp, scale, inv, cap2);
    const int64_t out_row = (int64_t)bh_of[r] * d.max_value_tokens + (t_of[r] - d.sink_tokens);
    uint8_t* codes = d.v_codes + out_row * d.value_row_bytes;
    if (VBITS == 2) {
      codes[lane] = (uint8_t)((c01 & 3u) | ((c01 >> 14) & 0xCu) | ((c23 & 3u) << 4) | ((c23 >> 10) & 0xC0u));
    } else if (VBITS == 4) {
      reinterpret_cast<uint16_t*>(codes)[lane] =
          (uint16_t)((c01 & 0xFu) | ((c01 >> 12) & 0xF0u) | ((c23 & 0xFu) << 8) | ((c23 >> 4) & 0xF000u));
    } else {
      reinterpret_cast<uint32_t*>(codes)[lane] =
          (c01 & 0xFFu) | ((c01 >> 8) & 0xFF00u) | ((c23 & 0xFFu) << 16) | ((c23 << 8) & 0xFF000000u);
    }
    if ((lane % lanes_per_group) == 0) {
      const int g = lane / lanes_per_group;
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
  if (d->value_group == 32 || d->value_group == 64 || d->value_group == 128) ok |= 2;
  return ok;
}

template <int DT>
static int launch_keys(const dartkv_cache_desc& d, const dartkv_append_plan& p, const RowSource& src,
                       const int32_t* indices, int32_t* nonfinite, cudaStream_t stream) {
  dim3 grid(d.batch * d.kv_heads, p.num_pages);
  if (d.key_mode == DARTKV_MIXED_PAGE)
    fast_key_pages_kernel<DT, 0><<<grid, 128, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite);
  else if (d.key_bits == 2)
    fast_key_pages_kernel<DT, 2><<<grid, 128, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite);
  else if (d.key_bits == 4)
    fast_key_pages_kernel<DT, 4><<<grid, 128, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite);
  else
    fast_key_pages_kernel<DT, 8><<<grid, 128, 0, stream>>>(d, src, p.first_page, p.num_pages, p.page_token_start, indices, nonfinite);
  DARTKV_LAUNCH_OK("fast_key_pages_kernel");
  return DARTKV_OK;
}

template <int DT>
static int launch_values(const dartkv_cache_desc& d, const dartkv_append_plan& p, const RowSource& src,
                         int32_t* nonfinite, cudaStream_t stream) {
  const int count = p.value_end - p.value_begin;
  const int64_t rows = (int64_t)d.batch * d.kv_heads * count;
  DARTKV_REQUIRE(rows < (1ll << 31), "too many value rows in one append (limit 2^31)");
  const unsigned blocks = (unsigned)((rows + 31) / 32);   // 8 warps per block, 4 rows per warp
  const int lpg = d.value_group / 4;
  if (d.value_bits == 2)
    fast_value_rows_kernel<DT, 2><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite);
  else if (d.value_bits == 4)
    fast_value_rows_kernel<DT, 4><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite);
  else
    fast_value_rows_kernel<DT, 8><<<blocks, 256, 0, stream>>>(d, src, p.value_begin, count, lpg, nonfinite);
  DARTKV_LAUNCH_OK("fast_value_rows_kernel");
  return DARTKV_OK;
}

int dartkv_append_fast_keys(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* keys, int64_t sb,
                            int64_t sh, int64_t st, const int32_t* indices, int32_t* nonfinite, cudaStream_t stream) {
  if (p->num_pages == 0) return DARTKV_OK;
  DARTKV_REQUIRE(p->num_pages <= 65535, "too many pages in one append (limit 65535)");
  RowSource src{keys, d->k_ring, sb, sh, st, p->chunk_start, d->ring_tokens, d->kv_heads};
  return d->dtype == DARTKV_F16 ? launch_keys<DARTKV_F16>(*d, *p, src, indices, nonfinite, stream)
                                : launch_keys<DARTKV_BF16>(*d, *p, src, indices, nonfinite, stream);
}

int dartkv_append_fast_values(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* values, int64_t sb,
                              int64_t sh, int64_t st, int32_t* nonfinite, cudaStream_t stream) {
  if (p->value_end <= p->value_begin) return DARTKV_OK;
  RowSource src{values, d->v_ring, sb, sh, st, p->chunk_start, d->ring_tokens, d->kv_heads};
  return d->dtype == DARTKV_F16 ? launch_values<DARTKV_F16>(*d, *p, src, nonfinite, stream)
                                : launch_values<DARTKV_BF16>(*d, *p, src, nonfinite, stream);
}
