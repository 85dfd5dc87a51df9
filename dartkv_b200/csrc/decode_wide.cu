// Tensor-core decode attention for every packed geometry with head_dim 128 and 128-token pages: keys with
// 2/4/8-bit codes or 2+2-bit promoted channels, key groups of 16..128 tokens, values with 2/4/8-bit codes and
// groups of 16..128 channels.  It takes the rounded flavours of the dequantization (per-op rounding in the
// metadata dtype = the reference's src/dart/quantization.py:96-109 and mixed.py:72-94; fp32 with one rounding
// to the cache dtype = src/dart/triton_ops.py:32-201), whose dequantized keys and values are 16-bit numbers.
// The 2-bit geometry of the headline workloads has kernels of its own (decode_fast.cu, decode_fused32.cu) that
// feed the MMAs from registers; this one trades some speed for generality:
//
//   * a warp owns 64 tokens of a page (the two warps of a pair share the page, four pairs per block) and walks
//     them in chunks of 16 tokens; the packed bytes of a chunk arrive through a two-stage cp.async ring that is
//     private to the warp, so the warps of a block never wait for each other while streaming;
//   * the chunk's keys are dequantized with packed 16-bit arithmetic (two tokens of a channel per register) into
//     a [channel][token] tile in shared memory, read back transposed by ldmatrix as the B operand of
//     S^T[head][token] = q K^T (m16n8k16, heads in the M rows);
//   * the chunk's values are dequantized (two channels of a token per register) into a [token][channel] tile,
//     read back transposed as the B operand of O[head][channel] += P V; the probabilities travel as a high and a
//     low 16-bit part in M rows 0..7 and 8..15 of one A operand, straight from the logits' accumulators;
//   * dense tokens, the block-level merge and the work split are those of the other tensor-core kernels.
//
// Algorithmic HBM bytes per page and (batch, kv head): key_page_bytes + 128 * (value_row_bytes + 4 * value_groups).

#include <atomic>

#include "decode_fast_common.cuh"

namespace {

// byte offsets of the fields of one staged chunk (16 tokens of one page), all multiples of 16
struct WideGeom {
  int k_high, k_index, k_scale, k_zero, v_codes, v_meta, stage_bytes;
  int key_kind;       // 2, 4, 8: uniform code width; 22: 2-bit codes plus a 2-bit plane for the promoted channels
  int key_groups;     // key groups per page
  int key_chunk;      // bytes of 16 tokens in one channel row of key codes (4, 8 or 16)
  int key_meta_bytes; // bytes of the page's scale (or zero point) array
  int warp_bytes;     // shared memory per warp: two stages, the tile, the promoted-slot map
};

constexpr int kTileBytes = 128 * 48;   // keys: [128 channels][16 tokens] rows of 48 B; values: [16 tokens] rows of 272 B
constexpr int kKeyRow = 48, kValueRow = 272;
static_assert(16 * kValueRow <= kTileBytes, "the value tile shares the key tile's memory");

struct WideBlockSmem {
  uint16_t q16[8][136];   // query heads of the row's KV head (rows rep.. are zero); 272-byte rows keep a quad's loads apart
  float merge_m[kWarps][4];
  float merge_l[kWarps][4];
  int slot_map[128];
};

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(row)));
}

// magic16(P) is the 16-bit float whose mantissa bit P weighs one: OR-ing a code into mantissa bits P.. of it
// gives exactly magic + code.  fp16 has 10 mantissa bits (magic 2^(10-P)), bf16 has 7 (magic 2^(7-P)).
template <int DT> __device__ __forceinline__ constexpr uint32_t magic16(int p) {
  return DT == DARTKV_F16 ? (uint32_t)(25 - p) << 10 : (uint32_t)(134 - p) << 7;
}

// One (scale, zero point) pair made ready for a run of code pairs whose codes sit at bit position PA or PB of
// their 16-bit halves.
// FP32 = false: fl(fl(code * scale) + zero) in the 16-bit metadata dtype DT, then cast to the cache dtype OUT;
// true: code * scale + zero in fp32, rounded once to the cache dtype
template <int DT, int OUT, bool FP32, int PA, int PB>
struct Restore {
  using H = Half2Ops<DT>;
  uint32_t s2, z2, nms_a, nms_b;
  float sf, zf;
  // fl(c * s) = fma(magic + c, s, -magic * s) needs magic * s exact: always in bf16; in fp16 magic 1024 could
  // overflow with scales above 63, so position 0 subtracts the magic first (one more packed operation)
  static constexpr bool kFmaA = !(DT == DARTKV_F16 && PA == 0), kFmaB = !(DT == DARTKV_F16 && PB == 0);
  __device__ __forceinline__ void init(uint16_t s, uint16_t z) {
    const uint32_t neg_a = (magic16<DT>(PA) * 0x00010001u) | 0x80008000u, neg_b = (magic16<DT>(PB) * 0x00010001u) | 0x80008000u;
    if (FP32) {
      sf = H::to_float(s);
      zf = H::to_float(z);
      nms_a = neg_a;
      nms_b = neg_b;
    } else {
      s2 = prmt(s, s, 0x1010);   // both halves
      z2 = prmt(z, z, 0x1010);
      nms_a = kFmaA ? H::mul(s2, neg_a) : neg_a;
      nms_b = kFmaB ? H::mul(s2, neg_b) : neg_b;
    }
  }
  // x: two codes, each OR-ed into the magic number of its half at position PA (SECOND = false) or PB
  template <bool SECOND>
  __device__ __forceinline__ uint32_t from_magic(uint32_t x) const {
    constexpr bool fma_form = SECOND ? kFmaB : kFmaA;
    const uint32_t nms = SECOND ? nms_b : nms_a;
    if (!FP32) {
      if (fma_form) return cast16<DT, OUT>(H::add(H::fma(x, s2, nms), z2));   // fl(fl(c * s) + z)
      return cast16<DT, OUT>(H::add(H::mul(H::add(x, nms), s2), z2));         // nms holds -magic here: x - magic = c exactly
    }
    float c0, c1;
    unpack16<DT>(H::add(x, nms), c0, c1);                    // nms holds -magic here: the codes, exactly
    return pack16<OUT>(__fmaf_rn(c0, sf, zf), __fmaf_rn(c1, sf, zf));
  }
  // two codes as exact floats
  __device__ __forceinline__ uint32_t from_codes(float c0, float c1) const {
    if (!FP32) return cast16<DT, OUT>(H::add(H::mul(pack16<DT>(c0, c1), s2), z2));   // small integers: exact in 16 bits
    return pack16<OUT>(__fmaf_rn(c0, sf, zf), __fmaf_rn(c1, sf, zf));
  }
};

// code positions per width: plain 2-bit codes sit at bits 2 and 6 of a byte in fp16 (magics 256 and 16) and at
// bits 0 and 4 in bf16; 4-bit codes at bit 4 in fp16 and bit 0 in bf16; two planes (a 4-bit code) at bits 0 and
// 4 in fp16 and at bit 0 only in bf16, whose 7 mantissa bits cannot hold a 4-bit code from bit 4 on
template <int DT, int OUT, bool FP32> using Restore2 = Restore<DT, OUT, FP32, DT == DARTKV_F16 ? 2 : 0, DT == DARTKV_F16 ? 6 : 4>;
template <int DT, int OUT, bool FP32> using Restore22 = Restore<DT, OUT, FP32, 0, DT == DARTKV_F16 ? 4 : 0>;
template <int DT, int OUT, bool FP32> using Restore4 = Restore<DT, OUT, FP32, DT == DARTKV_F16 ? 4 : 0, DT == DARTKV_F16 ? 4 : 0>;
template <int DT, int OUT, bool FP32> using Restore8 = Restore<DT, OUT, FP32, 0, 0>;

__device__ __forceinline__ constexpr uint32_t byte_pair_selector(int j) { return j | (j << 4) | ((4 + j) << 8) | ((4 + j) << 12); }

// Sixteen 2-bit codes of a word -> 8 registers, register i = elements (2i, 2i+1).
template <int DT, int OUT, bool FP32>
__device__ __forceinline__ void restore_2bit(uint32_t w, const Restore2<DT, OUT, FP32>& r, uint32_t (&out)[8]) {
  // byte j of `lo` / `hi` feeds the low / high halves: elements 4j and 4j+2 (low), 4j+1 and 4j+3 (high) at the same bits
  const uint32_t lo = DT == DARTKV_F16 ? w << 2 : w, hi = DT == DARTKV_F16 ? w : w >> 2;
  constexpr uint32_t mask_a = DT == DARTKV_F16 ? 0x000C000Cu : 0x00030003u, mask_b = mask_a << 4;
  const uint32_t m_a = magic16<DT>(DT == DARTKV_F16 ? 2 : 0) * 0x00010001u, m_b = magic16<DT>(DT == DARTKV_F16 ? 6 : 4) * 0x00010001u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t x = prmt(lo, hi, byte_pair_selector(j));
    out[2 * j] = r.template from_magic<false>(and_or(x, mask_a, m_a));
    out[2 * j + 1] = r.template from_magic<true>(and_or(x, mask_b, m_b));
  }
}

// Sixteen codes of two 2-bit planes (code = low | high << 2) -> 8 registers of adjacent elements.
template <int DT, int OUT, bool FP32>
__device__ __forceinline__ void restore_2plus2(uint32_t w, uint32_t high, const Restore22<DT, OUT, FP32>& r, uint32_t (&out)[8]) {
  const uint32_t t = w >> 2, hs = high << 2;
  const uint32_t m0 = magic16<DT>(0) * 0x00010001u, m4 = magic16<DT>(4) * 0x00010001u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t x = prmt(w, t, byte_pair_selector(j));       // low plane at bits 0 and 4 of both halves
    const uint32_t y = prmt(hs, high, byte_pair_selector(j));   // high plane of the same elements at bits 2 and 6
    out[2 * j] = r.template from_magic<false>(and_or(y, 0x000C000Cu, and_or(x, 0x00030003u, m0)));
    if (DT == DARTKV_F16) {
      out[2 * j + 1] = r.template from_magic<true>(and_or(y, 0x00C000C0u, and_or(x, 0x00300030u, m4)));
    } else {
      out[2 * j + 1] = r.template from_magic<true>(and_or(y >> 4, 0x000C000Cu, and_or(x >> 4, 0x00030003u, m0)));
    }
  }
}

// Eight 4-bit codes of a word -> 4 registers of adjacent elements.
template <int DT, int OUT, bool FP32>
__device__ __forceinline__ void restore_4bit(uint32_t w, const Restore4<DT, OUT, FP32>& r, uint32_t* out) {
  const uint32_t lo = DT == DARTKV_F16 ? w << 4 : w, hi = DT == DARTKV_F16 ? w : w >> 4;
  constexpr uint32_t mask = DT == DARTKV_F16 ? 0x00F000F0u : 0x000F000Fu;
  const uint32_t m = magic16<DT>(DT == DARTKV_F16 ? 4 : 0) * 0x00010001u;
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = r.template from_magic<false>(and_or(prmt(lo, hi, byte_pair_selector(j)), mask, m));
}

// Four 8-bit codes of a word -> 2 registers of adjacent elements.
template <int DT, int OUT, bool FP32>
__device__ __forceinline__ void restore_8bit(uint32_t w, const Restore8<DT, OUT, FP32>& r, uint32_t* out) {
  if (DT == DARTKV_F16) {
    // 1024 + code: the code byte is the low byte of the half, 0x64 its high byte
#pragma unroll
    for (int j = 0; j < 2; ++j)
      out[j] = r.template from_magic<false>(prmt(w, 0x64646464u, (2 * j) | (4 << 4) | ((2 * j + 1) << 8) | (4 << 12)));
  } else {
    // eight bits do not fit a bf16 mantissa: through fp32 (8388608 + code, exact)
    float c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      c[k] = __uint_as_float(prmt(w, 0x4B000000u, k | (4 << 4) | (5 << 8) | (7 << 12))) - 8388608.0f;
    out[0] = r.from_codes(c[0], c[1]);
    out[1] = r.from_codes(c[2], c[3]);
  }
}

// Keys of a staged chunk -> tile[channel][16 tokens] (rows of kKeyRow bytes).  KIND: 2, 4, 8 or 22 (two planes).
template <int DT, int MD, bool FP32, int KIND>
__device__ __forceinline__ void keys_to_tile(const uint8_t* st, const WideGeom& w, const uint8_t* slot_of, uint8_t* tile,
                                             int lane, int kg) {
  const uint16_t* kscale = reinterpret_cast<const uint16_t*>(st + w.k_scale);
  const uint16_t* kzero = reinterpret_cast<const uint16_t*>(st + w.k_zero);
#pragma unroll 2
  for (int r = 0; r < 4; ++r) {
    const int ch = lane + 32 * r;
    const uint16_t sc = kscale[ch * w.key_groups + kg], zr = kzero[ch * w.key_groups + kg];
    uint32_t out[8];
    if constexpr (KIND == 22) {
      Restore22<MD, DT, FP32> rs;
      rs.init(sc, zr);
      const uint32_t low = *reinterpret_cast<const uint32_t*>(st + ch * 4);
      const int slot = slot_of[ch];
      const uint32_t high = slot != 0xFF ? *reinterpret_cast<const uint32_t*>(st + w.k_high + slot * 4) : 0u;
      restore_2plus2<MD, DT, FP32>(low, high, rs, out);
    } else if constexpr (KIND == 2) {
      Restore2<MD, DT, FP32> rs;
      rs.init(sc, zr);
      restore_2bit<MD, DT, FP32>(*reinterpret_cast<const uint32_t*>(st + ch * 4), rs, out);
    } else if constexpr (KIND == 4) {
      Restore4<MD, DT, FP32> rs;
      rs.init(sc, zr);
      const uint2 words = *reinterpret_cast<const uint2*>(st + ch * 8);
      restore_4bit<MD, DT, FP32>(words.x, rs, out);
      restore_4bit<MD, DT, FP32>(words.y, rs, out + 4);
    } else {
      Restore8<MD, DT, FP32> rs;
      rs.init(sc, zr);
      const uint4 words = *reinterpret_cast<const uint4*>(st + ch * 16);
      restore_8bit<MD, DT, FP32>(words.x, rs, out);
      restore_8bit<MD, DT, FP32>(words.y, rs, out + 2);
      restore_8bit<MD, DT, FP32>(words.z, rs, out + 4);
      restore_8bit<MD, DT, FP32>(words.w, rs, out + 6);
    }
    uint4* row = reinterpret_cast<uint4*>(tile + ch * kKeyRow);
    row[0] = make_uint4(out[0], out[1], out[2], out[3]);
    row[1] = make_uint4(out[4], out[5], out[6], out[7]);
  }
}

// Values of a staged chunk -> tile[16 tokens][128 channels] (rows of kValueRow bytes).  A lane takes 64 channels
// of one token: 16 * BITS / 2 bytes, i.e. BITS / 2 pieces of 16 bytes.
template <int MD, int OUT, bool FP32, int BITS> struct ValueRestore;
template <int MD, int OUT, bool FP32> struct ValueRestore<MD, OUT, FP32, 2> { using type = Restore2<MD, OUT, FP32>; };
template <int MD, int OUT, bool FP32> struct ValueRestore<MD, OUT, FP32, 4> { using type = Restore4<MD, OUT, FP32>; };
template <int MD, int OUT, bool FP32> struct ValueRestore<MD, OUT, FP32, 8> { using type = Restore8<MD, OUT, FP32>; };

template <int DT, int MD, bool FP32, int BITS>
__device__ __forceinline__ void values_to_tile(const uint8_t* st, const WideGeom& w, uint8_t* tile, int lane, int vrb,
                                               int vgroups, int group_shift) {
  const int tok = lane & 15, half = lane >> 4;
  const uint8_t* codes = st + w.v_codes + tok * vrb + half * (vrb >> 1);
  const uint16_t* meta = reinterpret_cast<const uint16_t*>(st + w.v_meta) + tok * 2 * vgroups;
  uint8_t* row = tile + tok * kValueRow + half * 128;
  constexpr int kPieces = BITS / 2, kChannelsPerWord = 32 / BITS;
  typename ValueRestore<MD, DT, FP32, BITS>::type rs;
  // a 16-byte piece holds 64 / kPieces channels: one group, unless the groups are smaller than that (then every
  // word, which never straddles groups of 16 channels or more, looks its group up)
  const bool group_per_word = (64 / kPieces) >> group_shift;
#pragma unroll
  for (int p = 0; p < kPieces; ++p) {
    const int q = p;
    const uint4 words = *reinterpret_cast<const uint4*>(codes + 16 * q);
    const uint32_t ws[4] = {words.x, words.y, words.z, words.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int ch_local = (4 * q + k) * kChannelsPerWord;   // first channel of the word among this lane's 64
      if (k == 0 || group_per_word) {
        const int group = (64 * half + ch_local) >> group_shift;
        rs.init(meta[group], meta[vgroups + group]);
      }
      uint8_t* dst = row + ch_local * 2;
      if constexpr (BITS == 2) {
        uint32_t out[8];
        restore_2bit<MD, DT, FP32>(ws[k], rs, out);
        reinterpret_cast<uint4*>(dst)[0] = make_uint4(out[0], out[1], out[2], out[3]);
        reinterpret_cast<uint4*>(dst)[1] = make_uint4(out[4], out[5], out[6], out[7]);
      } else if constexpr (BITS == 4) {
        uint32_t out[4];
        restore_4bit<MD, DT, FP32>(ws[k], rs, out);
        *reinterpret_cast<uint4*>(dst) = make_uint4(out[0], out[1], out[2], out[3]);
      } else {
        uint32_t out[2];
        restore_8bit<MD, DT, FP32>(ws[k], rs, out);
        *reinterpret_cast<uint2*>(dst) = make_uint2(out[0], out[1]);
      }
    }
  }
}

template <int DT, int MD, bool FP32>
__global__ void __launch_bounds__(kThreads, 2) decode_wide_kernel(dartkv_cache_desc d, FastArgs a, WideGeom w) {
  using H = Half2Ops<DT>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  WideBlockSmem& bs = *reinterpret_cast<WideBlockSmem*>(smem_raw);
  uint8_t* warp_base = smem_raw + ((sizeof(WideBlockSmem) + 127) / 128) * 128;
  float* warp_out = reinterpret_cast<float*>(warp_base);   // merge buffer: aliases the warps' streaming memory
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int rep = a.query_heads / d.kv_heads;

  if ((int)blockIdx.x >= a.stream_blocks) {
    const int bh = blockIdx.x - a.stream_blocks;
    dense_block<DT, MD>(d, a, bs, warp_out, bh);
    __syncthreads();
    block_merge(a, bs, warp_out, bh / d.kv_heads, bh % d.kv_heads, rep, 0);
    return;
  }

  const int sb = blockIdx.x;
  int unit = (int)((int64_t)sb * a.units / a.stream_blocks);
  const int unit_end = (int)((int64_t)(sb + 1) * a.units / a.stream_blocks);
  const int pair = warp >> 1, hf = warp & 1;
  uint8_t* mine = warp_base + (size_t)warp * w.warp_bytes;
  uint8_t* stage_mem = mine;                               // [2][stage_bytes]
  uint8_t* tile = mine + 2 * w.stage_bytes;                // kTileBytes
  uint8_t* slot_of = tile + kTileBytes;                    // [128] promoted slot of a channel, 0xFF: none
  const int k_end = d.state[2], v_end = d.state[3], sink_filled = d.state[4];
  const int fast_end = fast_range_end(d.sink_tokens, d.page_size, k_end, v_end, sink_filled);
  const int total_pages = fast_end > d.sink_tokens ? (fast_end - d.sink_tokens) / 128 : 0;
  const float scale2 = a.scale * kLog2e;
  const int vrb = d.value_row_bytes, vgroups = d.value_groups, vbits = d.value_bits;
  const int vg_shift = 31 - __clz(d.value_group), kg_shift = 31 - __clz(d.key_group);   // group sizes are powers of two
  const int key_row_bytes = w.key_kind == 22 ? 32 : 16 * w.key_kind;
  const int promoted = w.key_kind == 22 ? d.promoted : 0;

  while (unit < unit_end) {
    const int bh = unit / a.quads;
    const int quad_begin = unit - bh * a.quads;
    const int quad_count = min(a.quads - quad_begin, unit_end - unit);
    unit += quad_count;
    const int b = bh / d.kv_heads, hkv = bh % d.kv_heads;
    // tokens before the row's first live one get no weight: whole pages of them are not even fetched
    const int row_first = a.row_start ? max(a.row_start[b], 0) : 0;
    const int p_begin = max(4 * quad_begin, row_first > d.sink_tokens ? (row_first - d.sink_tokens) >> 7 : 0);
    const int p_end = min(4 * (quad_begin + quad_count), total_pages);
    const int pg0 = p_begin + pair;
    const int chunks = pg0 < p_end ? 4 * ((p_end - pg0 + 3) / 4) : 0;   // 4 chunks of 16 tokens per page of this pair

    // chunk idx of this warp: page pg0 + 4 * (idx / 4), page tokens 64 * hf + 16 * (idx % 4) ..
    auto issue = [&](int idx) {
      if (idx < chunks) {
        const int pg = pg0 + 4 * (idx >> 2), t0 = 64 * hf + 16 * (idx & 3);
        uint8_t* st = stage_mem + (idx & 1) * w.stage_bytes;
        const uint8_t* blob = d.k_pages + ((int64_t)bh * d.max_key_pages + pg) * d.key_page_bytes;
        const int chunk_off = t0 * (w.key_kind == 22 ? 2 : w.key_kind) / 8;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int ch = lane + 32 * r;
          const uint8_t* src = blob + ch * key_row_bytes + chunk_off;
          uint8_t* dst = st + ch * w.key_chunk;
          if (w.key_chunk == 4) cp_async4(dst, src);
          else if (w.key_chunk == 8) cp_async8(dst, src);
          else cp_async16(dst, src);
        }
        if (promoted) {
          for (int slot = lane; slot < promoted; slot += 32)
            cp_async4(st + w.k_high + slot * 4, blob + d.key_off_high + slot * 32 + chunk_off);
          for (int piece = lane; piece * 4 < promoted; piece += 32)
            cp_async16(st + w.k_index + piece * 16, blob + d.key_off_index + piece * 16);
        }
        for (int piece = lane; piece * 16 < w.key_meta_bytes; piece += 32) {
          cp_async16(st + w.k_scale + piece * 16, blob + d.key_off_scale + piece * 16);
          cp_async16(st + w.k_zero + piece * 16, blob + d.key_off_zero + piece * 16);
        }
        const int64_t vrow = (int64_t)bh * d.max_value_tokens + (int64_t)pg * 128 + t0;
        for (int piece = lane; piece < vrb; piece += 32)       // 16 rows of vrb bytes = vrb pieces of 16 bytes
          cp_async16(st + w.v_codes + piece * 16, d.v_codes + vrow * vrb + piece * 16);
        if (lane < 4 * vgroups)                                 // 16 rows of (scale row, zero row): 64 * groups bytes
          cp_async16(st + w.v_meta + lane * 16,
                     reinterpret_cast<const uint8_t*>(d.v_meta) + vrow * (4 * vgroups) + lane * 16);
      }
      cp_async_commit();   // an empty group keeps the group count in step with the chunk index
    };
    issue(0);
    issue(1);

    // A operand of the logits: rows = query heads (rows rep.. are zero); kept in shared memory, the registers
    // are needed by the accumulators
    for (int i = tid; i < 8 * 128; i += kThreads) {
      const int r = i >> 7, ch = i & 127;
      bs.q16[r][ch] = r < rep ? reinterpret_cast<const uint16_t*>(a.q)[((int64_t)b * a.query_heads + hkv * rep + r) * 128 + ch] : (uint16_t)0;
    }
    __syncthreads();
    const uint16_t* q_lane = &bs.q16[g][2 * c];

    float o_acc[16][4];   // [n-tile: channels 8n..8n+7][c-reg]: (head g, channels 8n+2c, +1) from the high (0,1) / low (2,3) parts of P
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;   // head g, log2 domain; l_run: this lane's tokens only

    for (int idx = 0; idx < chunks; ++idx) {
      cp_async_wait<1>();
      __syncwarp();
      const uint8_t* st = stage_mem + (idx & 1) * w.stage_bytes;
      const int pg = pg0 + 4 * (idx >> 2), t0 = 64 * hf + 16 * (idx & 3);
      const int kg = t0 >> kg_shift;

      // ---- keys of the chunk -> tile[channel][16 tokens]
      if (promoted) {
        reinterpret_cast<uint32_t*>(slot_of)[lane] = 0xFFFFFFFFu;
        __syncwarp();
        const int32_t* index = reinterpret_cast<const int32_t*>(st + w.k_index);
        for (int k = lane; k < promoted; k += 32) slot_of[index[k] & 127] = (uint8_t)k;
        __syncwarp();
      }
      switch (w.key_kind) {
        case 22: keys_to_tile<DT, MD, FP32, 22>(st, w, slot_of, tile, lane, kg); break;
        case 2: keys_to_tile<DT, MD, FP32, 2>(st, w, slot_of, tile, lane, kg); break;
        case 4: keys_to_tile<DT, MD, FP32, 4>(st, w, slot_of, tile, lane, kg); break;
        default: keys_to_tile<DT, MD, FP32, 8>(st, w, slot_of, tile, lane, kg); break;
      }
      __syncwarp();

      // ---- S^T[head][token] = q K^T: two n-tiles of 8 tokens, 8 contraction steps of 16 channels
      float s_acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
      {
        // matrix m of an ldmatrix.x4: channels 16ks + 8(m&1).., tokens 8(m>>1)..; lane l addresses row l%8 of matrix l/8
        const uint8_t* lane_row = tile + (8 * ((lane >> 3) & 1) + (lane & 7)) * kKeyRow + 16 * (lane >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t kb[4];
          ldmatrix_x4_trans(kb, lane_row + 16 * ks * kKeyRow);
          const uint32_t qa0 = *reinterpret_cast<const uint32_t*>(q_lane + 16 * ks);
          const uint32_t qa1 = *reinterpret_cast<const uint32_t*>(q_lane + 16 * ks + 8);
          H::mma(s_acc[0], qa0, 0u, qa1, 0u, kb[0], kb[1]);
          H::mma(s_acc[1], qa0, 0u, qa1, 0u, kb[2], kb[3]);
        }
      }
      __syncwarp();   // every lane has its logits: the tile may take the values

      // ---- values of the chunk -> tile[16 tokens][128 channels]
      switch (vbits) {
        case 2: values_to_tile<DT, MD, FP32, 2>(st, w, tile, lane, vrb, vgroups, vg_shift); break;
        case 4: values_to_tile<DT, MD, FP32, 4>(st, w, tile, lane, vrb, vgroups, vg_shift); break;
        default: values_to_tile<DT, MD, FP32, 8>(st, w, tile, lane, vrb, vgroups, vg_shift); break;
      }
      __syncwarp();
      issue(idx + 2);   // the stage has been read by every lane

      // ---- online softmax of head g over the chunk's 16 tokens: this lane holds tokens 2c, 2c+1, 8+2c, 8+2c+1
      float sv[4] = {s_acc[0][0] * scale2, s_acc[0][1] * scale2, s_acc[1][0] * scale2, s_acc[1][1] * scale2};
      const int mask_below = row_first - (d.sink_tokens + 128 * pg + t0);
      if (mask_below > 0) {   // the page that holds the row's first live token: the tokens before it drop out
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (8 * (i >> 1) + 2 * c + (i & 1) < mask_below) sv[i] = -INFINITY;
      }
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);
      const float m_ref = m_new == -INFINITY ? 0.0f : m_new;   // nothing live yet: every weight below comes out zero
      const float alpha = fast_exp2(m_run - m_ref);
      m_run = m_new;
      uint32_t p_hi[2], p_lo[2];
      float psum = 0.0f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = fast_exp2(sv[2 * n] - m_ref), p1 = fast_exp2(sv[2 * n + 1] - m_ref);
        psum += p0 + p1;
        const uint16_t h0 = H::from_float(p0), h1 = H::from_float(p1);
        p_hi[n] = (uint32_t)h0 | ((uint32_t)h1 << 16);
        p_lo[n] = (uint32_t)H::from_float(p0 - H::to_float(h0)) | ((uint32_t)H::from_float(p1 - H::to_float(h1)) << 16);
      }
      l_run = l_run * alpha + psum;
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int n = 0; n < 16; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) o_acc[n][i] *= alpha;
      }

      // ---- O[head][channel] += P V: A rows 0..7 carry the high parts of P (head g), rows 8..15 the low parts
      {
        // matrix m of an ldmatrix.x4: tokens 8(m&1).., channels 16j + 8(m>>1)..
        const uint8_t* lane_row = tile + (8 * ((lane >> 3) & 1) + (lane & 7)) * kValueRow + 16 * (lane >> 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, lane_row + 32 * j);
          H::mma(o_acc[2 * j], p_hi[0], p_lo[0], p_hi[1], p_lo[1], vb[0], vb[1]);
          H::mma(o_acc[2 * j + 1], p_hi[0], p_lo[0], p_hi[1], p_lo[1], vb[2], vb[3]);
        }
      }
      __syncwarp();   // the tile is free for the next chunk's keys
    }
    cp_async_wait<0>();

    // ---- hand the warp state to the block merge
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    __syncthreads();   // every warp is done streaming: its memory becomes the merge buffer
    if (c == 0 && g < 4) { bs.merge_m[warp][g] = m_run; bs.merge_l[warp][g] = l_run; }
    if (g < 4) {
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        float2 v = make_float2(o_acc[n][0] + o_acc[n][2], o_acc[n][1] + o_acc[n][3]);
        *reinterpret_cast<float2*>(&warp_out[(warp * 4 + g) * 128 + 8 * n + 2 * c]) = v;
      }
    }
    __syncthreads();
    block_merge(a, bs, warp_out, b, hkv, rep,
                1 + sb - dartkv_block_of_unit((int64_t)bh * a.quads, a.stream_blocks, a.units));
    __syncthreads();   // the merge buffer is streaming memory again
  }
}

static WideGeom wide_geometry(const dartkv_cache_desc* d) {
  WideGeom w{};
  const bool mixed = d->key_mode == DARTKV_MIXED_PAGE;
  w.key_kind = mixed ? 22 : d->key_bits;
  w.key_groups = d->page_size / d->key_group;
  w.key_chunk = mixed ? 4 : 2 * d->key_bits;
  w.key_meta_bytes = 128 * w.key_groups * 2;
  int off = 128 * w.key_chunk;
  w.k_high = off;
  if (mixed) off += (d->promoted * 4 + 15) / 16 * 16;
  w.k_index = off;
  if (mixed) off += (d->promoted * 4 + 15) / 16 * 16;
  w.k_scale = off;
  off += w.key_meta_bytes;
  w.k_zero = off;
  off += w.key_meta_bytes;
  w.v_codes = off;
  off += 16 * d->value_row_bytes;
  w.v_meta = off;
  off += 64 * d->value_groups;
  w.stage_bytes = off;
  w.warp_bytes = 2 * w.stage_bytes + kTileBytes + 128;
  return w;
}

static size_t wide_smem_bytes(const WideGeom& w) {
  const size_t streaming = (size_t)kWarps * w.warp_bytes;
  const size_t merge = (size_t)(kWarps * 4 * 128 + kWarps * 64) * sizeof(float);   // warp states + dense-block tables
  return (sizeof(WideBlockSmem) + 127) / 128 * 128 + (streaming > merge ? streaming : merge);
}

using WideKernel = void (*)(dartkv_cache_desc, FastArgs, WideGeom);
template <int DT>
static WideKernel wide_variant_of(int md, bool fp32) {
  if (md == DARTKV_BF16) return fp32 ? decode_wide_kernel<DT, DARTKV_BF16, true> : decode_wide_kernel<DT, DARTKV_BF16, false>;
  return fp32 ? decode_wide_kernel<DT, DARTKV_F16, true> : decode_wide_kernel<DT, DARTKV_F16, false>;
}
static WideKernel wide_variant(int dtype, int md, bool fp32) {
  return dtype == DARTKV_BF16 ? wide_variant_of<DARTKV_BF16>(md, fp32) : wide_variant_of<DARTKV_F16>(md, fp32);
}

}  // namespace

int dartkv_decode_wide_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads) {
  if (d->head_dim != 128 || d->page_size != 128 || !d->regular_pages) return 0;
  if (d->dtype != DARTKV_F16 && d->dtype != DARTKV_BF16) return 0;
  if ((d->md_dtype != DARTKV_F16 && d->md_dtype != DARTKV_BF16) || q_dtype != d->dtype) return 0;
  if (d->key_group < 16 || d->key_group > 128 || (d->key_group & (d->key_group - 1))) return 0;
  if (d->value_group < 16 || d->value_group > 128 || (d->value_group & (d->value_group - 1))) return 0;
  if (d->value_bits != 2 && d->value_bits != 4 && d->value_bits != 8) return 0;
  if (d->key_mode == DARTKV_QUANTIZED_PAGE && d->key_bits != 2 && d->key_bits != 4 && d->key_bits != 8) return 0;
  if (d->key_mode == DARTKV_MIXED_PAGE && (d->promoted < 1 || d->promoted > 128)) return 0;
  if (d->key_page_bytes % 16) return 0;
  if (query_heads % d->kv_heads || query_heads / d->kv_heads > 4) return 0;
  if (d->max_value_tokens % 8) return 0;   // keeps every chunk of value metadata 16-byte aligned
  if ((uintptr_t)d->k_pages % 16 || (uintptr_t)d->v_codes % 16 || (uintptr_t)d->v_meta % 16) return 0;
  return wide_smem_bytes(wide_geometry(d)) <= 227 * 1024 ? 1 : 0;
}

// resident blocks per SM (1 or 2): the work split counts on it
int dartkv_decode_wide_blocks_per_sm(const dartkv_cache_desc* d) {
  return 2 * (wide_smem_bytes(wide_geometry(d)) + 1024) <= 228 * 1024 ? 2 : 1;
}

int dartkv_decode_wide_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
                              int flavour, int quads, int stream_blocks, long long units, int total_splits,
                              float* part_m, float* part_l, float* part_acc, int* status, const int32_t* row_start,
                              cudaStream_t stream) {
  (void)q_dtype;
  FastArgs a{query, query_heads, scale, flavour, quads, stream_blocks, units, total_splits, part_m, part_l, part_acc, status,
             row_start};
  const WideGeom w = wide_geometry(d);
  const size_t smem = wide_smem_bytes(w);
  dim3 grid(stream_blocks + d->batch * d->kv_heads);
  {
    // the shared-memory opt-in is per device and per kernel: ask once per device
    static std::atomic<bool> ready[64];
    int device = 0;
    DARTKV_CUDA_OK(cudaGetDevice(&device));
    if (device < 0 || device >= 64 || !ready[device].load(std::memory_order_acquire)) {
      for (int dt : {DARTKV_BF16, DARTKV_F16})
        for (int md : {DARTKV_BF16, DARTKV_F16})
          for (int fp32 : {0, 1})
            DARTKV_CUDA_OK(cudaFuncSetAttribute(wide_variant(dt, md, fp32 != 0), cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      if (device >= 0 && device < 64) ready[device].store(true, std::memory_order_release);
    }
  }
  wide_variant(d->dtype, d->md_dtype, flavour == DARTKV_DEQUANT_FP32)<<<grid, kThreads, smem, stream>>>(*d, a, w);
  DARTKV_LAUNCH_OK("decode_wide_kernel");
  return DARTKV_OK;
}
