// Pieces shared by the tensor-core decode kernels (decode_fast.cu: per-op rounded dequantization;
// decode_fused32.cu: unrounded fp32 dequantization): block geometry, the staged page layout, the block
// that handles dense tokens, and the block-level merge of the warps' online-softmax states.
#pragma once

#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int kPairs = 4;
constexpr int kWarps = 2 * kPairs;
constexpr int kThreads = kWarps * 32;
constexpr int kPageBytesK = 5760;
constexpr int kValueCodes = 4096;
constexpr int kStageBytes = 10880;            // key blob (<= 5760) | value codes 4096 | value metadata (<= 1024)
constexpr int kOffVCodes = kPageBytesK;       // 5760
constexpr int kOffVMeta = kPageBytesK + kValueCodes;  // 9856
constexpr int kPStride = 72;                  // 16-bit elements per (plane, head) row of a warp's probability tile
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void pair_barrier(int pair) {
  asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory");
}

struct FastArgs {
  const void* q;
  int query_heads;
  float scale;
  int flavour;
  // Work split: one unit = four consecutive pages of one (batch, kv head) (one page per warp pair); the units of
  // all (batch, kv head) rows, `quads` each, are dealt out evenly to `stream_blocks` blocks, so a block may finish
  // one row and start the next.  Partial slot 0 of a row belongs to its dense-token block, slot 1 + k to the
  // k-th stream block that touches the row.
  int quads, stream_blocks;
  long long units;
  int total_splits;
  float* part_m;
  float* part_l;
  float* part_acc;
  int* status;
  // optional [batch] first live token of every batch row (left padding): tokens before it get no weight
  const int32_t* row_start;
};

__host__ __device__ __forceinline__ int fast_range_end(int sink_tokens, int page_size, int k_end, int v_end,
                                                       int sink_filled) {
  int packed = min(k_end, v_end);
  if (packed <= sink_tokens) return sink_filled;
  return sink_tokens + (packed - sink_tokens) / page_size * page_size;
}

template <int DT>
__device__ __forceinline__ float rnd16(float x) { return Half2Ops<DT>::to_float(Half2Ops<DT>::from_float(x)); }

// code * scale + zero the way the chosen flavour rounds it: per-op in the metadata dtype MD and then cast to the
// cache dtype DT, or fp32 with one rounding to DT, or not rounded at all
template <int DT, int MD>
__device__ __forceinline__ float restore16(float code, float scale, float zero, int flavour) {
  if (flavour == DARTKV_DEQUANT_FUSED) return __fmaf_rn(code, scale, zero);
  if (flavour == DARTKV_DEQUANT_FP32) return rnd16<DT>(__fmaf_rn(code, scale, zero));
  const float md = rnd16<MD>(__fadd_rn(rnd16<MD>(__fmul_rn(code, scale)), zero));
  return MD == DT ? md : rnd16<DT>(md);
}

// ------------------------------------------------------------------------------------------------
// dense tokens (sink prefix, unpacked tail, and tokens packed on one side only).  Tokens whose key and value rows
// are both dense go through 16-token tiles: logits by m16n8k16 MMAs straight from the rows, probabilities
// through a small shared table, P.V on CUDA cores with four channels per lane.  Tokens packed on one side only
// (Kitty lifecycle) take one warp per token, four channels per lane, fp32 math.
// BS: the kernel's block-level shared struct (needs slot_map[128], merge_m / merge_l [kWarps][4])
// MD: metadata dtype of the packed tokens (the tensor-core kernels for 2-bit pages only take MD = DT)
template <int DT, int MD = DT, class BS>
__device__ void dense_block(const dartkv_cache_desc& d, const FastArgs& a, BS& bs, float* warp_out, int bh) {
  using H = Half2Ops<DT>;
  using HM = Half2Ops<MD>;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rep = a.query_heads / d.kv_heads;
  const int seen = d.state[0], pages = d.state[1], k_end = d.state[2], v_end = d.state[3], sink_filled = d.state[4];
  const int fast_end = fast_range_end(d.sink_tokens, d.page_size, k_end, v_end, sink_filled);
  const int b = bh / d.kv_heads, h = bh % d.kv_heads;
  float q[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int i = 0; i < 4; ++i)
      q[r][i] = r < rep ? load_f(a.q, d.dtype, ((int64_t)b * a.query_heads + h * rep + r) * 128 + lane * 4 + i) : 0.0f;
  float m[4], l[4], acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[r][i] = 0.0f;
  }
  const float scale2 = a.scale * kLog2e;
  const bool fused = a.flavour != DARTKV_DEQUANT_PER_OP;   // a page the other side cuts falls back to per-op
  // geometry of the packed rows (any code width; the key rows of a page are packed continuously over its groups)
  const int key_bits = d.key_mode == DARTKV_MIXED_PAGE ? 2 : d.key_bits;
  const int key_row_bytes = d.page_size * key_bits / 8;
  const int key_groups = d.page_size / d.key_group;
  const uint32_t key_mask = (1u << key_bits) - 1u, value_mask = (1u << d.value_bits) - 1u;
  // MMA operand of the tiles: column n = g is query head g (zero past the last head), two channels per register
  const int g = lane >> 2, c = lane & 3;
  uint32_t qb[8][2];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
#pragma unroll
    for (int j = 0; j < 2; ++j)
      qb[ks][j] = g < rep ? *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(a.q) +
                                ((int64_t)b * a.query_heads + h * rep + g) * 128 + 16 * ks + 8 * j + 2 * c)
                          : 0u;
  int tile_counter = 0;
  float* ptab = warp_out + 4096 + warp * 64;   // this warp's [16 tokens][4 heads] probabilities, beyond the merge buffer
  // segments: [0, sink_filled) then [fast_end, seen) cut at key page boundaries
  int t = a.row_start ? min(max(a.row_start[b], 0), seen) : 0;
#ifdef DENSE_SKIP
  t = seen;
#endif
  while (t < seen) {
    if (t >= sink_filled && t < fast_end) { t = fast_end; continue; }
    int seg_end, kind;
    bool fused_key = fused;
    const uint8_t* page = nullptr;
    int page_first = 0;
    if (t < sink_filled) { kind = 0; seg_end = sink_filled; }
    else if (t < k_end) {
      kind = 1;
      int pg = (t - d.sink_tokens) / d.page_size;   // pages are regular on this path
      page_first = d.sink_tokens + pg * d.page_size;
      seg_end = min(seen, page_first + d.page_size);
      page = d.k_pages + ((int64_t)bh * d.max_key_pages + pg) * d.key_page_bytes;
      // a key page that the end of the packed values cuts is materialized by the reference with its per-op
      // dequantization (src/dart/cache.py:557-560); only whole pages reach its fp32 kernels
      fused_key = fused && !(page_first < v_end && v_end < page_first + d.page_size);
      __syncthreads();
      if (tid < 128) bs.slot_map[tid] = -1;
      __syncthreads();
      if (d.key_mode == DARTKV_MIXED_PAGE && tid < d.promoted) {
        int ch = reinterpret_cast<const int32_t*>(page + d.key_off_index)[tid];
        if (ch >= 0 && ch < 128) bs.slot_map[ch] = tid;
      }
      __syncthreads();
    } else { kind = 2; seg_end = seen; }
    (void)pages;
    // dense rows of the next token are requested before the current one is consumed
    auto dense_ptr = [&](const void* sink, const void* ring, int tok) -> const uint16_t* {
      return tok < sink_filled
          ? reinterpret_cast<const uint16_t*>(sink) + ((int64_t)bh * d.sink_tokens + tok) * 128
          : reinterpret_cast<const uint16_t*>(ring) + ((int64_t)bh * d.ring_tokens + (tok % d.ring_tokens)) * 128;
    };
    auto dense_row = [&](const void* sink, const void* ring, int tok) -> uint2 {
      return *reinterpret_cast<const uint2*>(dense_ptr(sink, ring, tok) + lane * 4);
    };
    auto value_dense = [&](int tok) { return !(tok >= sink_filled && tok < v_end); };
    // [tile_from, seg_end): key and value rows both dense -> tiles; [t, tile_from): per-token path below
    const int tile_from = kind == 1 ? seg_end : (kind == 0 ? t : min(seg_end, max(t, v_end)));
    for (int tile = tile_from; tile < seg_end; tile += 16) {
      if ((tile_counter++ & (kWarps - 1)) != warp) continue;   // tiles of all segments go round the warps
      const int last = seg_end - 1;
      const uint8_t* k0 = reinterpret_cast<const uint8_t*>(dense_ptr(d.k_sink, d.k_ring, min(tile + g, last))) + 4 * c;
      const uint8_t* k1 = reinterpret_cast<const uint8_t*>(dense_ptr(d.k_sink, d.k_ring, min(tile + g + 8, last))) + 4 * c;
      float s_acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        H::mma(s_acc, *reinterpret_cast<const uint32_t*>(k0 + 32 * ks), *reinterpret_cast<const uint32_t*>(k1 + 32 * ks),
               *reinterpret_cast<const uint32_t*>(k0 + 32 * ks + 16), *reinterpret_cast<const uint32_t*>(k1 + 32 * ks + 16),
               qb[ks][0], qb[ks][1]);
      // the value rows of the whole tile are requested now; the softmax below hides their latency
      uint2 v_rows[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v_rows[j] = dense_row(d.v_sink, d.v_ring, min(tile + j, last));
      // s_acc: tokens tile+g (0,1) and tile+g+8 (2,3), heads 2c and 2c+1
      const bool live0 = tile + g < seg_end, live1 = tile + g + 8 < seg_end;
      float sv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sv[i] = ((i < 2) ? live0 : live1) ? s_acc[i] * scale2 : -INFINITY;
      float mt0 = fmaxf(sv[0], sv[2]), mt1 = fmaxf(sv[1], sv[3]);
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, off));
        mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, off));
      }
      // every lane needs the tile maxima of heads 0..3: heads 0,1 sit in lanes c = 0, heads 2,3 in lanes c = 1
      float m_tile[4];
      m_tile[0] = __shfl_sync(0xffffffffu, mt0, 0); m_tile[1] = __shfl_sync(0xffffffffu, mt1, 0);
      m_tile[2] = __shfl_sync(0xffffffffu, mt0, 1); m_tile[3] = __shfl_sync(0xffffffffu, mt1, 1);
      float alpha[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float m_new = fmaxf(m[r], m_tile[r]);
        alpha[r] = fast_exp2(m[r] - m_new);
        m[r] = m_new;
      }
      if (c < 2) {
        const float ma = c == 0 ? m[0] : m[2], mb = c == 0 ? m[1] : m[3];
        *reinterpret_cast<float2*>(ptab + 4 * g + 2 * c) = make_float2(fast_exp2(sv[0] - ma), fast_exp2(sv[1] - mb));
        *reinterpret_cast<float2*>(ptab + 4 * (g + 8) + 2 * c) = make_float2(fast_exp2(sv[2] - ma), fast_exp2(sv[3] - mb));
      }
      __syncwarp();
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        l[r] *= alpha[r];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][i] *= alpha[r];
      }
      // tokens past the end of the segment have probability zero
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint2 v_raw = v_rows[j];
        const float4 pj = *reinterpret_cast<const float4*>(ptab + 4 * j);
        const float vv[4] = {H::to_float((uint16_t)(v_raw.x & 0xFFFF)), H::to_float((uint16_t)(v_raw.x >> 16)),
                             H::to_float((uint16_t)(v_raw.y & 0xFFFF)), H::to_float((uint16_t)(v_raw.y >> 16))};
        const float pr[4] = {pj.x, pj.y, pj.z, pj.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          l[r] += pr[r];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[r][i] = fmaf(pr[r], vv[i], acc[r][i]);
        }
      }
      __syncwarp();   // the table is rewritten by the next tile
    }
    const int seg_stop = seg_end;
    seg_end = tile_from;   // what is left for the per-token path
    uint2 k_next = make_uint2(0, 0), v_next = make_uint2(0, 0);
    {
      const int first = t + warp;
      if (first < seg_end) {
        if (kind != 1) k_next = dense_row(d.k_sink, d.k_ring, first);
        if (value_dense(first)) v_next = dense_row(d.v_sink, d.v_ring, first);
      }
    }
    for (int tok = t + warp; tok < seg_end; tok += kWarps) {
      const uint2 k_raw = k_next, v_raw = v_next;
      const int nxt = tok + kWarps;
      if (nxt < seg_end) {
        if (kind != 1) k_next = dense_row(d.k_sink, d.k_ring, nxt);
        if (value_dense(nxt)) v_next = dense_row(d.v_sink, d.v_ring, nxt);
      }
      float kv[4];
      if (kind == 1) {
        const int j = tok - page_first;
        const int bit = j * key_bits, kg = j / d.key_group;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ch = lane * 4 + i;
          uint32_t code = (page[ch * key_row_bytes + (bit >> 3)] >> (bit & 7)) & key_mask;
          const int slot = bs.slot_map[ch];
          if (slot >= 0) code |= ((page[d.key_off_high + slot * key_row_bytes + (bit >> 3)] >> (bit & 7)) & 3u) << 2;
          const float s = HM::to_float(reinterpret_cast<const uint16_t*>(page + d.key_off_scale)[ch * key_groups + kg]);
          const float z = HM::to_float(reinterpret_cast<const uint16_t*>(page + d.key_off_zero)[ch * key_groups + kg]);
          kv[i] = restore16<DT, MD>((float)code, s, z, fused_key ? a.flavour : DARTKV_DEQUANT_PER_OP);
        }
      } else {
        kv[0] = H::to_float((uint16_t)(k_raw.x & 0xFFFF)); kv[1] = H::to_float((uint16_t)(k_raw.x >> 16));
        kv[2] = H::to_float((uint16_t)(k_raw.y & 0xFFFF)); kv[3] = H::to_float((uint16_t)(k_raw.y >> 16));
      }
      float s[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float dot = q[r][0] * kv[0];
        dot = fmaf(q[r][1], kv[1], dot);
        dot = fmaf(q[r][2], kv[2], dot);
        dot = fmaf(q[r][3], kv[3], dot);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        s[r] = dot * scale2;
      }
      // value row of the same token
      float vv[4];
      if (!value_dense(tok)) {
        const int64_t row = (int64_t)bh * d.max_value_tokens + (tok - d.sink_tokens);
        // the lane's four channels: one byte of 2-bit codes, two of 4-bit codes, four of 8-bit codes
        const uint8_t* packed = d.v_codes + row * d.value_row_bytes + lane * d.value_bits / 2;
        uint32_t word = packed[0];
        if (d.value_bits >= 4) word |= (uint32_t)packed[1] << 8;
        if (d.value_bits == 8) word |= (uint32_t)packed[2] << 16 | (uint32_t)packed[3] << 24;
        const int g = (lane * 4) / d.value_group;
        const uint16_t* meta = reinterpret_cast<const uint16_t*>(d.v_meta) + row * 2 * d.value_groups;
        const float sc = HM::to_float(meta[g]), z = HM::to_float(meta[d.value_groups + g]);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          vv[i] = restore16<DT, MD>((float)((word >> (d.value_bits * i)) & value_mask), sc, z, a.flavour);
      } else {
        vv[0] = H::to_float((uint16_t)(v_raw.x & 0xFFFF)); vv[1] = H::to_float((uint16_t)(v_raw.x >> 16));
        vv[2] = H::to_float((uint16_t)(v_raw.y & 0xFFFF)); vv[3] = H::to_float((uint16_t)(v_raw.y >> 16));
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float m_new = fmaxf(m[r], s[r]);
        const float alpha = fast_exp2(m[r] - m_new);
        const float p = fast_exp2(s[r] - m_new);
        m[r] = m_new;
        l[r] = l[r] * alpha + p;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][i] = acc[r][i] * alpha + p * vv[i];
      }
    }
    t = seg_stop;
  }
  // hand the warp state to the block merge: acc in channel order
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (lane == 0) { bs.merge_m[warp][r] = m[r]; bs.merge_l[warp][r] = l[r]; }
#pragma unroll
    for (int i = 0; i < 4; ++i) warp_out[(warp * 4 + r) * 128 + lane * 4 + i] = acc[r][i];
  }
}

// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// Block merge of the eight warp states: thread = (channel, head parity); partials leave in natural-log units.
template <class BS>
__device__ __forceinline__ void block_merge(const FastArgs& a, const BS& bs, const float* warp_out, int b, int hkv, int rep,
                                            int slot) {
  const int tid = threadIdx.x;
  const int ch = tid & 127;
  for (int r = tid >> 7; r < rep; r += kThreads / 128) {
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, bs.merge_m[w][r]);
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = bs.merge_m[w][r];
      if (mw != -INFINITY) {
        const float wgt = fast_exp2(mw - m);
        l += bs.merge_l[w][r] * wgt;
        acc += warp_out[(w * 4 + r) * 128 + ch] * wgt;
      }
    }
    const int64_t row = ((int64_t)b * a.query_heads + hkv * rep + r) * a.total_splits + slot;
    if (ch == 0) {
      a.part_m[row] = m == -INFINITY ? -INFINITY : m * 0.6931471805599453f;
      a.part_l[row] = l;
    }
    a.part_acc[row * 128 + ch] = acc;
  }
}

}  // namespace
