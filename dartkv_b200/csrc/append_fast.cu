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

template <int DT>
__device__ __forceinline__ uint32_t code_of(float x, float mn, float scale, float qmax) {
  float shifted = rnd<DT>(__fsub_rn(x, mn));
  float ratio = rnd<DT>(__fdiv_rn(shifted, scale));
  return (uint32_t)fminf(fmaxf(rintf(ratio), 0.0f), qmax);
}

// KBITS: 0 = mixed 2+2-bit keys, else uniform keys with KBITS bits
template <int DT, int KBITS>
__global__ void __launch_bounds__(128) fast_key_pages_kernel(dartkv_cache_desc d, RowSource src, int first_slot,
                                                             int num_pages, int page_token_start,
                                                             const int32_t* __restrict__ indices, int32_t* nonfinite) {
  using E = Elem<DT>;
  using T = typename E::type;
  __shared__ __align__(16) T s_page[kP * kD];
  __shared__ float s_score[kD];
  const int bh = blockIdx.x, pg = blockIdx.y, c = threadIdx.x;
  const int t0 = page_token_start + pg * kP;
  // stage the page: 2048 16-byte pieces, 16 per thread
  for (int i = c; i < kP * 16; i += 128) {
    int r = i >> 4, piece = i & 15;
    cp_async16(reinterpret_cast<char*>(s_page) + r * 256 + piece * 16,
               reinterpret_cast<const char*>(src.row(bh, t0 + r)) + piece * 16);
  }
  cp_async_wait_all();
  __syncthreads();

  uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + first_slot + pg) * d.key_page_bytes;
  float mn = INFINITY, mx = -INFINITY;
  double asum = 0.0;
  bool bad = false;
#pragma unroll 8
  for (int t = 0; t < kP; ++t) {
    float v = E::to_float(s_page[t * kD + c]);
    bad |= !isfinite(v);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
    if (KBITS == 0) asum += (double)fabsf(v);
  }
  int slot = -1;
  float qmax;
  if (KBITS == 0) {
    const int K = d.promoted;
    int32_t* idx_field = reinterpret_cast<int32_t*>(page + d.key_off_index);
    if (indices != nullptr) {
      // forced channels: find this channel in the list
      const int32_t* mine = indices + ((int64_t)bh * num_pages + pg) * K;
      for (int k = 0; k < K; ++k) {
        int ch = mine[k];
        if (ch == c) slot = k;
      }
      if (c < K) idx_field[c] = mine[c];
    } else if (K == kD) {
      slot = c;
      idx_field[c] = c;
    } else if (K > 0) {
      float score = rnd<DT>(__fdiv_rn((float)asum, (float)kP));
      s_score[c] = score;
      __syncthreads();
      int rank = 0;
#pragma unroll 8
      for (int o = 0; o < kD; ++o) {
        float other = s_score[o];
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

  if (KBITS == 0) {
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      uint32_t l = 0, h = 0;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        uint32_t code = code_of<DT>(E::to_float(s_page[(w * 16 + k) * kD + c]), mn, scale, qmax);
        l |= (code & 3u) << (2 * k);
        h |= (code >> 2) << (2 * k);
      }
      lo[w] = l;
      hi[w] = h;
    }
    uint4* lrow = reinterpret_cast<uint4*>(page + c * 32);
    lrow[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    lrow[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    if (slot >= 0) {
      uint4* hrow = reinterpret_cast<uint4*>(page + d.key_off_high + slot * 32);
      hrow[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      hrow[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    }
  } else {
    constexpr int VPW = 32 / (KBITS ? KBITS : 2);     // codes per 32-bit word
    constexpr int WORDS = kP / VPW;                    // 8, 16 or 32 words per channel row
    uint32_t* row = reinterpret_cast<uint32_t*>(page + c * (WORDS * 4));
#pragma unroll 4
    for (int w = 0; w < WORDS; w += 4) {
      uint32_t out[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t acc = 0;
#pragma unroll
        for (int k = 0; k < VPW; ++k) {
          uint32_t code = code_of<DT>(E::to_float(s_page[((w + q) * VPW + k) * kD + c]), mn, scale, qmax);
          acc |= code << ((KBITS ? KBITS : 2) * k);
        }
        out[q] = acc;
      }
      reinterpret_cast<uint4*>(row)[w / 4] = make_uint4(out[0], out[1], out[2], out[3]);
    }
  }
  if (bad && nonfinite) *nonfinite = 1;
}

// one warp per token row; VBITS in {2,4,8}; LPG = lanes per group (value_group / 4)
template <int DT, int VBITS>
__global__ void __launch_bounds__(256) fast_value_rows_kernel(dartkv_cache_desc d, RowSource src, int value_begin,
                                                              int count, int lanes_per_group, int32_t* nonfinite) {
  using E = Elem<DT>;
  using T = typename E::type;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int64_t total = (int64_t)d.batch * d.kv_heads * count;
  if (warp >= total) return;
  const int bh = warp / count, j = warp % count, t = value_begin + j;
  const uint16_t* row_ptr = src.row(bh, t);
  uint2 raw = *reinterpret_cast<const uint2*>(row_ptr + lane * 4);
  T e[4];
  *reinterpret_cast<uint2*>(e) = raw;
  float v[4];
  bool bad = false;
  float mn = INFINITY, mx = -INFINITY;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[k] = E::to_float(e[k]);
    bad |= !isfinite(v[k]);
    mn = fminf(mn, v[k]);
    mx = fmaxf(mx, v[k]);
  }
  for (int off = 1; off < lanes_per_group; off <<= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  constexpr float qmax = (float)((1 << VBITS) - 1);
  const float scale = scale_of<DT>(mn, mx, qmax);
  uint32_t packed = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) packed |= code_of<DT>(v[k], mn, scale, qmax) << (VBITS * k);
  const int64_t out_row = (int64_t)bh * d.max_value_tokens + (t - d.sink_tokens);
  uint8_t* codes = d.v_codes + out_row * d.value_row_bytes;
  if (VBITS == 2) codes[lane] = (uint8_t)packed;
  else if (VBITS == 4) reinterpret_cast<uint16_t*>(codes)[lane] = (uint16_t)packed;
  else reinterpret_cast<uint32_t*>(codes)[lane] = packed;
  if ((lane % lanes_per_group) == 0) {
    int g = lane / lanes_per_group;
    store_f(d.v_meta, d.md_dtype, (out_row * 2 + 0) * d.value_groups + g, scale);
    store_f(d.v_meta, d.md_dtype, (out_row * 2 + 1) * d.value_groups + g, mn);
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
  const unsigned blocks = (unsigned)((rows + 7) / 8);
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
