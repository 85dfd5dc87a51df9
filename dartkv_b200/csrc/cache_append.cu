// Device-resident paged cache: geometry, append (quantize + pack into the pools) and
// materialization.  The lifecycle decisions of src/dart/cache.py:168-190,403-470 are integer
// bookkeeping done by the host (dartkv_append_plan); everything that touches K/V data runs here.

#include "common.cuh"

static inline int align16(int v) { return (v + 15) & ~15; }

extern "C" int dartkv_cache_geometry(dartkv_cache_desc* d) {
  DARTKV_REQUIRE(d != nullptr, "null descriptor");
  DARTKV_REQUIRE(d->batch > 0 && d->kv_heads > 0 && d->head_dim > 0, "batch, kv_heads and head_dim must be positive");
  DARTKV_REQUIRE(d->head_dim <= 1024, "head_dim must be at most 1024");
  DARTKV_REQUIRE(dartkv_valid_dtype(d->dtype), "key_states and value_states must be floating-point tensors");
  DARTKV_REQUIRE(dartkv_valid_dtype(d->md_dtype), "metadata_dtype must be a floating-point dtype (f32, f16, bf16)");
  DARTKV_REQUIRE(d->page_size > 0, "page_size must be positive");
  DARTKV_REQUIRE(d->key_group > 0 && d->value_group > 0, "group sizes must be positive");
  DARTKV_REQUIRE(dartkv_valid_bits(d->value_bits), "value_bits must be one of 2, 4, or 8");
  DARTKV_REQUIRE(d->key_mode == DARTKV_QUANTIZED_PAGE || d->key_mode == DARTKV_MIXED_PAGE, "bad key_mode");
  DARTKV_REQUIRE(d->sink_tokens >= 0 && d->ring_tokens > 0, "sink_tokens >= 0 and ring_tokens > 0 required");
  const int mdb = dartkv_dtype_bytes(d->md_dtype);
  const int gmax = ceil_div(d->page_size, d->key_group);
  if (d->key_mode == DARTKV_MIXED_PAGE) {
    DARTKV_REQUIRE(d->promoted >= 0 && d->promoted <= d->head_dim, "promoted must be in [0, head_dim]");
    const int pb = ceil_div(d->key_group, 4);
    d->key_off_high = align16(d->head_dim * gmax * pb);
    d->key_off_index = d->key_off_high + align16(d->promoted * gmax * pb);
    d->key_off_scale = d->key_off_index + align16(d->promoted * 4);
  } else {
    DARTKV_REQUIRE(dartkv_valid_bits(d->key_bits), "key_bits must be one of 2, 4, or 8");
    const int row = ceil_div(gmax * d->key_group, 8 / d->key_bits);
    d->key_off_high = align16(d->head_dim * row);
    d->key_off_index = d->key_off_high;
    d->key_off_scale = d->key_off_high;
  }
  d->key_off_zero = d->key_off_scale + align16(d->head_dim * gmax * mdb);
  d->key_page_bytes = d->key_off_zero + align16(d->head_dim * gmax * mdb);
  d->value_groups = ceil_div(d->head_dim, d->value_group);
  d->value_row_bytes = ceil_div(d->value_groups * d->value_group, 8 / d->value_bits);
  return DARTKV_OK;
}

// ---------------------------------------------------------------------------- token sources
// Absolute token t comes from the incoming chunk when t >= chunk_start, else from the dense ring.
struct TokenSource {
  const void* chunk;
  const void* ring;
  int64_t sb, sh, st;
  int chunk_start, ring_tokens, head_dim, kv_heads, dt;

  __device__ __forceinline__ float get(int bh, int t, int c) const {
    if (t >= chunk_start) {
      int b = bh / kv_heads, h = bh % kv_heads;
      return load_f(chunk, dt, (int64_t)b * sb + (int64_t)h * sh + (int64_t)(t - chunk_start) * st + c);
    }
    return load_f(ring, dt, ((int64_t)bh * ring_tokens + (t % ring_tokens)) * head_dim + c);
  }
};

// ---------------------------------------------------------------------------- dense copies
// ---------------------------------------------------------------------------- device-side metadata
__device__ __forceinline__ void publish_append(const dartkv_cache_desc& d, const dartkv_append_plan& p) {
  for (int pg = threadIdx.x; pg < p.num_pages; pg += blockDim.x) {
    d.page_start[p.first_page + pg] = p.page_token_start + pg * d.page_size;
    d.page_tokens[p.first_page + pg] = (pg == p.num_pages - 1) ? p.last_page_tokens : d.page_size;
  }
  if (threadIdx.x == 0) {
    d.state[0] = p.seen_after;
    d.state[1] = p.key_pages_after;
    d.state[2] = p.k_packed_end_after;
    d.state[3] = p.v_packed_end_after;
    d.state[4] = min(p.seen_after, d.sink_tokens);
  }
}

// true when a 16-byte piece of `dt` elements holds an Inf or NaN
__device__ __forceinline__ bool piece_nonfinite(uint4 v, int dt) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t flag = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (dt == DARTKV_F32) flag |= ((w[i] & 0x7FFFFFFFu) + 0x00800000u) & 0x80000000u;
    else flag |= ((w[i] & 0x7FFF7FFFu) + (dt == DARTKV_BF16 ? 0x00800080u : 0x04000400u)) & 0x80008000u;
  }
  return flag != 0;
}

constexpr int kCopyRows = 8;   // rows per block of the dense copy

// grid (bh, blocks of kCopyRows copy rows, side): copies sink tokens into the sink rows and tail tokens into
// the ring; copy row r enumerates only the chunk tokens that can need a copy: the sink part, then
// [ring_first, chunk end).  Block (0,0,0) also publishes the page table rows and the state words of the step
// (nothing of this step reads them; later launches on the stream do).
// With device_plan the step was planned on the device: the plan, the first ring token and the row count come from
// there (the grid is sized for the most rows such a step can copy).
__global__ void copy_dense_kernel(dartkv_cache_desc d, dartkv_append_plan p, const void* keys, const void* values,
                                  int64_t sb, int64_t sh, int64_t st, int ring_first, int rows, int vector_ok,
                                  int32_t* nonfinite, const dartkv_append_plan* device_plan) {
  if (device_plan) {
    p = *device_plan;
    const int chunk_end = p.chunk_start + p.chunk_tokens;
    const bool copies = p.sink_copy > 0 || p.ring_begin < chunk_end || p.value_end < chunk_end;
    ring_first = p.chunk_tokens;
    rows = 0;
    if (copies) {
      ring_first = max(p.sink_copy, min(p.ring_begin, max(p.value_end, p.chunk_start)) - p.chunk_start);
      rows = p.sink_copy + (p.chunk_tokens - ring_first);
    }
  }
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) publish_append(d, p);
  const int bh = blockIdx.x, side = blockIdx.z;
  const int r_begin = blockIdx.y * kCopyRows, r_end = min(rows, r_begin + kCopyRows);
  if (r_begin >= r_end) return;
  const int ring_begin = side == 0 ? p.ring_begin : p.value_end;  // values not packed by this step stay dense
  const void* src = side == 0 ? keys : values;
  const int b = bh / d.kv_heads, h = bh % d.kv_heads;
  const int64_t src_base = (int64_t)b * sb + (int64_t)h * sh;
  const int esize = dartkv_dtype_size(d.dtype);
  const int pieces = vector_ok ? d.head_dim * esize / 16 : d.head_dim;   // units per row: 16-byte pieces or elements
  bool bad = false;
  for (int i = threadIdx.x; i < (r_end - r_begin) * pieces; i += blockDim.x) {
    const int r = r_begin + i / pieces, c = i % pieces;
    const int j = r < p.sink_copy ? r : ring_first + (r - p.sink_copy);
    const int t = p.chunk_start + j;
    const bool to_sink = j < p.sink_copy;
    if (!to_sink && t < ring_begin) continue;
    void* dst = to_sink ? (side == 0 ? d.k_sink : d.v_sink) : (side == 0 ? d.k_ring : d.v_ring);
    const int64_t drow = to_sink ? ((int64_t)bh * d.sink_tokens + t) : ((int64_t)bh * d.ring_tokens + (t % d.ring_tokens));
    const int64_t srow = src_base + (int64_t)j * st;
    if (vector_ok) {
      const uint4 v = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(src) + srow * esize)[c];
      bad |= piece_nonfinite(v, d.dtype);
      reinterpret_cast<uint4*>(reinterpret_cast<char*>(dst) + drow * d.head_dim * esize)[c] = v;
    } else {
      const float v = load_f(src, d.dtype, srow + c);
      bad |= !isfinite(v);
      store_f(dst, d.dtype, drow * d.head_dim + c, v);
    }
  }
  if (bad && nonfinite) *nonfinite = 1;
}

// ---------------------------------------------------------------------------- generic key pages
// One block per (bh, new page).  Mixed mode: score channels, rank them, then quantize with
// qmax 15 for promoted channels and 3 for the rest; uniform mode: plain group quantization along tokens.
__global__ void key_pages_kernel(dartkv_cache_desc d, TokenSource src, int first_slot, int num_pages,
                                 int page_token_start, int last_page_tokens, const int32_t* __restrict__ indices,
                                 int32_t* nonfinite) {
  extern __shared__ float s_mem[];
  float* s_score = s_mem;
  int* s_slot = reinterpret_cast<int*>(s_mem + d.head_dim);
  const int bh = blockIdx.x, pg = blockIdx.y;
  const int D = d.head_dim, P = d.page_size, Gk = d.key_group;
  const int t0 = page_token_start + pg * P;
  const int n = (pg == num_pages - 1) ? last_page_tokens : P;
  const int G = ceil_div(n, Gk);
  uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + first_slot + pg) * d.key_page_bytes;
  void* scale = page + d.key_off_scale;
  void* zero = page + d.key_off_zero;
  bool bad = false;

  if (d.key_mode == DARTKV_MIXED_PAGE) {
    const int K = d.promoted;
    int32_t* idx_field = reinterpret_cast<int32_t*>(page + d.key_off_index);
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_slot[c] = -1;
    __syncthreads();
    if (indices != nullptr) {
      for (int k = threadIdx.x; k < K; k += blockDim.x) {
        int c = indices[((int64_t)bh * num_pages + pg) * K + k];
        idx_field[k] = c;
        if (c >= 0 && c < D) s_slot[c] = k;
      }
    } else if (K == D) {
      for (int c = threadIdx.x; c < D; c += blockDim.x) { s_slot[c] = c; idx_field[c] = c; }
    } else if (K > 0) {
      for (int c = threadIdx.x; c < D; c += blockDim.x) {
        double sum = 0.0;
        for (int j = 0; j < n; ++j) sum += (double)fabsf(src.get(bh, t0 + j, c));
        s_score[c] = rnd_rt(__fdiv_rn((float)sum, (float)n), d.dtype);
      }
      __syncthreads();
      for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float mine = s_score[c];
        int rank = 0;
        for (int o = 0; o < D; ++o) rank += (s_score[o] > mine) || (s_score[o] == mine && o < c);
        if (rank < K) { s_slot[c] = rank; idx_field[rank] = c; }
      }
    }
    __syncthreads();
    const int pb = ceil_div(Gk, 4);
    uint8_t* low = page;
    uint8_t* high = page + d.key_off_high;
    for (int item = threadIdx.x; item < D * G; item += blockDim.x) {
      int c = item % D, g = item / D;
      int slot = s_slot[c];
      float qmax = slot >= 0 ? 15.0f : 3.0f;
      float mn = INFINITY, mx = -INFINITY;
      for (int j = 0; j < Gk; ++j) {
        float v = src.get(bh, t0 + min(g * Gk + j, n - 1), c);
        bad |= !isfinite(v);
        mn = fminf(mn, v);
        mx = fmaxf(mx, v);
      }
      float s = group_scale(mn, mx, qmax, d.dtype, DARTKV_DIV_TRUE);
      store_f(scale, d.md_dtype, c * G + g, s);
      store_f(zero, d.md_dtype, c * G + g, mn);
      uint8_t* lo = low + (c * G + g) * pb;
      uint8_t* hi = slot >= 0 ? high + (slot * G + g) * pb : nullptr;
      uint32_t lacc = 0, hacc = 0;
      int filled = 0;
      for (int j = 0; j < Gk; ++j) {
        uint32_t code = group_code(src.get(bh, t0 + min(g * Gk + j, n - 1), c), mn, s, qmax, d.dtype);
        lacc |= (code & 3u) << (2 * filled);
        hacc |= (code >> 2) << (2 * filled);
        if (++filled == 4) {
          *lo++ = (uint8_t)lacc;
          if (hi) *hi++ = (uint8_t)hacc;
          lacc = hacc = 0;
          filled = 0;
        }
      }
      if (filled) {
        *lo = (uint8_t)lacc;
        if (hi) *hi = (uint8_t)hacc;
      }
    }
  } else {
    const int bits = d.key_bits, vpb = 8 / bits;
    const float qmax = (float)((1 << bits) - 1);
    const int padded = G * Gk;
    const int row_bytes = ceil_div(padded, vpb);
    // a unit = lcm(Gk, vpb) codes: whole groups and whole bytes
    int gcd = Gk, tmp = vpb;
    while (tmp) { int r = gcd % tmp; gcd = tmp; tmp = r; }
    const int unit = Gk / gcd * vpb;
    const int units = ceil_div(padded, unit);
    for (int item = threadIdx.x; item < D * units; item += blockDim.x) {
      int c = item % D, u = item / D;
      int begin = u * unit, end = min(begin + unit, padded);
      uint8_t* out = page + (int64_t)c * row_bytes + begin / vpb;
      uint32_t acc = 0;
      int filled = 0;
      for (int g0 = begin; g0 < end; g0 += Gk) {
        float mn = INFINITY, mx = -INFINITY;
        for (int j = 0; j < Gk; ++j) {
          float v = src.get(bh, t0 + min(g0 + j, n - 1), c);
          bad |= !isfinite(v);
          mn = fminf(mn, v);
          mx = fmaxf(mx, v);
        }
        float s = group_scale(mn, mx, qmax, d.dtype, DARTKV_DIV_TRUE);
        store_f(scale, d.md_dtype, c * G + g0 / Gk, s);
        store_f(zero, d.md_dtype, c * G + g0 / Gk, mn);
        for (int j = 0; j < Gk; ++j) {
          acc |= group_code(src.get(bh, t0 + min(g0 + j, n - 1), c), mn, s, qmax, d.dtype) << (filled * bits);
          if (++filled == vpb) {
            *out++ = (uint8_t)acc;
            acc = 0;
            filled = 0;
          }
        }
      }
      if (filled) *out = (uint8_t)acc;
    }
  }
  if (bad && nonfinite) *nonfinite = 1;
}

// ---------------------------------------------------------------------------- generic value rows
// One thread per (bh, token, unit); a token's groups run along head_dim.
__global__ void value_rows_kernel(dartkv_cache_desc d, TokenSource src, int value_begin, int value_end, int unit,
                                  int units, int32_t* nonfinite) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int count = value_end - value_begin;
  int64_t total = (int64_t)d.batch * d.kv_heads * count * units;
  if (tid >= total) return;
  int u = (int)(tid % units);
  int j = (int)((tid / units) % count);
  int bh = (int)(tid / ((int64_t)units * count));
  int t = value_begin + j;
  int64_t row = (int64_t)bh * d.max_value_tokens + (t - d.sink_tokens);
  const int bits = d.value_bits, vpb = 8 / bits, Gv = d.value_group, D = d.head_dim;
  const float qmax = (float)((1 << bits) - 1);
  const int padded = d.value_groups * Gv;
  int begin = u * unit, end = min(begin + unit, padded);
  uint8_t* out = d.v_codes + row * d.value_row_bytes + begin / vpb;
  uint32_t acc = 0;
  int filled = 0;
  bool bad = false;
  for (int g0 = begin; g0 < end; g0 += Gv) {
    float mn = INFINITY, mx = -INFINITY;
    for (int k = 0; k < Gv; ++k) {
      float v = src.get(bh, t, min(g0 + k, D - 1));
      bad |= !isfinite(v);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
    float s = group_scale(mn, mx, qmax, d.dtype, DARTKV_DIV_TRUE);
    int g = g0 / Gv;
    store_f(d.v_meta, d.md_dtype, (row * 2 + 0) * d.value_groups + g, s);
    store_f(d.v_meta, d.md_dtype, (row * 2 + 1) * d.value_groups + g, mn);
    for (int k = 0; k < Gv; ++k) {
      acc |= group_code(src.get(bh, t, min(g0 + k, D - 1)), mn, s, qmax, d.dtype) << (filled * bits);
      if (++filled == vpb) {
        *out++ = (uint8_t)acc;
        acc = 0;
        filled = 0;
      }
    }
  }
  if (filled) *out = (uint8_t)acc;
  if (bad && nonfinite) *nonfinite = 1;
}

// ---------------------------------------------------------------------------- element access
// Dequantized key element (token j of a page, channel c); slot = promoted slot of c or -1.
__device__ __forceinline__ float page_key_element(const dartkv_cache_desc& d, const uint8_t* page, int n, int j, int c,
                                                  int slot, int flavour) {
  const int Gk = d.key_group, G = ceil_div(n, Gk), g = j / Gk;
  float s = load_f(page + d.key_off_scale, d.md_dtype, c * G + g);
  float z = load_f(page + d.key_off_zero, d.md_dtype, c * G + g);
  uint32_t code;
  if (d.key_mode == DARTKV_MIXED_PAGE) {
    const int pb = ceil_div(Gk, 4), jj = j % Gk;
    code = (page[(c * G + g) * pb + jj / 4] >> ((jj % 4) * 2)) & 3u;
    if (slot >= 0) code |= ((page[d.key_off_high + (slot * G + g) * pb + jj / 4] >> ((jj % 4) * 2)) & 3u) << 2;
  } else {
    const int bits = d.key_bits, vpb = 8 / bits;
    const int row_bytes = ceil_div(G * Gk, vpb);
    code = (page[(int64_t)c * row_bytes + j / vpb] >> ((j % vpb) * bits)) & ((1u << bits) - 1u);
  }
  return affine_restore((float)code, s, z, d.md_dtype, d.dtype, flavour);
}

__device__ __forceinline__ float packed_value_element(const dartkv_cache_desc& d, int bh, int t, int c, int flavour) {
  int64_t row = (int64_t)bh * d.max_value_tokens + (t - d.sink_tokens);
  const int bits = d.value_bits, vpb = 8 / bits, g = c / d.value_group;
  uint32_t code = (d.v_codes[row * d.value_row_bytes + c / vpb] >> ((c % vpb) * bits)) & ((1u << bits) - 1u);
  float s = load_f(d.v_meta, d.md_dtype, (row * 2 + 0) * d.value_groups + g);
  float z = load_f(d.v_meta, d.md_dtype, (row * 2 + 1) * d.value_groups + g);
  return affine_restore((float)code, s, z, d.md_dtype, d.dtype, flavour);
}

// first page whose range ends after token t (pages are contiguous from sink_tokens)
__device__ __forceinline__ int find_page(const dartkv_cache_desc& d, int pages, int t) {
  int lo = 0, hi = pages - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (d.page_start[mid] + d.page_tokens[mid] > t) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// grid (bh, token); out [B*H, t1-t0, D]
__global__ void materialize_kernel(dartkv_cache_desc d, int side, int t0, int t1, int flavour, void* out, int out_dt) {
  extern __shared__ int s_slot[];
  __shared__ int s_page;
  const int bh = blockIdx.x, t = t0 + blockIdx.y, D = d.head_dim;
  const int sink_filled = d.state[4];
  const int packed_end = side == 0 ? d.state[2] : d.state[3];
  int64_t orow = ((int64_t)bh * (t1 - t0) + (t - t0)) * D;
  if (t < sink_filled || t >= packed_end) {
    const void* src;
    int64_t row;
    if (t < sink_filled) {
      src = side == 0 ? d.k_sink : d.v_sink;
      row = (int64_t)bh * d.sink_tokens + t;
    } else {
      src = side == 0 ? d.k_ring : d.v_ring;
      row = (int64_t)bh * d.ring_tokens + (t % d.ring_tokens);
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      store_f(out, out_dt, orow + c, rnd_rt(load_f(src, d.dtype, row * D + c), out_dt));
    return;
  }
  if (side == 1) {
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      store_f(out, out_dt, orow + c, rnd_rt(packed_value_element(d, bh, t, c, flavour), out_dt));
    return;
  }
  if (threadIdx.x == 0) s_page = find_page(d, d.state[1], t);
  __syncthreads();
  const int pg = s_page;
  const uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + pg) * d.key_page_bytes;
  if (d.key_mode == DARTKV_MIXED_PAGE) {
    const int32_t* idx = reinterpret_cast<const int32_t*>(page + d.key_off_index);
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_slot[c] = -1;
    __syncthreads();
    for (int k = threadIdx.x; k < d.promoted; k += blockDim.x) {
      int c = idx[k];
      if (c >= 0 && c < D) s_slot[c] = k;
    }
    __syncthreads();
  }
  const int n = d.page_tokens[pg], j = t - d.page_start[pg];
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    int slot = d.key_mode == DARTKV_MIXED_PAGE ? s_slot[c] : -1;
    store_f(out, out_dt, orow + c, rnd_rt(page_key_element(d, page, n, j, c, slot, flavour), out_dt));
  }
}

// dequantize one key page back into the ring rows of its tokens (first half of the boundary
// re-quantization of src/dart/cache.py:427-439); grid (bh, token of the page)
__global__ void page_to_ring_kernel(dartkv_cache_desc d, int slot_index, int page_token_start, int n) {
  extern __shared__ int s_slot[];
  const int bh = blockIdx.x, j = blockIdx.y, D = d.head_dim;
  const uint8_t* page = d.k_pages + ((int64_t)bh * d.max_key_pages + slot_index) * d.key_page_bytes;
  if (d.key_mode == DARTKV_MIXED_PAGE) {
    const int32_t* idx = reinterpret_cast<const int32_t*>(page + d.key_off_index);
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_slot[c] = -1;
    __syncthreads();
    for (int k = threadIdx.x; k < d.promoted; k += blockDim.x) {
      int c = idx[k];
      if (c >= 0 && c < D) s_slot[c] = k;
    }
    __syncthreads();
  }
  int t = page_token_start + j;
  int64_t row = (int64_t)bh * d.ring_tokens + (t % d.ring_tokens);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    int slot = d.key_mode == DARTKV_MIXED_PAGE ? s_slot[c] : -1;
    store_f(d.k_ring, d.dtype, row * D + c, page_key_element(d, page, n, j, c, slot, DARTKV_DEQUANT_PER_OP));
  }
}

// ---------------------------------------------------------------------------- fast page kernels
// Common geometry (head_dim 128, 16-bit data, full 128-token pages, key group 128): append_fast.cu.
int dartkv_append_fast_supported(const dartkv_cache_desc* d, const dartkv_append_plan* p, int64_t st);
int dartkv_append_fast_keys(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* keys, int64_t sb,
                            int64_t sh, int64_t st, const int32_t* indices, int32_t* nonfinite, cudaStream_t stream,
                            const dartkv_append_plan* device_plan = nullptr);
int dartkv_append_fast_values(const dartkv_cache_desc* d, const dartkv_append_plan* p, const void* values, int64_t sb,
                              int64_t sh, int64_t st, int32_t* nonfinite, cudaStream_t stream,
                              const dartkv_append_plan* device_plan = nullptr);

static int validate_desc(const dartkv_cache_desc* d) {
  DARTKV_REQUIRE(d != nullptr, "null descriptor");
  DARTKV_REQUIRE(d->key_page_bytes > 0 && d->value_row_bytes > 0, "descriptor geometry not filled (call dartkv_cache_geometry)");
  DARTKV_REQUIRE(d->k_ring && d->v_ring && d->k_pages && d->v_codes && d->v_meta && d->page_start && d->page_tokens && d->state,
                 "descriptor has a null pool pointer");
  DARTKV_REQUIRE(d->sink_tokens == 0 || (d->k_sink && d->v_sink), "descriptor has a null sink pointer");
  return DARTKV_OK;
}

extern "C" int dartkv_cache_append(const dartkv_cache_desc* desc, const dartkv_append_plan* plan, const void* keys,
                                   const void* values, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                                   const int32_t* indices, int32_t* nonfinite, void* stream_) {
  int rc = validate_desc(desc);
  if (rc) return rc;
  DARTKV_REQUIRE(plan != nullptr && keys != nullptr && values != nullptr, "append received a null pointer");
  const dartkv_cache_desc& d = *desc;
  const dartkv_append_plan& p = *plan;
  cudaStream_t stream = (cudaStream_t)stream_;
  DARTKV_REQUIRE(p.chunk_tokens > 0, "key/value sequence and head dimensions must be non-empty");
  DARTKV_REQUIRE(p.first_page >= 0 && p.first_page + p.num_pages <= d.max_key_pages, "append exceeds the key page capacity");
  DARTKV_REQUIRE(p.value_end <= p.value_begin || p.value_end - d.sink_tokens <= d.max_value_tokens,
                 "append exceeds the packed value capacity");
  DARTKV_REQUIRE(p.sink_copy >= 0 && p.sink_copy <= p.chunk_tokens &&
                     (p.sink_copy == 0 || p.chunk_start + p.sink_copy <= d.sink_tokens),
                 "bad sink_copy");
  DARTKV_REQUIRE(p.num_pages == 0 || (p.last_page_tokens > 0 && p.last_page_tokens <= d.page_size), "bad last_page_tokens");
  const int bh = d.batch * d.kv_heads;
  const int chunk_end = p.chunk_start + p.chunk_tokens;
  const size_t page_smem = (size_t)d.head_dim * (sizeof(float) + sizeof(int));

  const int32_t* new_page_indices = indices;
  if (p.requantize_last_page) {
    DARTKV_REQUIRE(p.first_page > 0 && p.page_token_start - d.page_size >= 0, "nothing to re-quantize");
    const int slot = p.first_page - 1, start = p.page_token_start - d.page_size;
    page_to_ring_kernel<<<dim3(bh, d.page_size), 128, d.head_dim * sizeof(int), stream>>>(d, slot, start, d.page_size);
    DARTKV_LAUNCH_OK("page_to_ring_kernel");
    TokenSource ring_only{nullptr, d.k_ring, 0, 0, 0, INT32_MAX, d.ring_tokens, d.head_dim, d.kv_heads, d.dtype};
    key_pages_kernel<<<dim3(bh, 1), 128, page_smem, stream>>>(d, ring_only, slot, 1, start, d.page_size, indices, nullptr);
    DARTKV_LAUNCH_OK("key_pages_kernel (re-quantize)");
    // an explicit index list carries the re-quantized page first, one [promoted] row per (bh)
    if (indices) new_page_indices = indices + (int64_t)bh * d.promoted;
  }

  const bool copies = p.sink_copy > 0 || p.ring_begin < chunk_end || p.value_end < chunk_end;
  int fast = dartkv_append_fast_supported(desc, plan, stride_t);
  if (stride_b % 8 || stride_h % 8 || ((uintptr_t)keys | (uintptr_t)values) % 16) fast = 0;
  if (p.num_pages > 0) {
    if (fast & 1) {
      rc = dartkv_append_fast_keys(desc, plan, keys, stride_b, stride_h, stride_t, new_page_indices, nonfinite, stream);
      if (rc) return rc;
    } else {
      TokenSource ks{keys, d.k_ring, stride_b, stride_h, stride_t, p.chunk_start, d.ring_tokens, d.head_dim, d.kv_heads, d.dtype};
      DARTKV_REQUIRE(p.num_pages <= 65535, "too many pages in one append (limit 65535)");
      key_pages_kernel<<<dim3(bh, p.num_pages), 128, page_smem, stream>>>(d, ks, p.first_page, p.num_pages,
                                                                         p.page_token_start, p.last_page_tokens,
                                                                         new_page_indices, nonfinite);
      DARTKV_LAUNCH_OK("key_pages_kernel");
    }
  }
  if (p.value_end > p.value_begin) {
    if (fast & 2) {
      rc = dartkv_append_fast_values(desc, plan, values, stride_b, stride_h, stride_t, nonfinite, stream);
      if (rc) return rc;
    } else {
      TokenSource vs{values, d.v_ring, stride_b, stride_h, stride_t, p.chunk_start, d.ring_tokens, d.head_dim, d.kv_heads, d.dtype};
      const int vpb = 8 / d.value_bits;
      const int unit = d.value_group / dartkv_gcd(d.value_group, vpb) * vpb;
      const int units = ceil_div(d.value_groups * d.value_group, unit);
      int64_t threads = (int64_t)bh * (p.value_end - p.value_begin) * units;
      value_rows_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, stream>>>(d, vs, p.value_begin, p.value_end, unit, units, nonfinite);
      DARTKV_LAUNCH_OK("value_rows_kernel");
    }
  }
  {
    // dense copies of the step (possibly none) and the step's metadata, one launch
    int ring_first = p.chunk_tokens, rows = 0;
    if (copies) {
      ring_first = max(p.sink_copy, min(p.ring_begin, max(p.value_end, p.chunk_start)) - p.chunk_start);
      rows = p.sink_copy + (p.chunk_tokens - ring_first);
    }
    const int row_blocks = max(1, ceil_div(rows, kCopyRows));
    DARTKV_REQUIRE(row_blocks <= 65535, "append chunks this long must be split by the caller");
    const int esize = dartkv_dtype_size(d.dtype);
    const int vector_ok = (d.head_dim * esize) % 16 == 0 && (stride_b * esize) % 16 == 0 && (stride_h * esize) % 16 == 0 &&
                          (stride_t * esize) % 16 == 0 && ((uintptr_t)keys | (uintptr_t)values) % 16 == 0;
    copy_dense_kernel<<<dim3(rows > 0 ? bh : 1, row_blocks, rows > 0 ? 2 : 1), 128, 0, stream>>>(
        d, p, keys, values, stride_b, stride_h, stride_t, ring_first, rows, vector_ok, nonfinite, nullptr);
    DARTKV_LAUNCH_OK("copy_dense_kernel");
  }
  return DARTKV_OK;
}

extern "C" int dartkv_cache_materialize(const dartkv_cache_desc* desc, int side, int32_t t0, int32_t t1, int flavour,
                                        void* out, int out_dtype, void* stream) {
  int rc = validate_desc(desc);
  if (rc) return rc;
  DARTKV_REQUIRE(side == 0 || side == 1, "side must be 0 (keys) or 1 (values)");
  DARTKV_REQUIRE(t0 >= 0 && t1 >= t0, "bad token range");
  DARTKV_REQUIRE(dartkv_valid_dtype(out_dtype), "unsupported output dtype");
  DARTKV_REQUIRE(flavour == DARTKV_DEQUANT_PER_OP || flavour == DARTKV_DEQUANT_FP32, "unknown dequant flavour %d", flavour);
  if (t1 == t0) return DARTKV_OK;
  DARTKV_REQUIRE(out != nullptr, "materialize received a null output");
  DARTKV_REQUIRE(t1 - t0 <= 65535, "materialize at most 65535 tokens per call");
  const int bh = desc->batch * desc->kv_heads;
  materialize_kernel<<<dim3(bh, t1 - t0), 128, desc->head_dim * sizeof(int), (cudaStream_t)stream>>>(*desc, side, t0, t1, flavour, out, out_dtype);
  DARTKV_LAUNCH_OK("materialize_kernel");
  return DARTKV_OK;
}


// ---------------------------------------------------------------------------- host-side lifecycle planner
// The integer bookkeeping of the reference's cache lifecycle (src/dart/cache.py:168-190, 403-470) as a host
// function: which chunk tokens go to the sink rows, which become key pages, which value rows get packed and what
// stays dense in the ring.  Pages are appended in sequence order, so the state is four integers.
// The arithmetic itself, shared by the host entry point and the planner kernel of device-planned appends.
__host__ __device__ static inline void lifecycle_core(const dartkv_lifecycle_config& cfg, dartkv_lifecycle_state& state,
                                                      int chunk_tokens, dartkv_append_plan& plan) {
  const int page = cfg.page_size, sink_total = cfg.sink_tokens;
  const int seen = state.seen;
  const int sink_copy = min(max(0, sink_total - seen), chunk_tokens);
  const int rest = chunk_tokens - sink_copy;
  const int rest_start = seen + sink_copy;
  const int chunk_end = seen + chunk_tokens;
  const int sink_filled_after = min(chunk_end, sink_total);
  // invariant: packed_end is the end of the packed range, or min(seen, sink_tokens) while nothing is packed
  const int k_end = state.k_packed_end, v_end = state.v_packed_end;
  const int pending_k = seen - k_end, pending_v = seen - v_end;
  int num_pages = 0, last_page_tokens = page;
  const int page_token_start = pending_k ? k_end : rest_start;
  const int value_begin = pending_v ? v_end : rest_start;
  int value_end = value_begin;
  int requantize = 0;
  if (rest > 0) {
    if (cfg.value_local_tokens) {
      // keys page by page behind `local_tokens`, values token by token behind the newest `value_local_tokens`;
      // a one-token append right after a prompt that ended on a page boundary re-quantizes the last page
      if (seen > 0 && pending_k == 0 && cfg.local_tokens == 1 && rest == 1 && state.key_pages > 0) requantize = 1;
      const int stream = pending_k + rest;
      const int local = seen == 0 ? 0 : cfg.local_tokens;
      num_pages = max(0, stream - local) / page;
      value_end = value_begin + max(0, pending_v + rest - cfg.value_local_tokens);
    } else if (cfg.hold_partial_pages || cfg.local_tokens) {
      const int stream = pending_k + rest;
      num_pages = max(0, stream - cfg.local_tokens) / page;
      value_end = value_begin + num_pages * page;
    } else {
      num_pages = (rest + page - 1) / page;
      last_page_tokens = rest - (num_pages - 1) * page;
      value_end = value_begin + rest;
    }
  }
  int k_end_after;
  if (num_pages > 0) k_end_after = page_token_start + (num_pages - 1) * page + last_page_tokens;
  else if (state.key_pages > 0) k_end_after = k_end;
  else k_end_after = sink_filled_after;
  int v_end_after;
  if (value_end > value_begin) v_end_after = value_end;
  else if (v_end > sink_total) v_end_after = v_end;
  else v_end_after = sink_filled_after;
  plan.chunk_start = seen;
  plan.chunk_tokens = chunk_tokens;
  plan.sink_copy = sink_copy;
  plan.first_page = state.key_pages;
  plan.num_pages = num_pages;
  plan.page_token_start = page_token_start;
  plan.last_page_tokens = last_page_tokens;
  plan.value_begin = value_begin;
  plan.value_end = value_end;
  plan.ring_begin = max(k_end_after, rest_start);
  plan.reserved = 0;
  plan.seen_after = chunk_end;
  plan.k_packed_end_after = k_end_after;
  plan.v_packed_end_after = v_end_after;
  plan.key_pages_after = state.key_pages + num_pages;
  plan.requantize_last_page = requantize;
  state.seen = chunk_end;
  state.k_packed_end = k_end_after;
  state.v_packed_end = v_end_after;
  state.key_pages += num_pages;
}

extern "C" int dartkv_lifecycle_plan(const dartkv_lifecycle_config* cfg, dartkv_lifecycle_state* state,
                                     int chunk_tokens, dartkv_append_plan* plan) {
  DARTKV_REQUIRE(cfg != nullptr && state != nullptr && plan != nullptr, "lifecycle_plan received a null pointer");
  DARTKV_REQUIRE(chunk_tokens > 0, "key/value sequence and head dimensions must be non-empty");
  DARTKV_REQUIRE(cfg->page_size > 0 && cfg->sink_tokens >= 0 && cfg->local_tokens >= 0 && cfg->value_local_tokens >= 0,
                 "bad lifecycle configuration");
  DARTKV_REQUIRE((int64_t)state->seen + chunk_tokens < (1ll << 31) - 2 * cfg->page_size, "token count overflows 32 bits");
  lifecycle_core(*cfg, *state, chunk_tokens, *plan);
  return DARTKV_OK;
}

// Plan and append in one call.  The state advances only if every launch of the step was accepted.
extern "C" int dartkv_cache_append_step(const dartkv_cache_desc* desc, const dartkv_lifecycle_config* cfg,
                                        dartkv_lifecycle_state* state, const void* keys, const void* values,
                                        int chunk_tokens, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                                        const int32_t* indices, int32_t* nonfinite, dartkv_append_plan* plan_out,
                                        void* stream) {
  DARTKV_REQUIRE(state != nullptr, "append_step received a null pointer");
  dartkv_lifecycle_state next = *state;
  dartkv_append_plan plan;
  int rc = dartkv_lifecycle_plan(cfg, &next, chunk_tokens, &plan);
  if (rc) return rc;
  if (plan_out) *plan_out = plan;
  DARTKV_REQUIRE(desc != nullptr, "null descriptor");
  if (plan.key_pages_after > desc->max_key_pages ||
      (plan.value_end > plan.value_begin && plan.value_end - desc->sink_tokens > desc->max_value_tokens)) {
    dartkv_set_error("append needs %d key pages and %d packed value rows; the pools hold %d and %d: grow them first",
                     plan.key_pages_after, plan.value_end - desc->sink_tokens, desc->max_key_pages, desc->max_value_tokens);
    return DARTKV_ELIMIT;
  }
  rc = dartkv_cache_append(desc, &plan, keys, values, stride_b, stride_h, stride_t, indices, nonfinite, stream);
  if (rc) return rc;
  *state = next;
  return DARTKV_OK;
}

// ---------------------------------------------------------------------------- device-planned append
// The same step with nothing decided on the host: a one-thread kernel reads the lifecycle state the cache keeps on
// the device (desc->state[0..3]), runs the planner above and leaves the plan in desc->state[8..23]; the page, value
// row and copy kernels that follow on the stream read it there.  Their grids cover the most a chunk of this length
// can bring, blocks beyond the step's real work return at once.  Every launch has the same shape whatever the
// state, so a decode step (append + attention) can be captured in a CUDA graph once and replayed token after token.
// One step of the reference's lifecycle is not served: the one-token append that re-quantizes the boundary page
// (src/dart/cache.py:427-439) can only be the first append after a prompt, and the host, whose copy of the state
// tells it so, sends that one through the host-planned path.
__global__ void plan_append_kernel(dartkv_cache_desc d, dartkv_lifecycle_config cfg, int chunk_tokens) {
  dartkv_lifecycle_state state{d.state[0], d.state[2], d.state[3], d.state[1]};
  dartkv_append_plan plan;
  lifecycle_core(cfg, state, chunk_tokens, plan);
  *reinterpret_cast<dartkv_append_plan*>(d.state + 8) = plan;
}

extern "C" int dartkv_cache_append_device_planned(const dartkv_cache_desc* desc, const dartkv_lifecycle_config* cfg,
                                                  const void* keys, const void* values, int chunk_tokens,
                                                  int64_t stride_b, int64_t stride_h, int64_t stride_t,
                                                  int32_t* nonfinite, void* stream_) {
  int rc = validate_desc(desc);
  if (rc) return rc;
  DARTKV_REQUIRE(cfg != nullptr && keys != nullptr && values != nullptr, "append received a null pointer");
  DARTKV_REQUIRE(chunk_tokens > 0 && chunk_tokens <= 32768, "device-planned appends take 1..32768 tokens");
  DARTKV_REQUIRE(cfg->hold_partial_pages || cfg->local_tokens > 0 || cfg->value_local_tokens > 0,
                 "device-planned appends serve the lifecycles that only pack full pages (hold_partial_pages, local_tokens or "
                 "value_local_tokens)");
  DARTKV_REQUIRE(cfg->local_tokens >= 0 && cfg->value_local_tokens >= 0, "bad lifecycle configuration");
  DARTKV_REQUIRE(cfg->page_size == desc->page_size && cfg->sink_tokens == desc->sink_tokens,
                 "lifecycle configuration and descriptor disagree");
  const dartkv_cache_desc& d = *desc;
  cudaStream_t stream = (cudaStream_t)stream_;
  // the most this chunk can bring: pending tokens (fewer than a page) may complete one page more
  dartkv_append_plan most{};
  most.chunk_tokens = chunk_tokens;
  most.num_pages = chunk_tokens / d.page_size + 1;
  most.last_page_tokens = d.page_size;
  most.value_begin = 0;
  most.value_end = most.num_pages * d.page_size + chunk_tokens;   // whole pages, or token by token behind a local window
  const int fast = dartkv_append_fast_supported(desc, &most, stride_t);
  DARTKV_REQUIRE(fast == 3 && stride_b % 8 == 0 && stride_h % 8 == 0 && ((uintptr_t)keys | (uintptr_t)values) % 16 == 0,
                 "device-planned appends need the geometry of the page kernels (head_dim 128, 16-bit data, 128-token "
                 "pages and key groups, aligned inputs)");
  const dartkv_append_plan* device_plan = reinterpret_cast<const dartkv_append_plan*>(d.state + 8);
  plan_append_kernel<<<1, 1, 0, stream>>>(d, *cfg, chunk_tokens);
  DARTKV_LAUNCH_OK("plan_append_kernel");
  rc = dartkv_append_fast_keys(desc, &most, keys, stride_b, stride_h, stride_t, nullptr, nonfinite, stream, device_plan);
  if (rc) return rc;
  rc = dartkv_append_fast_values(desc, &most, values, stride_b, stride_h, stride_t, nonfinite, stream, device_plan);
  if (rc) return rc;
  const int bh = d.batch * d.kv_heads;
  const int row_blocks = max(1, ceil_div(chunk_tokens, kCopyRows));
  DARTKV_REQUIRE(row_blocks <= 65535, "append chunks this long must be split by the caller");
  const int esize = dartkv_dtype_size(d.dtype);
  const int vector_ok = (d.head_dim * esize) % 16 == 0 && (stride_b * esize) % 16 == 0 && (stride_h * esize) % 16 == 0 &&
                        (stride_t * esize) % 16 == 0;
  copy_dense_kernel<<<dim3(bh, row_blocks, 2), 128, 0, stream>>>(d, most, keys, values, stride_b, stride_h, stride_t, 0, 0,
                                                                 vector_ok, nonfinite, device_plan);
  DARTKV_LAUNCH_OK("copy_dense_kernel");
  return DARTKV_OK;
}
