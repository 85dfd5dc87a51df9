// Generic (any shape, any supported dtype) quantize / pack / dequantize primitives.
//
// These back the functional API (quantize, quantize_axis, dequantize, quantize_key_mixed,
// select_key_channels) for arbitrary geometry; the page-shaped fast kernels used by the cache
// live in cache_append.cu.  Arithmetic follows the reference's per-op rounding in the data
// dtype (src/dart/quantization.py:178-186, src/dart/mixed.py:200-209).

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

// ---------------------------------------------------------------------------- error plumbing
static thread_local char g_error[512] = "";

void dartkv_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

static std::atomic<long long> g_launches{0};
void dartkv_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" long long dartkv_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" const char* dartkv_last_error(void) { return g_error; }
extern "C" int dartkv_version(void) { return 110; }

// ---------------------------------------------------------------------------- sharding rule (host arithmetic)
// Every (batch row, KV head) is independent on this path, so ranks own rectangles of rows x heads.  The batch is
// split first; KV heads are split too only when there are more ranks than batch rows.  With `g` head groups
// (the smallest divisor of kv_heads that divides world_size and leaves world_size / g <= batch) rank r belongs
// to batch group r / g and head group r % g; the first batch % (world_size / g) batch groups hold one row more.
extern "C" int dartkv_shard_range(int batch, int kv_heads, int world_size, int rank, dartkv_shard* out) {
  DARTKV_REQUIRE(out != nullptr, "shard_range received a null pointer");
  DARTKV_REQUIRE(batch > 0 && kv_heads > 0, "batch and kv_heads must be positive");
  DARTKV_REQUIRE(world_size > 0 && rank >= 0 && rank < world_size, "rank must be in [0, world_size)");
  int groups = 0;
  for (int g = 1; g <= kv_heads; ++g) {
    if (kv_heads % g || world_size % g) continue;
    if (world_size / g <= batch) { groups = g; break; }
  }
  DARTKV_REQUIRE(groups > 0,
                 "cannot shard batch %d x %d KV heads over %d ranks: no divisor of the KV heads divides the rank "
                 "count and leaves at most one batch group per row", batch, kv_heads, world_size);
  const int batch_groups = world_size / groups;
  const int bg = rank / groups, hg = rank % groups;
  const int base = batch / batch_groups, extra = batch % batch_groups;
  out->row_begin = bg * base + (bg < extra ? bg : extra);
  out->row_end = out->row_begin + base + (bg < extra ? 1 : 0);
  out->head_begin = hg * (kv_heads / groups);
  out->head_end = out->head_begin + kv_heads / groups;
  out->batch_groups = batch_groups;
  out->head_groups = groups;
  out->rows_padded = base + (extra ? 1 : 0);
  out->reserved = 0;
  return DARTKV_OK;
}

static inline unsigned grid_for(int64_t threads, int block) { return (unsigned)((threads + block - 1) / block); }

// ---------------------------------------------------------------------------- pack / unpack
__global__ void pack_kernel(const uint8_t* __restrict__ codes, int64_t rows, int64_t n, int bits, int64_t packed_bytes,
                            uint8_t* __restrict__ packed) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= rows * packed_bytes) return;
  int64_t row = tid / packed_bytes, byte = tid % packed_bytes;
  int vpb = 8 / bits;
  uint32_t acc = 0;
  for (int i = 0; i < vpb; ++i) {
    int64_t j = byte * vpb + i;
    if (j < n) acc |= (uint32_t)(codes[row * n + j] & ((1u << bits) - 1u)) << (i * bits);
  }
  packed[tid] = (uint8_t)acc;
}

__global__ void unpack_kernel(const uint8_t* __restrict__ packed, int64_t rows, int64_t packed_bytes, int bits,
                              int64_t count, uint8_t* __restrict__ codes) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= rows * count) return;
  int64_t row = tid / count, j = tid % count;
  int vpb = 8 / bits;
  uint32_t byte = packed[row * packed_bytes + j / vpb];
  codes[tid] = (uint8_t)((byte >> ((j % vpb) * bits)) & ((1u << bits) - 1u));
}

extern "C" int dartkv_pack(const uint8_t* codes, int64_t rows, int64_t n, int bits, uint8_t* packed, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_bits(bits), "bits must be one of (2, 4, 8), got %d", bits);
  DARTKV_REQUIRE(rows >= 0 && n > 0, "pack expects rows >= 0 and n > 0");
  if (rows == 0) return DARTKV_OK;
  DARTKV_REQUIRE(codes && packed, "pack received a null pointer");
  int64_t packed_bytes = ceil_div64(n, 8 / bits);
  pack_kernel<<<grid_for(rows * packed_bytes, 256), 256, 0, (cudaStream_t)stream>>>(codes, rows, n, bits, packed_bytes, packed);
  DARTKV_LAUNCH_OK("pack_kernel");
  return DARTKV_OK;
}

extern "C" int dartkv_unpack(const uint8_t* packed, int64_t rows, int64_t packed_bytes, int bits, int64_t count,
                             uint8_t* codes, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_bits(bits), "bits must be one of (2, 4, 8), got %d", bits);
  DARTKV_REQUIRE(rows >= 0 && count > 0 && count <= packed_bytes * (8 / bits), "unpack count exceeds the packed row");
  if (rows == 0) return DARTKV_OK;
  DARTKV_REQUIRE(codes && packed, "unpack received a null pointer");
  unpack_kernel<<<grid_for(rows * count, 256), 256, 0, (cudaStream_t)stream>>>(packed, rows, packed_bytes, bits, count, codes);
  DARTKV_LAUNCH_OK("unpack_kernel");
  return DARTKV_OK;
}

// ---------------------------------------------------------------------------- uniform quantizer
// One thread per (row, unit).  A unit is lcm(group, values-per-byte) consecutive codes, so it
// holds whole groups and whole bytes and no two threads share a byte.
struct QuantArgs {
  const void* x;
  int dtype;
  int64_t outer, n, inner, so, sn, si;
  int bits, group, md, div_mode;
  int64_t groups, padded, packed_bytes, unit, units;
  uint8_t* values;
  void* scale;
  void* zero;
  int32_t* nonfinite;
};

__global__ void quantize_kernel(QuantArgs a) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = a.outer * a.units * a.inner;
  if (tid >= total) return;
  int64_t i = tid % a.inner;
  int64_t u = (tid / a.inner) % a.units;
  int64_t o = tid / (a.inner * a.units);
  int64_t row = o * a.inner + i;
  const int64_t base = o * a.so + i * a.si;
  const int vpb = 8 / a.bits;
  const float qmax = (float)((1 << a.bits) - 1);
  int64_t begin = u * a.unit;
  int64_t end = min(begin + a.unit, a.padded);
  uint8_t* out = a.values + row * a.packed_bytes + begin / vpb;
  uint32_t acc = 0;
  int filled = 0;
  bool bad = false;
  for (int64_t g0 = begin; g0 < end; g0 += a.group) {
    float mn = INFINITY, mx = -INFINITY;
    for (int j = 0; j < a.group; ++j) {
      int64_t idx = min(g0 + j, a.n - 1);  // the last group is padded by repeating the final element
      float v = load_f(a.x, a.dtype, base + idx * a.sn);
      bad |= !isfinite(v);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
    float scale = group_scale(mn, mx, qmax, a.dtype, a.div_mode);
    int64_t g = g0 / a.group;
    store_f(a.scale, a.md, row * a.groups + g, scale);
    store_f(a.zero, a.md, row * a.groups + g, mn);
    for (int j = 0; j < a.group; ++j) {
      int64_t idx = min(g0 + j, a.n - 1);
      float v = load_f(a.x, a.dtype, base + idx * a.sn);
      acc |= group_code(v, mn, scale, qmax, a.dtype) << (filled * a.bits);
      if (++filled == vpb) {
        *out++ = (uint8_t)acc;
        acc = 0;
        filled = 0;
      }
    }
  }
  if (filled) *out = (uint8_t)acc;
  if (bad && a.nonfinite) *a.nonfinite = 1;
}

extern "C" int dartkv_quantize(const void* x, int dtype, int64_t outer, int64_t n, int64_t inner, int64_t stride_outer,
                               int64_t stride_n, int64_t stride_inner, int bits, int group_size, int md_dtype,
                               int div_mode, uint8_t* values, void* scale, void* zero, int32_t* nonfinite,
                               void* stream) {
  DARTKV_REQUIRE(dartkv_valid_bits(bits), "bits must be one of (2, 4, 8), got %d", bits);
  DARTKV_REQUIRE(group_size > 0, "group_size must be a positive integer, got %d", group_size);
  DARTKV_REQUIRE(dartkv_valid_dtype(dtype), "quantize expects a floating-point tensor (f32, f16 or bf16)");
  DARTKV_REQUIRE(dartkv_valid_dtype(md_dtype), "metadata dtype must be floating point (f32, f16 or bf16)");
  DARTKV_REQUIRE(n > 0, "quantize does not support an empty final dimension");
  DARTKV_REQUIRE(outer >= 0 && inner >= 0, "negative extent");
  DARTKV_REQUIRE(div_mode == DARTKV_DIV_TRUE || div_mode == DARTKV_DIV_RECIPROCAL, "unknown div_mode %d", div_mode);
  if (outer == 0 || inner == 0) return DARTKV_OK;
  DARTKV_REQUIRE(x && values && scale && zero, "quantize received a null pointer");
  QuantArgs a;
  a.x = x; a.dtype = dtype; a.outer = outer; a.n = n; a.inner = inner;
  a.so = stride_outer; a.sn = stride_n; a.si = stride_inner;
  a.bits = bits; a.group = group_size; a.md = md_dtype; a.div_mode = div_mode;
  a.groups = ceil_div64(n, group_size);
  a.padded = a.groups * group_size;
  int vpb = 8 / bits;
  a.packed_bytes = ceil_div64(a.padded, vpb);
  a.unit = (int64_t)group_size / dartkv_gcd(group_size, vpb) * vpb;
  a.units = ceil_div64(a.padded, a.unit);
  a.values = values; a.scale = scale; a.zero = zero; a.nonfinite = nonfinite;
  int64_t threads = outer * a.units * inner;
  quantize_kernel<<<grid_for(threads, 128), 128, 0, (cudaStream_t)stream>>>(a);
  DARTKV_LAUNCH_OK("quantize_kernel");
  return DARTKV_OK;
}

__global__ void dequantize_kernel(const uint8_t* __restrict__ values, const void* __restrict__ scale,
                                  const void* __restrict__ zero, int md, int64_t outer, int64_t n, int64_t inner,
                                  int bits, int group, int flavour, void* out, int out_dt, int64_t so, int64_t sn,
                                  int64_t si, int64_t groups, int64_t packed_bytes) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= outer * n * inner) return;
  int64_t i = tid % inner;
  int64_t j = (tid / inner) % n;
  int64_t o = tid / (inner * n);
  int64_t row = o * inner + i;
  int vpb = 8 / bits;
  uint32_t byte = values[row * packed_bytes + j / vpb];
  float code = (float)((byte >> ((j % vpb) * bits)) & ((1u << bits) - 1u));
  int64_t g = j / group;
  float s = load_f(scale, md, row * groups + g);
  float z = load_f(zero, md, row * groups + g);
  store_f(out, out_dt, o * so + j * sn + i * si, affine_restore(code, s, z, md, out_dt, flavour));
}

extern "C" int dartkv_dequantize(const uint8_t* values, const void* scale, const void* zero, int md_dtype,
                                 int64_t outer, int64_t n, int64_t inner, int bits, int group_size, int flavour,
                                 void* out, int out_dtype, int64_t stride_outer, int64_t stride_n,
                                 int64_t stride_inner, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_bits(bits), "bits must be one of (2, 4, 8), got %d", bits);
  DARTKV_REQUIRE(group_size > 0, "group_size must be a positive integer, got %d", group_size);
  DARTKV_REQUIRE(dartkv_valid_dtype(md_dtype) && dartkv_valid_dtype(out_dtype), "unsupported dtype");
  DARTKV_REQUIRE(flavour == DARTKV_DEQUANT_PER_OP || flavour == DARTKV_DEQUANT_FP32, "unknown dequant flavour %d", flavour);
  DARTKV_REQUIRE(n > 0 && outer >= 0 && inner >= 0, "bad extents");
  if (outer == 0 || inner == 0) return DARTKV_OK;
  DARTKV_REQUIRE(values && scale && zero && out, "dequantize received a null pointer");
  int64_t groups = ceil_div64(n, group_size);
  int64_t packed_bytes = ceil_div64(groups * group_size, 8 / bits);
  dequantize_kernel<<<grid_for(outer * n * inner, 256), 256, 0, (cudaStream_t)stream>>>(
      values, scale, zero, md_dtype, outer, n, inner, bits, group_size, flavour, out, out_dtype, stride_outer,
      stride_n, stride_inner, groups, packed_bytes);
  DARTKV_LAUNCH_OK("dequantize_kernel");
  return DARTKV_OK;
}

// ---------------------------------------------------------------------------- channel scores / selection
// Sums run in double: for 16-bit inputs the sum of |k| over a page is then exact, so the score
// does not depend on summation order (the reference accumulates in fp32, whose last-bit noise
// only matters at exact rounding boundaries).
__global__ void channel_scores_kernel(const void* __restrict__ keys, int dt, int64_t bh, int64_t tokens, int64_t d,
                                      int64_t sbh, int64_t st, int strategy, void* scores) {
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= bh * d) return;
  int64_t c = tid % d, r = tid / d;
  const int64_t base = r * sbh + c;
  float score;
  if (strategy == DARTKV_SCORE_MAGNITUDE) {
    double sum = 0.0;
    for (int64_t t = 0; t < tokens; ++t) sum += (double)fabsf(load_f(keys, dt, base + t * st));
    score = rnd_rt(__fdiv_rn((float)sum, (float)tokens), dt);
  } else {
    double sum = 0.0;
    for (int64_t t = 0; t < tokens; ++t) sum += (double)load_f(keys, dt, base + t * st);
    float mean = rnd_rt(__fdiv_rn((float)sum, (float)tokens), dt);
    double sq = 0.0;
    for (int64_t t = 0; t < tokens; ++t) {
      float centered = rnd_rt(__fsub_rn(load_f(keys, dt, base + t * st), mean), dt);
      sq += (double)rnd_rt(__fmul_rn(centered, centered), dt);
    }
    score = rnd_rt(__fdiv_rn((float)sq, (float)tokens), dt);
  }
  store_f(scores, dt, tid, score);
}

extern "C" int dartkv_channel_scores(const void* keys, int dtype, int64_t bh, int64_t tokens, int64_t head_dim,
                                     int64_t stride_bh, int64_t stride_token, int strategy, void* scores,
                                     void* stream) {
  DARTKV_REQUIRE(dartkv_valid_dtype(dtype), "key_states must be floating point");
  DARTKV_REQUIRE(tokens > 0 && head_dim > 0, "key_states sequence and head dimensions must be non-empty");
  DARTKV_REQUIRE(strategy == DARTKV_SCORE_MAGNITUDE || strategy == DARTKV_SCORE_VARIANCE,
                 "strategy must be 'magnitude', 'random', or 'variance'");
  if (bh == 0) return DARTKV_OK;
  DARTKV_REQUIRE(keys && scores, "channel_scores received a null pointer");
  channel_scores_kernel<<<grid_for(bh * head_dim, 128), 128, 0, (cudaStream_t)stream>>>(
      keys, dtype, bh, tokens, head_dim, stride_bh, stride_token, strategy, scores);
  DARTKV_LAUNCH_OK("channel_scores_kernel");
  return DARTKV_OK;
}

// rank by (score descending, channel ascending); one block per row
__global__ void select_channels_kernel(const void* __restrict__ scores, int dt, int64_t d, int count,
                                       int32_t* __restrict__ indices) {
  extern __shared__ float s_score[];
  int64_t r = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) s_score[c] = load_f(scores, dt, r * d + c);
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float mine = s_score[c];
    int rank = 0;
    for (int o = 0; o < d; ++o) {
      float other = s_score[o];
      rank += (other > mine) || (other == mine && o < c);
    }
    if (rank < count) indices[r * count + rank] = c;
  }
}

extern "C" int dartkv_select_channels(const void* scores, int dtype, int64_t bh, int64_t head_dim, int count,
                                      int32_t* indices, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_dtype(dtype), "scores must be floating point");
  DARTKV_REQUIRE(head_dim > 0 && head_dim <= 8192, "head_dim must be in [1, 8192]");
  DARTKV_REQUIRE(count >= 0 && count <= head_dim, "count must be in [0, head_dim]");
  if (bh == 0 || count == 0) return DARTKV_OK;
  DARTKV_REQUIRE(scores && indices, "select_channels received a null pointer");
  select_channels_kernel<<<(unsigned)bh, 128, head_dim * sizeof(float), (cudaStream_t)stream>>>(scores, dtype, head_dim,
                                                                                             count, indices);
  DARTKV_LAUNCH_OK("select_channels_kernel");
  return DARTKV_OK;
}

// ---------------------------------------------------------------------------- mixed key quantizer
// grid (bh, blocks over D*G); each block rebuilds the channel -> promoted-slot map of its row.
__global__ void quantize_key_mixed_kernel(const void* __restrict__ keys, int dt, int64_t tokens, int64_t d, int64_t sbh,
                                          int64_t st, int group, const int32_t* __restrict__ indices, int promoted,
                                          int md, uint8_t* __restrict__ low, uint8_t* __restrict__ high, void* scale,
                                          void* zero, int32_t* nonfinite) {
  extern __shared__ int s_slot[];
  int64_t r = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) s_slot[c] = -1;
  __syncthreads();
  for (int k = threadIdx.x; k < promoted; k += blockDim.x) {
    int c = indices[r * promoted + k];
    if (c >= 0 && c < d) s_slot[c] = k;
  }
  __syncthreads();
  int64_t groups = ceil_div64(tokens, group);
  int pb = ceil_div(group, 4);
  int64_t item = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= d * groups) return;
  int64_t c = item % d, g = item / d;
  int slot = s_slot[c];
  float qmax = slot >= 0 ? 15.0f : 3.0f;
  const int64_t base = r * sbh + c;
  float mn = INFINITY, mx = -INFINITY;
  bool bad = false;
  for (int j = 0; j < group; ++j) {
    int64_t t = min(g * group + j, tokens - 1);
    float v = load_f(keys, dt, base + t * st);
    bad |= !isfinite(v);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  float s = group_scale(mn, mx, qmax, dt, DARTKV_DIV_TRUE);
  store_f(scale, md, (r * d + c) * groups + g, s);
  store_f(zero, md, (r * d + c) * groups + g, mn);
  uint8_t* lo = low + ((r * d + c) * groups + g) * pb;
  uint8_t* hi = slot >= 0 ? high + ((r * promoted + slot) * groups + g) * pb : nullptr;
  uint32_t lacc = 0, hacc = 0;
  int filled = 0;
  for (int j = 0; j < group; ++j) {
    int64_t t = min(g * group + j, tokens - 1);
    uint32_t code = group_code(load_f(keys, dt, base + t * st), mn, s, qmax, dt);
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
  if (bad && nonfinite) *nonfinite = 1;
}

extern "C" int dartkv_quantize_key_mixed(const void* keys, int dtype, int64_t bh, int64_t tokens, int64_t head_dim,
                                         int64_t stride_bh, int64_t stride_token, int group_size,
                                         const int32_t* indices, int promoted, int md_dtype, uint8_t* low,
                                         uint8_t* high, void* scale, void* zero, int32_t* nonfinite, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_dtype(dtype), "key_states must be floating point");
  DARTKV_REQUIRE(dartkv_valid_dtype(md_dtype), "metadata_dtype must be floating point");
  DARTKV_REQUIRE(tokens > 0 && head_dim > 0, "key_states sequence and head dimensions must be non-empty");
  DARTKV_REQUIRE(group_size > 0, "group_size must be a positive integer");
  DARTKV_REQUIRE(head_dim <= 8192, "head_dim must be at most 8192");
  DARTKV_REQUIRE(promoted >= 0 && promoted <= head_dim, "promoted channel count must be in [0, head_dim]");
  if (bh == 0) return DARTKV_OK;
  DARTKV_REQUIRE(keys && low && scale && zero && (promoted == 0 || (indices && high)),
                 "quantize_key_mixed received a null pointer");
  int64_t groups = ceil_div64(tokens, group_size);
  dim3 grid((unsigned)bh, grid_for(head_dim * groups, 128));
  quantize_key_mixed_kernel<<<grid, 128, head_dim * sizeof(int), (cudaStream_t)stream>>>(
      keys, dtype, tokens, head_dim, stride_bh, stride_token, group_size, indices, promoted, md_dtype, low, high, scale,
      zero, nonfinite);
  DARTKV_LAUNCH_OK("quantize_key_mixed_kernel");
  return DARTKV_OK;
}

__global__ void dequantize_key_mixed_kernel(const uint8_t* __restrict__ low, const uint8_t* __restrict__ high,
                                            const int32_t* __restrict__ indices, const void* __restrict__ scale,
                                            const void* __restrict__ zero, int md, int64_t tokens, int64_t d, int group,
                                            int promoted, int flavour, void* out, int out_dt) {
  extern __shared__ int s_slot[];
  int64_t r = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) s_slot[c] = -1;
  __syncthreads();
  for (int k = threadIdx.x; k < promoted; k += blockDim.x) {
    int c = indices[r * promoted + k];
    if (c >= 0 && c < d) s_slot[c] = k;
  }
  __syncthreads();
  int64_t item = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (item >= tokens * d) return;
  int64_t c = item % d, t = item / d;
  int64_t groups = ceil_div64(tokens, group);
  int pb = ceil_div(group, 4);
  int64_t g = t / group;
  int j = (int)(t % group);
  uint32_t code = (low[((r * d + c) * groups + g) * pb + j / 4] >> ((j % 4) * 2)) & 3u;
  int slot = s_slot[c];
  if (slot >= 0) code |= ((high[((r * promoted + slot) * groups + g) * pb + j / 4] >> ((j % 4) * 2)) & 3u) << 2;
  float s = load_f(scale, md, (r * d + c) * groups + g);
  float z = load_f(zero, md, (r * d + c) * groups + g);
  store_f(out, out_dt, (r * tokens + t) * d + c, affine_restore((float)code, s, z, md, out_dt, flavour));
}

extern "C" int dartkv_dequantize_key_mixed(const uint8_t* low, const uint8_t* high, const int32_t* indices,
                                           const void* scale, const void* zero, int md_dtype, int64_t bh,
                                           int64_t tokens, int64_t head_dim, int group_size, int promoted, int flavour,
                                           void* out, int out_dtype, void* stream) {
  DARTKV_REQUIRE(dartkv_valid_dtype(md_dtype) && dartkv_valid_dtype(out_dtype), "unsupported dtype");
  DARTKV_REQUIRE(tokens > 0 && head_dim > 0 && head_dim <= 8192 && group_size > 0, "bad geometry");
  DARTKV_REQUIRE(promoted >= 0 && promoted <= head_dim, "promoted channel count must be in [0, head_dim]");
  DARTKV_REQUIRE(flavour == DARTKV_DEQUANT_PER_OP || flavour == DARTKV_DEQUANT_FP32, "unknown dequant flavour %d", flavour);
  if (bh == 0) return DARTKV_OK;
  DARTKV_REQUIRE(low && scale && zero && out && (promoted == 0 || (indices && high)),
                 "dequantize_key_mixed received a null pointer");
  dim3 grid((unsigned)bh, grid_for(tokens * head_dim, 256));
  dequantize_key_mixed_kernel<<<grid, 256, head_dim * sizeof(int), (cudaStream_t)stream>>>(
      low, high, indices, scale, zero, md_dtype, tokens, head_dim, group_size, promoted, flavour, out, out_dtype);
  DARTKV_LAUNCH_OK("dequantize_key_mixed_kernel");
  return DARTKV_OK;
}
