// Fused single-token decode attention over the device-resident paged cache.
//
// Split-K over the token range: every (batch, KV head, split) block keeps an fp32 online-softmax
// state (m, l, acc) for the query heads of its KV head (GQA group) and writes one partial; a merge
// kernel combines the partials, normalizes and casts.  Numerics follow the reference's
// page-streaming attention (src/dart/attention.py:60-87): dequantize to the cache dtype, fp32
// logits q.k * scale, fp32 online softmax, acc / max(l, 1e-20), cast to the query dtype.
//
// This file holds the generic kernel (any page geometry, bit width, dtype; CUDA-core fp32 math)
// and the merge; the tensor-core kernel for the headline geometry is in decode_fast.cu.

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

#define GEN_THREADS 128
#define GEN_TILE 32
#define GEN_MAX_REP 16
#define GEN_MAX_D 256

__device__ __forceinline__ int gen_find_page(const dartkv_cache_desc& d, int pages, int t) {
  int lo = 0, hi = pages - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (d.page_start[mid] + d.page_tokens[mid] > t) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// Tokens [sink_tokens, fast_range_end) are whole pages packed on both the key and the value side.
__host__ __device__ __forceinline__ int dartkv_fast_range_end(int sink_tokens, int page_size, int k_end, int v_end,
                                                              int sink_filled) {
  int packed = min(k_end, v_end);
  if (packed <= sink_tokens) return sink_filled;
  return sink_tokens + (packed - sink_tokens) / page_size * page_size;
}

struct GenericArgs {
  const void* q;
  int q_dt, query_heads, flavour;
  float scale;
  int tok_begin, tok_end;   // tok_end < 0: up to the number of tokens seen
  int chunk, split_base, total_splits;
  float* part_m;
  float* part_l;
  float* part_acc;
  const int32_t* row_start;   // optional [batch] first live token of every batch row
};

__global__ void __launch_bounds__(GEN_THREADS) decode_generic_kernel(dartkv_cache_desc d, GenericArgs a) {
  extern __shared__ float smem[];
  const int D = d.head_dim, DP = D + 1;
  const int rep = a.query_heads / d.kv_heads;
  float* s_q = smem;                              // [rep][D]
  float* s_tile = s_q + rep * D;                  // [GEN_TILE][D+1]
  float* s_p = s_tile + GEN_TILE * DP;            // [rep][GEN_TILE]
  float* s_alpha = s_p + rep * GEN_TILE;          // [rep]
  float* s_m = s_alpha + rep;                     // [rep]
  float* s_l = s_m + rep;                         // [rep]
  int* s_slot = reinterpret_cast<int*>(s_l + rep);// [D]

  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / d.kv_heads, h = bh % d.kv_heads;
  const int tid = threadIdx.x;
  const int seen = d.state[0], pages = d.state[1], k_end = d.state[2], v_end = d.state[3], sink_filled = d.state[4];
  const int end = a.tok_end < 0 ? seen : min(a.tok_end, seen);
  // tok_begin < 0: start where the tensor-core kernel stops (last full page packed on both sides)
  int begin = a.tok_begin;
  if (begin < 0) begin = dartkv_fast_range_end(d.sink_tokens, d.page_size, k_end, v_end, sink_filled);
  const int first = begin + split * a.chunk;
  const int hi = (int)min((int64_t)first + a.chunk, (int64_t)end);
  // left padding: the tokens before the row's first live one get no weight (a split wholly before it stays empty)
  const int lo = a.row_start ? max(first, a.row_start[b]) : first;

  for (int i = tid; i < rep * D; i += GEN_THREADS) {
    int r = i / D, c = i % D;
    s_q[i] = load_f(a.q, a.q_dt, ((int64_t)b * a.query_heads + h * rep + r) * D + c);
  }
  if (tid < rep) { s_m[tid] = -INFINITY; s_l[tid] = 0.0f; }
  float acc[GEN_MAX_REP][GEN_MAX_D / GEN_THREADS];
#pragma unroll
  for (int r = 0; r < GEN_MAX_REP; ++r)
#pragma unroll
    for (int k = 0; k < GEN_MAX_D / GEN_THREADS; ++k) acc[r][k] = 0.0f;
  __syncthreads();

  // A packed value segment [vs, ve) (page_size tokens from sink_tokens on, the last one ending at the packed end)
  // that a key-segment boundary cuts is materialized by the reference with its per-op dequantization: the key
  // boundaries are the page edges and the end of the packed keys.
  auto value_flavour = [&](int tok) -> int {
    if (a.flavour == DARTKV_DEQUANT_PER_OP || d.regular_pages) return a.flavour;   // regular pages share the value edges
    const int vs = d.sink_tokens + (tok - d.sink_tokens) / d.page_size * d.page_size;
    const int ve = min(v_end, vs + d.page_size);
    if (vs >= k_end) return a.flavour;
    const int pg = gen_find_page(d, pages, vs);
    return d.page_start[pg] + d.page_tokens[pg] < ve ? DARTKV_DEQUANT_PER_OP : a.flavour;
  };
  int t = lo;
  while (t < hi) {
    // ---- locate the key segment that holds token t
    int seg_end, kind, page_first = 0, page_n = 0;
    int key_flavour = a.flavour;
    const uint8_t* page = nullptr;
    if (t < sink_filled) {
      kind = 0; seg_end = min(hi, sink_filled);
    } else if (t < k_end) {
      kind = 1;
      int pg = gen_find_page(d, pages, t);
      page_first = d.page_start[pg];
      page_n = d.page_tokens[pg];
      seg_end = min(hi, page_first + page_n);
      page = d.k_pages + ((int64_t)bh * d.max_key_pages + pg) * d.key_page_bytes;
      // A key page that a value-segment boundary cuts is materialized by the reference with its per-op
      // dequantization whatever the device (src/dart/cache.py:557-560); only whole pages reach its fp32 kernels.
      // Value boundaries: sink_tokens + i * page_size below the packed end of the values, and that end itself.
      if (a.flavour != DARTKV_DEQUANT_PER_OP && page_first < v_end) {
        const int next_value_edge = d.sink_tokens + ((page_first - d.sink_tokens) / d.page_size + 1) * d.page_size;
        if (min(next_value_edge, v_end) < page_first + page_n) key_flavour = DARTKV_DEQUANT_PER_OP;
      }
      if (d.key_mode == DARTKV_MIXED_PAGE) {
        __syncthreads();
        for (int c = tid; c < D; c += GEN_THREADS) s_slot[c] = -1;
        __syncthreads();
        const int32_t* idx = reinterpret_cast<const int32_t*>(page + d.key_off_index);
        for (int k = tid; k < d.promoted; k += GEN_THREADS) {
          int c = idx[k];
          if (c >= 0 && c < D) s_slot[c] = k;
        }
        __syncthreads();
      }
    } else {
      kind = 2; seg_end = hi;
    }
    for (int tile0 = t; tile0 < seg_end; tile0 += GEN_TILE) {
      const int nt = min(GEN_TILE, seg_end - tile0);
      // ---- K tile, dequantized to the cache dtype
      for (int i = tid; i < nt * D; i += GEN_THREADS) {
        int tt = i / D, c = i % D, tok = tile0 + tt;
        float v;
        if (kind == 0) v = load_f(d.k_sink, d.dtype, ((int64_t)bh * d.sink_tokens + tok) * D + c);
        else if (kind == 2) v = load_f(d.k_ring, d.dtype, ((int64_t)bh * d.ring_tokens + (tok % d.ring_tokens)) * D + c);
        else {
          const int Gk = d.key_group, G = ceil_div(page_n, Gk), j = tok - page_first, g = j / Gk;
          float s = load_f(page + d.key_off_scale, d.md_dtype, c * G + g);
          float z = load_f(page + d.key_off_zero, d.md_dtype, c * G + g);
          uint32_t code;
          if (d.key_mode == DARTKV_MIXED_PAGE) {
            const int pb = ceil_div(Gk, 4), jj = j % Gk, slot = s_slot[c];
            code = (page[(c * G + g) * pb + jj / 4] >> ((jj % 4) * 2)) & 3u;
            if (slot >= 0) code |= ((page[d.key_off_high + (slot * G + g) * pb + jj / 4] >> ((jj % 4) * 2)) & 3u) << 2;
          } else {
            const int bits = d.key_bits, vpb = 8 / bits, row_bytes = ceil_div(G * Gk, vpb);
            code = (page[(int64_t)c * row_bytes + j / vpb] >> ((j % vpb) * bits)) & ((1u << bits) - 1u);
          }
          v = affine_restore((float)code, s, z, d.md_dtype, d.dtype, key_flavour);
        }
        s_tile[tt * DP + c] = v;
      }
      __syncthreads();
      // ---- logits
      for (int i = tid; i < rep * nt; i += GEN_THREADS) {
        int r = i / nt, tt = i % nt;
        const float* qr = s_q + r * D;
        const float* kr = s_tile + tt * DP;
        float dot = 0.0f;
        for (int c = 0; c < D; ++c) dot = fmaf(qr[c], kr[c], dot);
        s_p[r * GEN_TILE + tt] = dot * a.scale;
      }
      __syncthreads();
      // ---- online softmax state per query head
      if (tid < rep) {
        float* pr = s_p + tid * GEN_TILE;
        float mx = -INFINITY;
        for (int tt = 0; tt < nt; ++tt) mx = fmaxf(mx, pr[tt]);
        float m_old = s_m[tid], m_new = fmaxf(m_old, mx);
        float alpha = expf(m_old - m_new);
        float sum = 0.0f;
        for (int tt = 0; tt < nt; ++tt) { float p = expf(pr[tt] - m_new); pr[tt] = p; sum += p; }
        s_alpha[tid] = alpha;
        s_m[tid] = m_new;
        s_l[tid] = s_l[tid] * alpha + sum;
      }
      __syncthreads();
      // ---- V tile
      for (int i = tid; i < nt * D; i += GEN_THREADS) {
        int tt = i / D, c = i % D, tok = tile0 + tt;
        float v;
        if (tok < sink_filled) v = load_f(d.v_sink, d.dtype, ((int64_t)bh * d.sink_tokens + tok) * D + c);
        else if (tok >= v_end) v = load_f(d.v_ring, d.dtype, ((int64_t)bh * d.ring_tokens + (tok % d.ring_tokens)) * D + c);
        else {
          int64_t row = (int64_t)bh * d.max_value_tokens + (tok - d.sink_tokens);
          const int bits = d.value_bits, vpb = 8 / bits, g = c / d.value_group;
          uint32_t code = (d.v_codes[row * d.value_row_bytes + c / vpb] >> ((c % vpb) * bits)) & ((1u << bits) - 1u);
          float s = load_f(d.v_meta, d.md_dtype, (row * 2 + 0) * d.value_groups + g);
          float z = load_f(d.v_meta, d.md_dtype, (row * 2 + 1) * d.value_groups + g);
          v = affine_restore((float)code, s, z, d.md_dtype, d.dtype, value_flavour(tok));
        }
        s_tile[tt * DP + c] = v;
      }
      __syncthreads();
      // ---- accumulate
#pragma unroll
      for (int k = 0; k < GEN_MAX_D / GEN_THREADS; ++k) {
        int c = tid + k * GEN_THREADS;
        if (c < D) {
#pragma unroll
          for (int r = 0; r < GEN_MAX_REP; ++r) {
            if (r < rep) {
              float sum = 0.0f;
              const float* pr = s_p + r * GEN_TILE;
              for (int tt = 0; tt < nt; ++tt) sum = fmaf(pr[tt], s_tile[tt * DP + c], sum);
              acc[r][k] = acc[r][k] * s_alpha[r] + sum;
            }
          }
        }
      }
      __syncthreads();
    }
    t = seg_end;
  }

  const int slot = a.split_base + split;
#pragma unroll
  for (int r = 0; r < GEN_MAX_REP; ++r) {
    if (r < rep) {
      int64_t row = ((int64_t)b * a.query_heads + h * rep + r) * a.total_splits + slot;
      if (tid == 0) { a.part_m[row] = s_m[r]; a.part_l[row] = s_l[r]; }
#pragma unroll
      for (int k = 0; k < GEN_MAX_D / GEN_THREADS; ++k) {
        int c = tid + k * GEN_THREADS;
        if (c < D) a.part_acc[row * D + c] = acc[r][k];
      }
    }
  }
}

// one block per (batch, query head): combine split partials, normalize, cast
// With stream_blocks > 0 (tensor-core layouts) a row's valid slots are its dense slot 0 plus one per stream block
// that touched its (batch, kv head); the remaining slots of the row hold stale data and are skipped.
// With peers.world_size > 1 the normalized rows are also stored into every rank's gathered output tensor (plain
// stores through peer-mapped pointers over NVLink), and the block that finishes last publishes this rank's arrival
// flag on every peer and then waits, with a bound, for every peer's flag on this rank: when the kernel ends, the
// gathered tensor of this rank is complete.  Nothing here waits on another kernel of the same GPU.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void decode_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                    const float* __restrict__ part_acc, int total_splits, int D, void* out, int out_dt,
                                    int stream_blocks, int64_t units, int quads, int query_heads, int kv_heads,
                                    dartkv_peer_scatter peers, int* status, unsigned int* done_counter) {
  // launched with programmatic stream serialization: the grid may become resident while the kernel before it
  // drains, and waits here until that kernel's memory is visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  int64_t row = blockIdx.x;
  int splits = total_splits;
  if (stream_blocks > 0) {
    const int rep = query_heads / kv_heads;
    const int64_t bh = (row / query_heads) * kv_heads + (row % query_heads) / rep;
    splits = 2 + dartkv_block_of_unit(bh * quads + quads - 1, stream_blocks, units) -
             dartkv_block_of_unit(bh * quads, stream_blocks, units);
  }
  part_m += row * (total_splits - splits);   // rows are total_splits slots apart, the loops below index row * splits
  part_l += row * (total_splits - splits);
  part_acc += row * (total_splits - splits) * D;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_m[row * splits + s]);
  float l = 0.0f;
  for (int s = 0; s < splits; ++s) {
    float ms = part_m[row * splits + s];
    if (ms != -INFINITY) l += part_l[row * splits + s] * expf(ms - m);
  }
  float inv = 1.0f / fmaxf(l, 1e-20f);
  const int64_t out_row = blockIdx.x;
  const int64_t peer_row = (int64_t)(peers.dst_row_begin + out_row / query_heads) * peers.dst_heads_total +
                           peers.dst_head_begin + out_row % query_heads;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) {
      float ms = part_m[row * splits + s];
      if (ms != -INFINITY) acc += part_acc[(row * splits + s) * D + c] * expf(ms - m);
    }
    store_f(out, out_dt, out_row * D + c, acc * inv);
    for (int p = 0; p < peers.world_size; ++p) store_f(peers.out[p], out_dt, peer_row * D + c, acc * inv);
  }
  if (peers.world_size > 1) {
    // the block's peer stores are ordered before the barrier; one cumulative system-scope fence after it makes
    // them all visible system-wide before the block reports in (a fence per thread costs microseconds per wave)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int ticket = atomicAdd(done_counter, 1u);
      if (ticket == gridDim.x - 1) {
        *done_counter = 0;      // ready for the next call on this stream
        __threadfence_system();
        for (int p = 0; p < peers.world_size; ++p) st_release_sys(peers.flags[p] + peers.rank, peers.epoch);
        // every peer's rows have landed here once its flag shows this step (or a later one)
        bool ok = true;
        for (int p = 0; p < peers.world_size && ok; ++p) {
          ok = false;
          for (int spin = 0; spin < (1 << 21); ++spin) {   // about half a second with the sleep below
            if ((int)(ld_acquire_sys(peers.flags[peers.rank] + p) - peers.epoch) >= 0) { ok = true; break; }
            __nanosleep(200);
          }
        }
        if (!ok) atomicExch(status, 2);
      }
    }
  }
}

// ---------------------------------------------------------------------------- host side
struct DecodeLayout {
  int generic_splits, generic_chunk;   // generic kernel over the whole range (fallback)
  int fast;                            // tensor-core kernel for the packed pages: 1 per-op rounded, 2 unrounded fp32
  int quads, stream_blocks;            // tensor-core layouts: four-page units per (batch, kv head), stream blocks
  long long units;
  int total_splits;
};

int dartkv_decode_fast_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads);
int dartkv_decode_fast_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
                              int flavour, int quads, int stream_blocks, long long units, int total_splits,
                              float* part_m, float* part_l, float* part_acc, int* status, const int32_t* row_start,
                              cudaStream_t stream);
int dartkv_decode_fused32_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads);
int dartkv_decode_fused32_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
                                 int flavour, int quads, int stream_blocks, long long units, int total_splits,
                                 float* part_m, float* part_l, float* part_acc, int* status, const int32_t* row_start,
                              cudaStream_t stream);

int dartkv_decode_wide_supported(const dartkv_cache_desc* d, int q_dtype, int query_heads);
int dartkv_decode_wide_blocks_per_sm(const dartkv_cache_desc* d);
int dartkv_decode_wide_launch(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads, float scale,
                              int flavour, int quads, int stream_blocks, long long units, int total_splits,
                              float* part_m, float* part_l, float* part_acc, int* status, const int32_t* row_start,
                              cudaStream_t stream);

static int dartkv_sm_count() {
  // per device: a process may drive GPUs of different sizes
  static std::atomic<int> cached[64];
  int device = 0, count = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  count = cached[device].load(std::memory_order_relaxed);
  if (count == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 148;   // B200
    cached[device].store(count, std::memory_order_relaxed);
  }
  return count;
}

// work-split override: a debugging / testing knob, kept off the per-call path (the environment is read once)
static char g_split_override[64] = "";
static bool g_split_override_ready = false;
static const char* split_override() {
  if (!g_split_override_ready) {
    const char* env = getenv("DARTKV_DECODE_SPLIT");
    if (env) { strncpy(g_split_override, env, sizeof(g_split_override) - 1); g_split_override[sizeof(g_split_override) - 1] = 0; }
    g_split_override_ready = true;
  }
  return g_split_override[0] ? g_split_override : nullptr;
}
extern "C" int dartkv_decode_split_override(const char* spec) {
  g_split_override_ready = true;
  g_split_override[0] = 0;
  if (spec) { strncpy(g_split_override, spec, sizeof(g_split_override) - 1); g_split_override[sizeof(g_split_override) - 1] = 0; }
  return DARTKV_OK;
}

static DecodeLayout decode_layout(const dartkv_cache_desc* d, int q_dtype, int query_heads, int flavour, int tokens) {
  DecodeLayout L{};
  const int bh = d->batch * d->kv_heads;
  L.fast = 0;
  if (flavour == DARTKV_DEQUANT_PER_OP && dartkv_decode_fast_supported(d, q_dtype, query_heads)) L.fast = 1;
  if (flavour == DARTKV_DEQUANT_FUSED && dartkv_decode_fused32_supported(d, q_dtype, query_heads)) L.fast = 2;
  // every other packed geometry with 128-token pages and head_dim 128, and the fp32 flavour of all of them
  if (!L.fast && flavour != DARTKV_DEQUANT_FUSED && dartkv_decode_wide_supported(d, q_dtype, query_heads)) L.fast = 3;
  // the tensor-core kernels index (row, four-page unit) pairs with 32 bits
  if (L.fast && (long long)bh * ((max(1, (tokens - d->sink_tokens) / d->page_size) + 3) / 4) >= (1ll << 31)) L.fast = 0;
  if (L.fast) {
    // One unit = four consecutive pages of a (batch, kv head) (a block hands them to its four warp pairs).  The
    // units of all rows are dealt out evenly to `stream_blocks` blocks.  Two families of splits are compared with a
    // cost model in units of one page per pair (a block costs its pages per pair plus 1.75 per row it touches:
    // query load, first-page latency, merge of its eight warps; the dense block of a row about 2; blocks run in
    // waves of two per SM; constants fitted to B200 timings):
    //   aligned    rows * s blocks, s = 1..16 pieces per row;
    //   unaligned  one block per resident slot, a block may finish one row and start the next (at most 16 blocks
    //              touch a row); measured ~3 % slower per unit than aligned blocks, but it fills every slot when
    //              the rows do not (e.g. 256 rows on 296 slots: 9 % faster at context 32768).
    const int pages = max(1, (tokens - d->sink_tokens) / d->page_size);
    L.quads = (pages + 3) / 4;
    L.units = (long long)bh * L.quads;
    const int resident = (L.fast == 3 ? dartkv_decode_wide_blocks_per_sm(d) : 2) * dartkv_sm_count();
    const double block_fixed = 1.75, dense_cost = 2.0;
    int best_pieces = 1;
    double best_cost = 1e30;
    for (int q = max(1, (L.quads + 15) / 16); q <= L.quads; ++q) {
      const int pieces = (L.quads + q - 1) / q;
      const long long blocks = (long long)bh * pieces;
      const long long waves = (blocks + resident - 1) / resident;
      const double by_waves = (double)waves * (q + block_fixed);
      const double by_work = (double)bh * (pieces * (q + block_fixed) + dense_cost) / resident;
      const double cost = by_waves > by_work ? by_waves : by_work;
      if (cost < best_cost - 1e-9) { best_cost = cost; best_pieces = pieces; }
    }
    L.stream_blocks = bh * best_pieces;
    L.total_splits = best_pieces + 1;
    {
      const long long min_share = (L.quads + 14) / 15;
      long long blocks = resident;
      if (blocks > L.units / min_share) blocks = L.units / min_share;
      // "aligned" | "unaligned" | "unaligned:<blocks>" overrides the model (tests exercise both families, and
      // blocks that span several rows, with it): set through dartkv_decode_split_override(), or once per process
      // from the environment variable DARTKV_DECODE_SPLIT
      const char* force = split_override();
      const bool force_unaligned = force && force[0] == 'u', force_aligned = force && force[0] == 'a';
      if (force_unaligned && strchr(force, ':')) {
        const long long wanted = atoll(strchr(force, ':') + 1);
        if (wanted >= 1 && wanted < blocks) blocks = wanted;
      }
      if (blocks >= 1 && !force_aligned) {
        const double share = (double)L.units / blocks;
        const double cost = 1.03 * (share + block_fixed * (share / L.quads + 1.0)) + (double)bh * dense_cost / resident;
        if (cost < best_cost || force_unaligned) {
          const long long w = L.units / blocks;   // smallest share of a block
          L.stream_blocks = (int)blocks;
          L.total_splits = (int)((L.quads + w - 2) / w + 1) + 1;
        }
      }
    }
  } else {
    int max_splits = max(1, (tokens + 63) / 64);
    int want = max(1, (148 * 4 + bh - 1) / bh);
    L.generic_splits = min(want, max_splits);
    int chunk = (tokens + L.generic_splits - 1) / L.generic_splits;
    L.generic_chunk = max(GEN_TILE, (chunk + GEN_TILE - 1) / GEN_TILE * GEN_TILE);
    L.generic_splits = max(1, (tokens + L.generic_chunk - 1) / L.generic_chunk);
    L.total_splits = L.generic_splits;
  }
  return L;
}

static int64_t layout_bytes(const dartkv_cache_desc* d, int query_heads, const DecodeLayout& L) {
  int64_t rows = (int64_t)d->batch * query_heads * L.total_splits;
  return 16 + rows * (2 + d->head_dim) * (int64_t)sizeof(float);
}

extern "C" int64_t dartkv_decode_workspace_bytes(const dartkv_cache_desc* d, int query_heads, int max_tokens) {
  if (!d || query_heads <= 0 || max_tokens <= 0) return 0;
  // upper bound over query dtypes, dequant flavours and every token count up to max_tokens
  int64_t best = 0;
  for (int dt = 0; dt < 3; ++dt)
    for (int flavour = 0; flavour < 3; ++flavour) {
      DecodeLayout L = decode_layout(d, dt, query_heads, flavour, max_tokens);
      // the tensor-core layouts use at most 16 stream slots + 1 dense slot per row whatever the token count
      if (L.fast) L.total_splits = 17;
      best = max(best, layout_bytes(d, query_heads, L));
    }
  // The generic layout may serve any smaller token count (and is what a tensor-core cache falls back to for other
  // query dtypes).  Its split count is not monotonic in the token count, because the chunk is rounded up to whole
  // tiles, but it never exceeds min(blocks wanted, tokens / 64 rounded up): rounding the chunk up only lowers it.
  {
    const int bh = d->batch * d->kv_heads;
    DecodeLayout L{};
    L.total_splits = min(max(1, (148 * 4 + bh - 1) / bh), max(1, (max_tokens + 63) / 64));
    best = max(best, layout_bytes(d, query_heads, L));
  }
  return best;
}

extern "C" int dartkv_decode_plan(const dartkv_cache_desc* d, int q_dtype, int query_heads, int flavour, int tokens,
                                  dartkv_decode_plan_info* out) {
  DARTKV_REQUIRE(d != nullptr && out != nullptr, "decode_plan received a null pointer");
  DARTKV_REQUIRE(dartkv_valid_dtype(q_dtype), "query must be f32, f16 or bf16");
  DARTKV_REQUIRE(query_heads > 0 && query_heads % d->kv_heads == 0, "query heads must be divisible by cache KV heads");
  DARTKV_REQUIRE(tokens > 0, "cache is empty");
  DARTKV_REQUIRE(flavour >= DARTKV_DEQUANT_PER_OP && flavour <= DARTKV_DEQUANT_FUSED, "unknown dequant flavour %d", flavour);
  const DecodeLayout L = decode_layout(d, q_dtype, query_heads, flavour, tokens);
  out->kernel = L.fast;
  out->quads = L.fast ? L.quads : 0;
  out->stream_blocks = L.fast ? L.stream_blocks : 0;
  out->total_splits = L.total_splits;
  out->units = L.fast ? L.units : 0;
  out->generic_splits = L.fast ? 0 : L.generic_splits;
  out->generic_chunk = L.fast ? 0 : L.generic_chunk;
  return DARTKV_OK;
}

extern "C" int dartkv_decode_status(const void* workspace, int* status_out, void* stream) {
  DARTKV_REQUIRE(workspace && status_out, "decode_status received a null pointer");
  DARTKV_CUDA_OK(cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  DARTKV_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return DARTKV_OK;
}

static int decode_attention_impl(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads,
                                 float scale, int flavour, int tokens, void* workspace, int64_t workspace_bytes,
                                 void* out, const dartkv_peer_scatter* peers, const int32_t* row_start,
                                 void* stream_) {
  DARTKV_REQUIRE(d != nullptr, "null descriptor");
  DARTKV_REQUIRE(query && out && workspace, "decode_attention received a null pointer");
  DARTKV_REQUIRE(dartkv_valid_dtype(q_dtype), "query must be f32, f16 or bf16");
  DARTKV_REQUIRE(query_heads > 0 && query_heads % d->kv_heads == 0, "query heads must be divisible by cache KV heads");
  DARTKV_REQUIRE(tokens > 0, "cache is empty");
  DARTKV_REQUIRE(flavour >= DARTKV_DEQUANT_PER_OP && flavour <= DARTKV_DEQUANT_FUSED, "unknown dequant flavour %d", flavour);
  const int rep = query_heads / d->kv_heads;
  DARTKV_REQUIRE(rep <= GEN_MAX_REP, "at most %d query heads per KV head are supported", GEN_MAX_REP);
  DARTKV_REQUIRE(d->head_dim <= GEN_MAX_D, "decode attention supports head_dim up to %d", GEN_MAX_D);
  cudaStream_t stream = (cudaStream_t)stream_;
  DecodeLayout L = decode_layout(d, q_dtype, query_heads, flavour, tokens);
  const int64_t rows = (int64_t)d->batch * query_heads * L.total_splits;
  DARTKV_REQUIRE(workspace_bytes >= layout_bytes(d, query_heads, L), "decode workspace too small: need %lld bytes",
                 (long long)layout_bytes(d, query_heads, L));
  int* status = reinterpret_cast<int*>(workspace);
  float* part_m = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 16);
  float* part_l = part_m + rows;
  float* part_acc = part_l + rows;
  const int bh = d->batch * d->kv_heads;
  const int D = d->head_dim;
  if (L.fast) {
    int rc = (L.fast == 3 ? dartkv_decode_wide_launch : L.fast == 2 ? dartkv_decode_fused32_launch : dartkv_decode_fast_launch)(
        d, query, q_dtype, query_heads, scale, flavour, L.quads, L.stream_blocks, L.units, L.total_splits, part_m,
        part_l, part_acc, status, row_start, stream);
    if (rc) return rc;
  } else {
    size_t smem = ((size_t)rep * D + (size_t)GEN_TILE * (D + 1) + (size_t)rep * GEN_TILE + 3 * rep) * sizeof(float) +
                  (size_t)D * sizeof(int);
    GenericArgs a;
    a.q = query; a.q_dt = q_dtype; a.query_heads = query_heads; a.flavour = flavour; a.scale = scale;
    a.total_splits = L.total_splits; a.part_m = part_m; a.part_l = part_l; a.part_acc = part_acc;
    a.tok_begin = 0; a.tok_end = -1; a.chunk = L.generic_chunk; a.split_base = 0;
    a.row_start = row_start;
    if (smem > 48 * 1024)
      DARTKV_CUDA_OK(cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    DARTKV_REQUIRE(L.generic_splits <= 65535, "too many splits");
    decode_generic_kernel<<<dim3(bh, L.generic_splits), GEN_THREADS, smem, stream>>>(*d, a);
    DARTKV_LAUNCH_OK("decode_generic_kernel");
  }
  {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)((int64_t)d->batch * query_heads));
    config.blockDim = dim3(128);
    config.stream = stream;
    cudaLaunchAttribute attribute = {};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    dartkv_peer_scatter none{};
    unsigned int* done_counter = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(workspace) + 4);
    DARTKV_CUDA_OK(cudaLaunchKernelEx(&config, decode_merge_kernel, (const float*)part_m, (const float*)part_l,
                                      (const float*)part_acc, L.total_splits, D, out, q_dtype,
                                      L.fast ? L.stream_blocks : 0, (int64_t)L.units, L.quads, query_heads, d->kv_heads,
                                      peers ? *peers : none, status, done_counter));
  }
  DARTKV_LAUNCH_OK("decode_merge_kernel");
  return DARTKV_OK;
}

extern "C" int dartkv_decode_attention(const dartkv_cache_desc* d, const void* query, int q_dtype, int query_heads,
                                       float scale, int flavour, int tokens, void* workspace,
                                       int64_t workspace_bytes, void* out, void* stream) {
  return decode_attention_impl(d, query, q_dtype, query_heads, scale, flavour, tokens, workspace, workspace_bytes, out,
                               nullptr, nullptr, stream);
}

extern "C" int dartkv_decode_attention_padded(const dartkv_cache_desc* d, const void* query, int q_dtype,
                                              int query_heads, float scale, int flavour, int tokens,
                                              const int32_t* row_start, void* workspace, int64_t workspace_bytes,
                                              void* out, void* stream) {
  return decode_attention_impl(d, query, q_dtype, query_heads, scale, flavour, tokens, workspace, workspace_bytes, out,
                               nullptr, row_start, stream);
}

extern "C" int dartkv_decode_attention_scatter(const dartkv_cache_desc* d, const void* query, int q_dtype,
                                               int query_heads, float scale, int flavour, int tokens, void* workspace,
                                               int64_t workspace_bytes, void* out, const dartkv_peer_scatter* peers,
                                               void* stream) {
  DARTKV_REQUIRE(peers != nullptr, "decode_attention_scatter received a null pointer");
  DARTKV_REQUIRE(peers->world_size >= 1 && peers->world_size <= DARTKV_MAX_PEERS, "world_size must be in [1, %d]",
                 DARTKV_MAX_PEERS);
  DARTKV_REQUIRE(peers->rank >= 0 && peers->rank < peers->world_size, "rank must be in [0, world_size)");
  DARTKV_REQUIRE(peers->dst_row_begin >= 0 && peers->dst_head_begin >= 0 &&
                     peers->dst_head_begin + query_heads <= peers->dst_heads_total,
                 "the rows of this rank do not fit the gathered tensor");
  for (int p = 0; p < peers->world_size; ++p)
    DARTKV_REQUIRE(peers->out[p] != nullptr && peers->flags[p] != nullptr, "peer %d has a null pointer", p);
  return decode_attention_impl(d, query, q_dtype, query_heads, scale, flavour, tokens, workspace, workspace_bytes, out,
                               peers, nullptr, stream);
}

// ---------------------------------------------------------------------------- built-in scratch variant
// Split-K scratch that lives in the library image instead of caller memory.  Every device that
// loads the library carries these 32 MiB until the process exits.
#define DARTKV_BUILTIN_SCRATCH_BYTES (32ll << 20)
static __device__ __align__(256) unsigned char g_builtin_scratch[DARTKV_BUILTIN_SCRATCH_BYTES];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kMaxDevices] = {};   // device address of g_builtin_scratch, per device ordinal
}  // namespace

// In host code `g_builtin_scratch` is only a handle for the symbol, not memory a kernel can use:
// the device address has to be asked for, with the target device current, once per device.
static int builtin_scratch_address(void** out) {
  int device = -1;
  DARTKV_CUDA_OK(cudaGetDevice(&device));
  DARTKV_REQUIRE(device >= 0 && device < kMaxDevices, "device ordinal %d is outside the supported range", device);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    DARTKV_CUDA_OK(cudaGetSymbolAddress(&address, g_builtin_scratch));
    DARTKV_REQUIRE(address != nullptr, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return DARTKV_OK;
}

extern "C" int64_t dartkv_builtin_scratch_bytes(void) { return DARTKV_BUILTIN_SCRATCH_BYTES; }

extern "C" int dartkv_decode_attention_builtin_scratch(const dartkv_cache_desc* d, const void* query, int q_dtype,
                                                       int query_heads, float scale, int flavour, int tokens,
                                                       void* out, void* stream) {
  DARTKV_REQUIRE(d != nullptr, "null descriptor");
  DARTKV_REQUIRE(dartkv_valid_dtype(q_dtype), "query must be f32, f16 or bf16");
  DARTKV_REQUIRE(query_heads > 0 && query_heads % d->kv_heads == 0, "query heads must be divisible by cache KV heads");
  DARTKV_REQUIRE(tokens > 0, "cache is empty");
  DARTKV_REQUIRE(flavour >= DARTKV_DEQUANT_PER_OP && flavour <= DARTKV_DEQUANT_FUSED, "unknown dequant flavour %d", flavour);
  const DecodeLayout L = decode_layout(d, q_dtype, query_heads, flavour, tokens);
  const int64_t need = layout_bytes(d, query_heads, L);
  if (need > DARTKV_BUILTIN_SCRATCH_BYTES) {
    dartkv_set_error("this call needs %lld bytes of split scratch but the built-in scratch holds %lld; "
                     "use dartkv_decode_attention with a caller-provided workspace",
                     (long long)need, (long long)DARTKV_BUILTIN_SCRATCH_BYTES);
    return DARTKV_ELIMIT;
  }
  void* scratch = nullptr;
  int rc = builtin_scratch_address(&scratch);
  if (rc) return rc;
  // the array keeps whatever the previous call left; only the status word has to start at zero
  DARTKV_CUDA_OK(cudaMemsetAsync(scratch, 0, 16, (cudaStream_t)stream));
  return dartkv_decode_attention(d, query, q_dtype, query_heads, scale, flavour, tokens, scratch,
                                 DARTKV_BUILTIN_SCRATCH_BYTES, out, stream);
}
