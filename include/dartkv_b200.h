/*
 * dartkv_b200 -- C ABI of the B200 (sm_100a) DartKV KV-cache hot path.
 *
 * Every entry point is plain C: device pointers, sizes and a CUDA stream passed
 * as void*.  Nothing here allocates device memory unless stated; the caller
 * (PyTorch in the Python binding, anything else through FFI) owns every buffer.
 * All functions return 0 on success or a negative DARTKV_E* code;
 * dartkv_last_error() returns the message of the calling thread's last failure.
 *
 * Each declaration cites the reference interface it replaces, by path inside
 * the reference project.
 */
#ifndef DARTKV_B200_H
#define DARTKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of data and of scale / zero-point metadata */
enum { DARTKV_F32 = 0, DARTKV_F16 = 1, DARTKV_BF16 = 2 };
/* key page modes, numbered like src/dart/page_table.py:24-26 */
enum { DARTKV_DENSE_PAGE = 0, DARTKV_QUANTIZED_PAGE = 1, DARTKV_MIXED_PAGE = 2 };
/* scale = range / qmax evaluated as a true division (PyTorch CPU) or as range * (1/qmax) (PyTorch CUDA scalar path) */
enum { DARTKV_DIV_TRUE = 0, DARTKV_DIV_RECIPROCAL = 1 };
/* dequantization arithmetic: multiply and add each rounded to the metadata dtype
 * (src/dart/quantization.py:103-106, src/dart/mixed.py:91-94), or one fp32 multiply-add
 * rounded once to the output dtype (src/dart/triton_ops.py:59,110,201), or -- decode attention only -- one
 * fp32 multiply-add that is never rounded to the cache dtype, the arithmetic of the reference's Triton
 * attention kernels (src/dart/fused_attention.py:149-262) */
enum { DARTKV_DEQUANT_PER_OP = 0, DARTKV_DEQUANT_FP32 = 1, DARTKV_DEQUANT_FUSED = 2 };
/* channel scoring, src/dart/mixed.py:154-162 */
enum { DARTKV_SCORE_MAGNITUDE = 0, DARTKV_SCORE_VARIANCE = 1 };

enum {
  DARTKV_OK = 0,
  DARTKV_EINVAL = -1,   /* bad argument (message says which) */
  DARTKV_ECUDA = -2,    /* a CUDA runtime call failed */
  DARTKV_ELIMIT = -3    /* size beyond a documented limit of this build */
};

const char* dartkv_last_error(void);
int dartkv_version(void);
/* Number of kernels this library has launched in this process (for launch accounting in benchmarks). */
long long dartkv_launch_count(void);

/* ------------------------------------------------------------------ bit packing
 * Replaces _pack / _unpack (src/dart/quantization.py:25-45): element i of a byte
 * occupies bits [i*bits, (i+1)*bits); rows are padded with zero bits to a byte. */
int dartkv_pack(const uint8_t* codes, int64_t rows, int64_t n, int bits, uint8_t* packed, void* stream);
int dartkv_unpack(const uint8_t* packed, int64_t rows, int64_t packed_bytes, int bits, int64_t count,
                  uint8_t* codes, void* stream);

/* ------------------------------------------------------------------ group-wise quantizer
 * Replaces quantize / quantize_axis (src/dart/quantization.py:134-223).
 * The input is viewed as [outer, n, inner] with element strides; the quantized
 * axis is n.  Row r = o*inner + i.  Outputs: values [rows, packed_bytes] with
 * packed_bytes = ceil(ceil(n/group)*group / (8/bits)); scale, zero [rows, groups]
 * in md_dtype.  nonfinite (may be NULL) is set to 1 if any input is NaN/Inf
 * (the reference's isfinite().all() check, src/dart/quantization.py:159, read lazily). */
int dartkv_quantize(const void* x, int dtype, int64_t outer, int64_t n, int64_t inner,
                    int64_t stride_outer, int64_t stride_n, int64_t stride_inner,
                    int bits, int group_size, int md_dtype, int div_mode,
                    uint8_t* values, void* scale, void* zero, int32_t* nonfinite, void* stream);

/* Replaces QuantizedTensor.dequantize (src/dart/quantization.py:96-109) and the two uniform
 * Triton dequant kernels (src/dart/triton_ops.py:32-110).  Output is written as
 * [outer, n, inner] with the given element strides. */
int dartkv_dequantize(const uint8_t* values, const void* scale, const void* zero, int md_dtype,
                      int64_t outer, int64_t n, int64_t inner, int bits, int group_size, int flavour,
                      void* out, int out_dtype, int64_t stride_outer, int64_t stride_n, int64_t stride_inner,
                      void* stream);

/* ------------------------------------------------------------------ promoted key channels
 * Replaces the scoring half of select_key_channels (src/dart/mixed.py:154-162):
 * keys [bh, tokens, head_dim] (element strides, head_dim contiguous) -> scores [bh, head_dim] in dtype. */
int dartkv_channel_scores(const void* keys, int dtype, int64_t bh, int64_t tokens, int64_t head_dim,
                          int64_t stride_bh, int64_t stride_token, int strategy, void* scores, void* stream);
/* Replaces torch.topk in select_key_channels (src/dart/mixed.py:156): the `count` largest
 * scores per row, ordered by (score descending, channel ascending); indices int32 [bh, count]. */
int dartkv_select_channels(const void* scores, int dtype, int64_t bh, int64_t head_dim, int count,
                           int32_t* indices, void* stream);
/* Replaces quantize_key_mixed (src/dart/mixed.py:166-244) for given promoted channels.
 * low [bh, D, G, ceil(Gk/4)], high [bh, K, G, ceil(Gk/4)], scale/zero [bh, D, G]. */
int dartkv_quantize_key_mixed(const void* keys, int dtype, int64_t bh, int64_t tokens, int64_t head_dim,
                              int64_t stride_bh, int64_t stride_token, int group_size,
                              const int32_t* indices, int promoted, int md_dtype,
                              uint8_t* low, uint8_t* high, void* scale, void* zero, int32_t* nonfinite,
                              void* stream);
/* Replaces MixedQuantizedKey.dequantize (src/dart/mixed.py:72-94) and the mixed Triton
 * dequant kernel (src/dart/triton_ops.py:113-201); out [bh, tokens, head_dim] contiguous. */
int dartkv_dequantize_key_mixed(const uint8_t* low, const uint8_t* high, const int32_t* indices,
                                const void* scale, const void* zero, int md_dtype, int64_t bh, int64_t tokens,
                                int64_t head_dim, int group_size, int promoted, int flavour,
                                void* out, int out_dtype, void* stream);

/* ------------------------------------------------------------------ device-resident paged cache
 * Replaces the storage of DartKVCache (src/dart/cache.py:115-190): instead of Python
 * lists of tensors, one set of caller-allocated pools per layer plus device-side
 * page metadata that the attention kernel walks by itself.
 *
 * Token t of the sequence lives in exactly one place per side (K or V):
 *   t < sink_tokens                         -> k_sink / v_sink row t
 *   key page p with start[p] <= t < start[p]+tokens[p]  -> k_pages slot p
 *   sink_tokens <= t < v_packed_end         -> value row t - sink_tokens
 *   otherwise (not packed yet)              -> ring row t % ring_tokens
 */
typedef struct dartkv_cache_desc {
  int32_t batch, kv_heads, head_dim;
  int32_t dtype, md_dtype;
  int32_t page_size, key_group, value_group;
  int32_t key_bits, value_bits;
  int32_t key_mode;        /* DARTKV_QUANTIZED_PAGE or DARTKV_MIXED_PAGE */
  int32_t promoted;        /* promoted channels per head (mixed mode) */
  int32_t sink_tokens;     /* configured sink length S */
  int32_t ring_tokens;     /* rows of the dense ring R */
  int32_t max_key_pages;   /* page slots per (b,h) */
  int32_t max_value_tokens;/* packed value rows per (b,h) */
  /* byte geometry (filled by dartkv_cache_geometry) */
  int32_t key_page_bytes;  /* stride between page slots */
  int32_t key_off_high, key_off_index, key_off_scale, key_off_zero;   /* field offsets in a slot; low / values at 0 */
  int32_t value_row_bytes; /* packed codes per token */
  int32_t value_groups;    /* groups per token */
  int32_t regular_pages;   /* 1: every key page holds page_size tokens (pages are held until full) */
  /* pools (device pointers) */
  void* k_sink;            /* [B,H,S,D] dtype */
  void* v_sink;
  void* k_ring;            /* [B,H,R,D] dtype */
  void* v_ring;
  uint8_t* k_pages;        /* [B,H,max_key_pages,key_page_bytes] */
  uint8_t* v_codes;        /* [B,H,max_value_tokens,value_row_bytes] */
  void* v_meta;            /* [B,H,max_value_tokens,2,value_groups] md_dtype: scale row then zero row */
  int32_t* page_start;     /* [max_key_pages] first token of each key page */
  int32_t* page_tokens;    /* [max_key_pages] tokens in each key page */
  int32_t* state;          /* [32]: seen, key_pages, k_packed_end, v_packed_end, sink_filled, 0, 0, 0, then the
                            * plan of a device-planned append (16 words) */
} dartkv_cache_desc;

/* Fill the byte-geometry fields from the configuration fields. */
int dartkv_cache_geometry(dartkv_cache_desc* desc);

/* One append step, planned on the host (the lifecycle rules of src/dart/cache.py:168-190,403-470
 * are integer bookkeeping) and executed by the device: tokens [chunk_start, chunk_start+chunk_tokens)
 * arrive in keys/values [B,H,chunk_tokens,D] (element strides for b, h, token; D contiguous). */
typedef struct dartkv_append_plan {
  int32_t chunk_start, chunk_tokens;
  int32_t sink_copy;           /* leading chunk tokens copied into the sink rows */
  int32_t first_page;          /* slot of the first key page produced by this step */
  int32_t num_pages;           /* key pages produced */
  int32_t page_token_start;    /* absolute token of the first new key page */
  int32_t last_page_tokens;    /* tokens in the last new page (others hold page_size) */
  int32_t value_begin, value_end; /* absolute tokens whose values are packed by this step */
  int32_t ring_begin;          /* chunk tokens >= ring_begin keep dense keys in the ring (values: >= value_end) */
  int32_t reserved;
  int32_t seen_after, k_packed_end_after, v_packed_end_after, key_pages_after;
  int32_t requantize_last_page;   /* 1: re-quantize page first_page-1 in place first (src/dart/cache.py:427-439) */
} dartkv_append_plan;

/* indices: optional [B*H, num_pages, promoted] int32 promoted channels to use instead of
 * selecting them (parity with a particular reference run); NULL selects by score. */
int dartkv_cache_append(const dartkv_cache_desc* desc, const dartkv_append_plan* plan,
                        const void* keys, const void* values,
                        int64_t stride_b, int64_t stride_h, int64_t stride_t,
                        const int32_t* indices, int32_t* nonfinite, void* stream);

/* The lifecycle rules themselves as host arithmetic, so that an append needs no bookkeeping in the caller's
 * language: dartkv_lifecycle_plan turns (configuration, state, chunk length) into the plan of the step and
 * advances the state (src/dart/cache.py:168-190,403-470; the state is what the reference keeps in its segment
 * lists: tokens seen, end of the packed keys, end of the packed values, key pages so far).
 * dartkv_cache_append_step plans and appends in one call; the state advances only if the step was accepted, and
 * DARTKV_ELIMIT is returned (nothing launched, state unchanged) when the pools of desc are too small for the step. */
typedef struct dartkv_lifecycle_config {
  int32_t page_size, sink_tokens, local_tokens, value_local_tokens, hold_partial_pages;
} dartkv_lifecycle_config;
typedef struct dartkv_lifecycle_state {
  int32_t seen, k_packed_end, v_packed_end, key_pages;
} dartkv_lifecycle_state;
int dartkv_lifecycle_plan(const dartkv_lifecycle_config* cfg, dartkv_lifecycle_state* state, int chunk_tokens,
                          dartkv_append_plan* plan);
int dartkv_cache_append_step(const dartkv_cache_desc* desc, const dartkv_lifecycle_config* cfg,
                             dartkv_lifecycle_state* state, const void* keys, const void* values, int chunk_tokens,
                             int64_t stride_b, int64_t stride_h, int64_t stride_t, const int32_t* indices,
                             int32_t* nonfinite, dartkv_append_plan* plan_out, void* stream);
/* The same step planned on the device (no counterpart in the reference, whose page bookkeeping is Python,
 * src/dart/cache.py:403-470): a one-thread kernel runs the planner on the lifecycle state the cache keeps in
 * desc->state[0..3] and leaves the plan in desc->state[8..23], where the page, value-row and copy kernels that
 * follow on the stream read it.  Every launch has the same shape whatever the state, so append + decode attention
 * can be captured in a CUDA graph once and replayed token after token (give dartkv_decode_attention the token
 * capacity as `tokens`: the kernels read the exact count from desc->state).  For the lifecycles that only pack
 * full pages (hold_partial_pages, local_tokens, value_local_tokens) on the geometry of the page kernels (head_dim
 * 128, 16-bit data, 128-token pages and key groups, 16-byte aligned inputs), promoted channels selected by magnitude.
 * The caller keeps the pools large enough and sends a step that re-quantizes the boundary page (it can only be the
 * first append after a prompt) through dartkv_cache_append_step: dartkv_lifecycle_plan on a host copy of the state
 * tells both. */
int dartkv_cache_append_device_planned(const dartkv_cache_desc* desc, const dartkv_lifecycle_config* cfg,
                                       const void* keys, const void* values, int chunk_tokens, int64_t stride_b,
                                       int64_t stride_h, int64_t stride_t, int32_t* nonfinite, void* stream);

/* Materialize tokens [t0, t1) of the cache as dense [B,H,t1-t0,D] tensors (cache.get(),
 * src/dart/cache.py:192-199); side 0 = keys, 1 = values. */
int dartkv_cache_materialize(const dartkv_cache_desc* desc, int side, int32_t t0, int32_t t1, int flavour,
                             void* out, int out_dtype, void* stream);

/* ------------------------------------------------------------------ fused decode attention
 * Replaces fused_dart_attention (src/dart/fused_attention.py:654-771) and, numerically,
 * streamed_dart_attention (src/dart/attention.py:32-87): one query token per (batch, query head),
 * GQA by contiguous head groups, split-K over the token range with a cross-split merge.
 * query/out [B,Hq,D] (q_dtype, contiguous).
 * workspace: split-K scratch of at least dartkv_decode_workspace_bytes(desc, Hq, max_tokens) bytes
 * for any call with tokens <= max_tokens; zero it once after allocating (its first word is a status
 * word that a kernel sets if a bounded wait on an async copy ran out).
 * tokens: tokens currently in the cache (sizes the split grid; the kernels read the exact count and
 * the page metadata from desc->state on the device). */
int64_t dartkv_decode_workspace_bytes(const dartkv_cache_desc* desc, int query_heads, int max_tokens);
int dartkv_decode_attention(const dartkv_cache_desc* desc, const void* query, int q_dtype, int query_heads,
                            float scale, int flavour, int tokens, void* workspace, int64_t workspace_bytes,
                            void* out, void* stream);
/* How dartkv_decode_attention would split a call; host arithmetic only, nothing is launched (no counterpart in
 * the reference: it exists so that integrators and tests can see the plan).  kernel: 0 generic, 1 tensor-core
 * per-op flavour (2-bit pages), 2 tensor-core unrounded flavour (2-bit pages), 3 tensor-core kernel for every
 * other packed geometry and the fp32 flavour.  On the tensor-core layouts one unit is four consecutive pages
 * of a (batch, kv head) row; block j of `stream_blocks` owns units [j*units/stream_blocks, (j+1)*units/stream_blocks)
 * and every row is touched by at most total_splits - 1 of them (plus its dense-token block). */
typedef struct {
  int32_t kernel;
  int32_t quads;          /* units per row */
  int32_t stream_blocks;
  int32_t total_splits;   /* partial slots per (batch, query head) row of the workspace */
  int64_t units;          /* rows * quads */
  int32_t generic_splits; /* generic kernel only */
  int32_t generic_chunk;
} dartkv_decode_plan_info;
int dartkv_decode_plan(const dartkv_cache_desc* desc, int q_dtype, int query_heads, int flavour, int tokens,
                       dartkv_decode_plan_info* out);
/* Testing / debugging knob (no counterpart in the reference): force the family of work splits of the tensor-core
 * layouts for this process: "aligned", "unaligned", "unaligned:<blocks>", or NULL / "" for the cost model.  The
 * environment variable DARTKV_DECODE_SPLIT gives the initial value (read once).  Not thread-safe. */
int dartkv_decode_split_override(const char* spec);
/* Copies the workspace status word to the host (synchronizes the stream): 0 = no bounded wait expired. */
int dartkv_decode_status(const void* workspace, int* status_out, void* stream);

/* Decode attention over a left-padded batch.  The reference's fused call takes no mask (its Qwen3 adapter serves
 * uniform-length batches only, src/dart/integrations/qwen3.py:78-87); here `row_start` ([batch] int32 on the
 * device, or NULL for none) gives the first live token of every batch row and the tokens before it get no weight,
 * exactly as if the eager path had masked them with -inf.  Pages that lie wholly before a row's first live token
 * are not read.  Every row needs at least one live token (row_start[b] < tokens). */
int dartkv_decode_attention_padded(const dartkv_cache_desc* desc, const void* query, int q_dtype, int query_heads,
                                   float scale, int flavour, int tokens, const int32_t* row_start, void* workspace,
                                   int64_t workspace_bytes, void* out, void* stream);

/* Decode attention for callers that cannot hand over scratch memory.  No counterpart in the
 * reference: this exists for hosts embedding the library where device allocation is off limits at
 * the call site -- a serving loop whose memory pool is sized and frozen at start-up, a plugin
 * running inside another runtime's allocator-free callback, a real-time path that must not touch
 * the driver's allocator.  Same arguments and results as dartkv_decode_attention minus the
 * workspace: the split-K partials go to a 32 MiB array that is part of the library image (every
 * GPU that loads the library holds it until the process exits).
 *  - Calls whose partials need more than dartkv_builtin_scratch_bytes() fail with DARTKV_ELIMIT
 *    and a message giving both sizes (roughly batch * query_heads * splits * 520 bytes).
 *  - The first call on each device looks up the array's device address; make that first call
 *    outside any stream capture.  The call itself allocates nothing.
 *  - All calls share the one array and it keeps the previous call's contents (the status word is
 *    re-zeroed on the stream each call): two calls that overlap on the GPU, e.g. on different
 *    streams, race.  Serialize them or use the workspace variant. */
int64_t dartkv_builtin_scratch_bytes(void);
int dartkv_decode_attention_builtin_scratch(const dartkv_cache_desc* desc, const void* query, int q_dtype,
                                            int query_heads, float scale, int flavour, int tokens, void* out,
                                            void* stream);

/* Decode attention whose final step also delivers the output rows to every GPU of the node (no counterpart in the
 * reference, which is single-device; it replaces an all-gather of the outputs after dartkv_decode_attention).
 * The kernel that normalizes the rows stores them, besides `out`, into each rank's gathered tensor
 * [batch, dst_heads_total, head_dim] through peer-mapped pointers (plain stores over NVLink, no multicast), at batch
 * row dst_row_begin and query head dst_head_begin; its last block then writes `epoch` into flags[p][rank] on every
 * peer p and waits until flags[rank][p] of every peer shows `epoch` (or a later one).  When the call's kernels have
 * finished on this rank's stream, this rank's gathered tensor holds every rank's rows of the step.
 *  - out[p] / flags[p]: the gathered tensor and the uint32 flag array [world_size] of rank p, as mapped into this
 *    process (out[rank] / flags[rank] are this rank's own); flags start at zero and epochs grow by one per step.
 *  - A rank may run at most one step ahead of its slowest peer, so callers alternate between two gathered tensors.
 *  - The wait is bounded (about half a second): if a peer never arrives the workspace status word becomes 2 and the
 *    kernel returns; nothing spins on a kernel of the same GPU.  All ranks must make the call for the step to end. */
#define DARTKV_MAX_PEERS 8
typedef struct dartkv_peer_scatter {
  int32_t world_size, rank;
  int32_t dst_row_begin, dst_head_begin, dst_heads_total;
  uint32_t epoch;
  void* out[DARTKV_MAX_PEERS];
  uint32_t* flags[DARTKV_MAX_PEERS];
} dartkv_peer_scatter;
int dartkv_decode_attention_scatter(const dartkv_cache_desc* desc, const void* query, int q_dtype, int query_heads,
                                    float scale, int flavour, int tokens, void* workspace, int64_t workspace_bytes,
                                    void* out, const dartkv_peer_scatter* peers, void* stream);

/* ------------------------------------------------------------------ sharding over the GPUs of one node
 * No counterpart in the reference (it is single-device): every (batch row, KV head) is independent on this path,
 * so a rank owns rows [row_begin,row_end) x KV heads [head_begin,head_end) with its own pools and no exchange on
 * the hot path; only the attention outputs are gathered.  The batch is split first (ragged splits allowed: the
 * first batch groups hold one row more); KV heads are split as well only when world_size > batch.  rows_padded
 * is the largest row count of any rank (the per-rank extent of an equal-sized all-gather). */
typedef struct dartkv_shard {
  int32_t row_begin, row_end;
  int32_t head_begin, head_end;
  int32_t batch_groups, head_groups;
  int32_t rows_padded, reserved;
} dartkv_shard;
int dartkv_shard_range(int batch, int kv_heads, int world_size, int rank, dartkv_shard* out);

#ifdef __cplusplus
}
#endif
#endif /* DARTKV_B200_H */
