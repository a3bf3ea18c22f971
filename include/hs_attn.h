/*
 * hs_attn.h — C ABI of the B200-native (sm_100a) attention + quantised KV-cache kernels.
 *
 * This is the boundary a `hyprstream-attn-sys` crate (a sibling of the reference's
 * crates/bitsandbytes-sys) binds.  It follows that crate's conventions
 * (crates/bitsandbytes-sys/src/bindings.rs:10-334): one extern "C" block, plain C scalars and raw
 * pointers, `void*` for bf16 buffers, an opaque stream handle where NULL means the default stream,
 * and caller-owned memory — no function here allocates, frees or retains device memory
 * (the reference allocates every buffer with libtorch and passes data_ptr(),
 * crates/hyprstream/src/runtime/kv_cache.rs:804-839).
 *
 * Deliberate tightenings over bitsandbytes' `void` entry points: every function returns an int32
 * status (0 = ok, < 0 = argument error found on the host before any launch, > 0 = a cudaError_t),
 * `hs_attn_last_error()` returns a thread-local message, sizes are 64-bit, and every launch takes a
 * stream.  All launches are asynchronous.  There is no CPU fallback: on a device that is not
 * compute capability 10.x every compute entry point returns HS_ERR_DEVICE.
 *
 * Logical K/V geometry is the reference's: [tokens, kv_heads, head_dim], token-major, head_dim
 * contiguous, K stored after RoPE (kv_cache.rs:1160-1164,1281-1285; architectures/llama.rs:598-607).
 * Quantised storage keeps the reference's block geometry (a block is `block` consecutive elements
 * of that flattened tensor, one absmax per block, bitsandbytes-sys/src/lib.rs:104-105) but lives
 * in device memory instead of host Vec<u8> (kv_cache.rs:721-732).
 */
#ifndef HS_ATTN_H
#define HS_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *hs_stream_t; /* a cudaStream_t; NULL = default stream (cf. bnb_stream_t, bindings.rs:10-13) */

/* status codes */
#define HS_OK 0
#define HS_ERR_ARG (-1)       /* null / misaligned pointer, negative size, inconsistent geometry */
#define HS_ERR_UNSUPPORTED (-2) /* head_dim / group / block combination with no kernel */
#define HS_ERR_DEVICE (-3)    /* current device is not sm_100 */
#define HS_ERR_WORKSPACE (-4) /* workspace too small */
#define HS_ERR_POOL_EXHAUSTED (-5) /* block pool has no free page (typed, fail-soft: kv_cache.rs:482-505) */
#define HS_ERR_CACHE_OVERFLOW (-6) /* update past max_seq_len (kv_cache.rs:1288-1294) */
#define HS_ERR_CACHE_EMPTY (-7)    /* get() on an empty cache (kv_cache.rs:1500-1503) */

/* storage kinds: mirrors KVQuantType {None, Int8, Nf4, Fp4}
 * (crates/hyprstream-rpc-std/schema/model.capnp:252-257; kv_cache.rs:741-788) */
#define HS_KV_BF16 0
#define HS_KV_INT8 1 /* u8 index into code[i] = (i-127)/127, bitsandbytes-sys/src/lib.rs:108-111 */
#define HS_KV_NF4 2  /* lib.rs:131-148; two elements per byte, even element in the high nibble */
#define HS_KV_FP4 3  /* lib.rs:152-169 (the reference's unsigned table) */

#define HS_SCALE_F32 0 /* reference layout: f32 absmax (lib.rs:89) */
#define HS_SCALE_F16 1 /* absmax rounded to f16 before it normalises the block */

#define HS_DTYPE_BF16 0
#define HS_DTYPE_F16 1
#define HS_DTYPE_F32 2

/*
 * A view of one layer's K/V cache for `n_seqs` sequences.  Every sequence owns `pages_per_seq`
 * consecutive entries of the four page-pointer tables (device arrays of device pointers).
 * A page holds `page_tokens` tokens: K/V data [page_tokens, n_kv_heads, head_dim] (bf16, or u8
 * codes, or packed 4-bit codes of head_dim/2 bytes per row) and scales
 * [page_tokens, n_kv_heads, head_dim/block].  A contiguous per-sequence cache
 * (KVStorage::FullPrecision / Quantized, kv_cache.rs:967-996) is pages_per_seq = 1 with
 * page_tokens = its capacity; the paged pool (BlockPool, kv_cache.rs:477,515-680) is
 * page_tokens = 256.  Token t of sequence s lives in page s*pages_per_seq + t/page_tokens.
 */
typedef struct hs_kv_view {
    int32_t kind;        /* HS_KV_* */
    int32_t scale_dtype; /* HS_SCALE_*; ignored for HS_KV_BF16 */
    int32_t block;       /* elements per quantisation block: 64 (reference), 128 or 256; must divide head_dim */
    int32_t n_kv_heads;
    int32_t head_dim;    /* 64, 128 or 256 */
    int32_t page_tokens;
    int32_t pages_per_seq;
    int32_t reserved;
    void *const *k_pages;
    void *const *v_pages;
    void *const *k_scale_pages; /* NULL for HS_KV_BF16 */
    void *const *v_scale_pages;
} hs_kv_view;

/* ---- library ---------------------------------------------------------------------------- */
int32_t hs_attn_version(void);
/* 0 if `device` (or the current device when < 0) is compute capability 10.x, else HS_ERR_DEVICE. */
int32_t hs_attn_device_check(int32_t device);
const char *hs_attn_last_error(void);
/* Kernels never fault on a bad index: an out-of-range token position, page or RoPE row is skipped
 * and recorded in a per-device word.  This call synchronises with the device, returns the recorded
 * flags (0 = none) and clears them. */
#define HS_DEVERR_KV_WRITE_RANGE 1 /* hs_kv_quantize_write: position outside the view's pages or the RoPE table */
#define HS_DEVERR_ROPE_RANGE 2     /* hs_rope_apply: position outside the table; row copied unrotated */
#define HS_DEVERR_DECODE_RANGE 4   /* hs_attn_decode: seq_len beyond the view's pages; tokens past them ignored */
#define HS_DEVERR_WAIT_TIMEOUT 8   /* a bounded device-side wait ran out */
int32_t hs_attn_take_device_error(int32_t *flags);
/* The flags are a report, not a precondition: entry points launch and produce valid results while flags are pending
 * (a kernel only cuts a launch short for a wait that ran out inside that same launch).  Test hook: ORs `flags` into the
 * current device's word from the host, so that this can be checked without making a wait run out. */
int32_t hs_attn_inject_device_error(int32_t flags);

/* Tracing hook: while profiling is on, each compute entry point brackets its dominant kernel with two
 * CUDA events on the launch stream; hs_attn_last_kernel_ms() waits for the latest pair and returns the
 * elapsed device time.  Off by default; one set of events per process, so profile one stream at a time. */
int32_t hs_attn_set_profiling(int32_t on);
int32_t hs_attn_last_kernel_ms(float *ms);
/* Kernels this library has launched in this process so far (all entry points, all streams). */
int64_t hs_attn_launch_count(void);

/* ---- blockwise quantiser (flat tensors) --------------------------------------------------
 * Replaces cquantize_blockwise_{bf16,fp16,fp32}[_nf4,_fp4] and cdequantize_blockwise_*
 * (bitsandbytes-sys/src/bindings.rs:20-197; called from kv_cache.rs:771-779,823-840,882-899,929-946).
 * `src`/`out` hold n elements of `dtype`; `codes` holds n bytes (INT8) or (n+1)/2 bytes (4-bit);
 * `absmax` holds ceil(n/block) f32 or f16 values.  All pointers are device pointers. */
int32_t hs_quantize_blockwise(int32_t kind, const void *src, int32_t dtype, int64_t n, int32_t block,
                              int32_t scale_dtype, uint8_t *codes, void *absmax, hs_stream_t stream);
int32_t hs_dequantize_blockwise(int32_t kind, const uint8_t *codes, const void *absmax, int64_t n, int32_t block,
                                int32_t scale_dtype, void *out, int32_t dtype, hs_stream_t stream);

/* ---- RoPE ---------------------------------------------------------------------------------
 * RoPE::apply_rotary_pos_emb (runtime/rope.rs:206-248) on x [n_rows, n_heads, head_dim] bf16, out
 * of place (out != x): half-split rotation of the first `rotary_dim` dims, every multiply, subtract
 * and add rounded to bf16 as libtorch does; `sin`/`cos` are the caller's bf16 tables
 * [n_positions, rotary_dim/2] (rope.rs:100-122) and `positions` int32 [n_rows]. */
int32_t hs_rope_apply(const void *x, void *out, const void *sin, const void *cos, const int32_t *positions,
                      int64_t n_rows, int32_t n_heads, int32_t head_dim, int32_t rotary_dim, int32_t n_positions,
                      hs_stream_t stream);

/* Per-head RMS norm + (partial) RoPE + gate split in one pass: the steps between the q/k/v projections and the
 * cache / attention call of Qwen3_5FullAttention::forward (architectures/qwen3_5.rs:963-990; apply_qknorm :1077-1091)
 * and LlamaAttention's optional QK-norm (architectures/llama.rs:929-992).
 *   x         bf16, row (t, h) at x + t*token_stride + h*head_stride (elements): e.g. the doubled q projection
 *             [n_tokens, n_heads, 2*head_dim] with head_stride = 2*head_dim, or a dense k
 *   out       bf16 [n_tokens, n_heads, head_dim] = rope(bf16(x * rsqrt(mean(x^2) + eps) * (w or 1 + w)))
 *   gate_out  optional bf16 [n_tokens, n_heads, head_dim] = x[.., head_dim : 2*head_dim] (qwen3_5.rs:965-967)
 *   norm_weight f32 [head_dim] or NULL (no norm); weight_plus_one != 0 for Qwen3.5's (1 + w)
 *   sin, cos  bf16 [n_positions, rotary_dim/2] or NULL (no rotation); positions int32 [n_tokens]; a position outside
 *             the table leaves the row unrotated and records HS_DEVERR_ROPE_RANGE */
int32_t hs_qk_norm_rope(const void *x, int64_t token_stride, int64_t head_stride, void *out, void *gate_out,
                        const float *norm_weight, float eps, int32_t weight_plus_one, const void *sin, const void *cos,
                        const int32_t *positions, int32_t n_positions, int32_t rotary_dim, int64_t n_tokens,
                        int32_t n_heads, int32_t head_dim, hs_stream_t stream);

/* ---- KV quantise-on-write -----------------------------------------------------------------
 * LayerKVCache::update (kv_cache.rs:1275-1496) for device-resident storage: appends
 * k_new/v_new [n_seqs, n_tokens, n_kv_heads, head_dim] bf16 to the caches in `view`, sequence s at
 * token positions dst_pos[s] .. dst_pos[s]+n_tokens-1 (dst_pos: device int32 [n_seqs]).
 * HS_KV_BF16 copies; the quantised kinds write codes + scales bit-identical to
 * hs_quantize_blockwise on the same rows.  If `sin` is non-NULL, K is rotated first exactly as
 * hs_rope_apply would with position dst_pos[s]+t (V is never rotated). */
int32_t hs_kv_quantize_write(const hs_kv_view *view, const void *k_new, const void *v_new, int32_t n_seqs,
                             int32_t n_tokens, const int32_t *dst_pos, const void *sin, const void *cos,
                             int32_t rotary_dim, int32_t n_positions, hs_stream_t stream);

/* The same with K's per-head RMS norm fused in front of the rotation: k_proj is the raw k projection
 * [n_seqs, n_tokens, n_kv_heads, head_dim]; K = rope(bf16(k * rsqrt(mean(k^2) + eps) * (w or 1 + w))) at position
 * dst_pos[s] + t is what gets quantised and stored (Qwen3_5FullAttention::forward, architectures/qwen3_5.rs:971-999:
 * apply_qknorm :1077-1091, partial RoPE, cache.update; LlamaAttention's optional QK-norm, llama.rs:929-992), in one pass
 * over the new keys instead of hs_qk_norm_rope followed by hs_kv_quantize_write - bit-identical to that route.
 * k_out (optional, bf16, same shape) receives the normed, rotated keys for a prompt's own attention. */
int32_t hs_kv_norm_rope_quantize_write(const hs_kv_view *view, const void *k_proj, const void *v_new, int32_t n_seqs,
                                       int32_t n_tokens, const int32_t *dst_pos, const float *k_norm_weight, float eps,
                                       int32_t weight_plus_one, const void *sin, const void *cos, int32_t rotary_dim,
                                       int32_t n_positions, void *k_out, hs_stream_t stream);

/* LayerKVCache::get (kv_cache.rs:1499-1643) compatibility path: dequantise (or copy) tokens
 * [0, seq_lens[s]) of every sequence into k_out/v_out [n_seqs, out_tokens, n_kv_heads, head_dim] bf16;
 * rows past seq_lens[s] are zero-filled like the reference's right padding (llama.rs:787-813). */
int32_t hs_kv_gather_dequantize(const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t out_tokens,
                                void *k_out, void *v_out, hs_stream_t stream);

/* ---- decode attention ---------------------------------------------------------------------
 * One query token per sequence against its cache: the fused replacement of cache.get() + GQA
 * expansion + compute_attention_masked for q_len == 1 (llama.rs:605-640,710-844,847-872,1023-1119)
 * and of Qwen3_5FullAttention's decode branch (qwen3_5.rs:992-1059).
 *   q        bf16 [n_seqs, n_q_heads, head_dim]      seq_lens  device int32 [n_seqs] (ragged; no padding)
 *   out      bf16 [n_seqs, n_q_heads, head_dim]      gate      optional bf16, same shape: out *= sigmoid(gate)
 *   softmax_scale  normally 1/sqrt(head_dim)
 * Query head h reads kv head h / (n_q_heads / n_kv_heads).  The KV range is split across CTAs and the
 * partials are merged by log-sum-exp inside the call; `workspace` (>= hs_attn_decode_workspace_bytes)
 * is scratch for those partials.  If `o_shard`/`lse_shard` are non-NULL the call instead writes the
 * merged, normalised fp32 result [n_seqs, n_q_heads, head_dim] and its log-sum-exp
 * [n_seqs, n_q_heads] (natural log, scaled scores) for a KV-length shard, to be combined across
 * GPUs with hs_attn_merge_partials; `out` may then be NULL. */
int64_t hs_attn_decode_workspace_bytes(int32_t n_seqs, int32_t n_q_heads, int32_t head_dim);
int32_t hs_attn_decode(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs,
                       int32_t n_q_heads, float softmax_scale, void *out, const void *gate, void *workspace,
                       int64_t workspace_bytes, float *o_shard, float *lse_shard, hs_stream_t stream);

/* Concurrency: two hs_attn_decode (/ _static / _step / _sharded) launches must not be in flight on one device at the
 * same time.  Launches on one stream are ordered by the stream; launches on different streams of one device, or from
 * different host threads, must be serialised by the caller (an event between them is enough).  The tensor-core kernel
 * is a cooperative launch whose CTAs meet at a grid-wide barrier that counts arrivals in a per-device counter; the
 * arrivals of two overlapping launches would mix.  If the rule is broken the barrier's bounded wait runs out:
 * HS_DEVERR_WAIT_TIMEOUT is recorded and that step's result is undefined; nothing hangs. */

/* hs_attn_decode for callers that cannot hand over a workspace.  (No counterpart in the reference: there the
 * caller allocates every buffer with libtorch.)  Some hosts of this library cannot allocate device memory at
 * the point where they decode: an embedder whose whole device budget is owned by another allocator, a worker
 * that must not synchronise the device (cudaMalloc / cudaFree do), or a step function that runs where allocation
 * is forbidden.  For them the split-KV partials go into an array that is part of the library image itself: 24 MiB
 * (hs_attn_decode_static_max_bytes()), resident on every GPU that loads the library for as long as the process
 * lives.  Inputs and outputs are still the caller's; the arguments mean what they mean for hs_attn_decode, minus
 * workspace and shard outputs.
 *   - Shapes whose hs_attn_decode_workspace_bytes() exceeds the array are refused with HS_ERR_WORKSPACE and a
 *     message that states both sizes (at 32 query heads and head_dim 128 that is n_seqs above 170).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress), and the first call
 *     per device and cache layout (kind, block, scale type, head shape) configures that layout's kernel
 *     (cudaFuncSetAttribute, an occupancy query).  Make those first calls before any stream capture begins.
 *     No call allocates or frees device memory (tested: the device's free-memory figure does not move).
 *   - All calls share the one array, and it keeps whatever the previous call left; nothing in it needs to be
 *     zero, because a launch only reads partial slots it has just written.  Two calls whose kernels overlap on
 *     the GPU (different streams, or different host threads on one device) race on it: serialise them. */
int64_t hs_attn_decode_static_max_bytes(void);
int32_t hs_attn_decode_static(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs,
                              int32_t n_q_heads, float softmax_scale, void *out, const void *gate, hs_stream_t stream);

/* LayerKVCache::update of one new token per sequence followed by the attention over the cache, as LlamaAttention::forward
 * does them back to back (architectures/llama.rs:598-640; forward_batched :772-828): hs_kv_quantize_write (n_tokens = 1,
 * optional fused K RoPE) + hs_attn_decode in one call.  k_new, v_new bf16 [n_seqs, 1, n_kv_heads, head_dim]; seq_lens the
 * lengths attended, the new token included; dst_pos the new tokens' cache positions, or NULL for "position
 * seq_lens[s] - 1", the normal case; the rest as for the two calls.
 *   dst_pos == NULL, u8 cache, a shape the tensor-core decode kernel serves: ONE launch - the CTA that owns a sequence's
 *     last tile quantises that sequence's new K and V rows into the cache (same codes and scales as the write kernel,
 *     bit for bit) before it streams the tile.
 *   otherwise: the write kernel, then the attention kernel launched as its programmatic dependent (its launch and set-up
 *     run under the write; only its first cache read waits for it).  q may come from any earlier work on the stream. */
int32_t hs_attn_decode_append(const void *q, const void *k_new, const void *v_new, const hs_kv_view *view,
                              const int32_t *dst_pos, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads,
                              float softmax_scale, const void *sin, const void *cos, int32_t rotary_dim, int32_t n_positions,
                              void *out, const void *gate, void *workspace, int64_t workspace_bytes, hs_stream_t stream);

/* One decode step of a batch as ONE call, for a host whose step inputs and result live in host memory: the
 * reference's engine loop runs one forward per step on one thread and reads the result back
 * (crates/hyprstream/src/runtime/torch_engine.rs:3719-3731, forward_batched_step :1475-1501); through this entry that
 * host pays one FFI call per layer and step instead of four (copy in, cache update, attention, copy out).
 *   host_in   pinned host memory, bf16: q [n_seqs, n_q_heads, D] | k_new [n_seqs, n_kv_heads, D] | v_new [same]
 *   dev_in    device staging buffer of the same size (16-byte aligned); dev_out device bf16 [n_seqs, n_q_heads, D]
 *   host_out  pinned host memory for the result, same shape as q
 *   dst_pos, seq_lens  device int32 [n_seqs]: where each sequence's new token goes (NULL: seq_lens - 1, which lets the
 *             attention kernel write it: see hs_attn_decode_append), and the length attended, the new token included;
 *             sin / cos / rotary_dim / n_positions as for hs_kv_quantize_write (K rotated)
 * Enqueues on `stream`: one host-to-device copy, hs_kv_quantize_write of the one new token per sequence,
 * hs_attn_decode, one device-to-host copy.  With HS_STEP_SYNC in `flags` the call returns when host_out is valid;
 * otherwise the caller synchronises the stream. */
#define HS_STEP_SYNC 1
int32_t hs_attn_decode_step(const hs_kv_view *view, const void *host_in, void *dev_in, const int32_t *dst_pos,
                            const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads, float softmax_scale, const void *sin,
                            const void *cos, int32_t rotary_dim, int32_t n_positions, void *dev_out, void *host_out,
                            void *workspace, int64_t workspace_bytes, int32_t flags, hs_stream_t stream);

/* ---- KV-length shards across GPUs, one launch per GPU and step -------------------------------------
 * New design (the reference has no collective: crates/hyprstream/src/runtime/architectures/llama.rs:776-781 keeps
 * every sequence's cache on one device).  One long context is cut into contiguous KV-length shards, one per GPU;
 * every GPU runs hs_attn_decode_sharded over its shard with the same q.  Inside that one launch the kernel merges its
 * own split-KV partials, stores the shard's (o, lse) into every rank's inbox with ordinary stores over NVLink - each
 * value travels in one 8-byte word together with the step's number, so a reader that sees the number sees the value -
 * waits, bounded, for the other ranks' parts and merges them: every rank ends with the same bf16 out.  (The three-call form - hs_attn_decode with o_shard / lse_shard, an all-gather,
 * hs_attn_merge_partials_strided - stays available and serves the shapes the tensor-core kernel does not cover.)
 *
 * hs_shard_group owns this rank's inbox (one cudaMalloc allocation sized for max_seqs x n_q_heads rows).
 *   several processes (one per GPU): create -> export (hs_shard_group_handle_bytes() bytes, a CUDA IPC handle) ->
 *     exchange the handles by any host channel -> connect with all `world` handles in rank order;
 *   one process: create every rank's group (each with its device current) -> hs_shard_group_connect_local.
 * Every rank must call hs_attn_decode_sharded the same number of times (the step number is counted per group); a rank
 * may run at most one step ahead of the slowest.  If a rank does not deliver within the wait limit (default 2000 ms,
 * hs_shard_group_set_wait_ms), the waiting ranks record HS_DEVERR_WAIT_TIMEOUT, leave the affected rows of `out`
 * unwritten and finish the launch; the context stays usable.  HS_SHARD_PUSH_ONLY makes a call deliver its part
 * without waiting or writing an output (out may be NULL): for a rank that does not need the result, and for running
 * several ranks one after the other on one GPU; such a rank is not held back by the others, so the caller paces it.
 * Supported shapes: those of the tensor-core decode kernel (quantised cache; 8 kv heads x 128 with 32 query heads, or
 * 2 x 256 with 16); others return HS_ERR_UNSUPPORTED.  No multicast load of any kind touches peer memory. */
typedef struct hs_shard_group hs_shard_group;
#define HS_SHARD_PUSH_ONLY 1
int32_t hs_shard_group_create(int32_t rank, int32_t world, int32_t max_seqs, int32_t n_q_heads, int32_t head_dim,
                              hs_shard_group **out);
int32_t hs_shard_group_handle_bytes(void);
int32_t hs_shard_group_export(hs_shard_group *group, void *handle_out);
int32_t hs_shard_group_connect(hs_shard_group *group, const void *handles);
int32_t hs_shard_group_connect_local(hs_shard_group *const *groups, int32_t world);
int32_t hs_shard_group_set_wait_ms(hs_shard_group *group, int32_t wait_ms);
int32_t hs_shard_group_epoch(const hs_shard_group *group); /* steps delivered so far */
void hs_shard_group_destroy(hs_shard_group *group);
int32_t hs_attn_decode_sharded(hs_shard_group *group, const void *q, const hs_kv_view *view, const int32_t *seq_lens,
                               int32_t n_seqs, int32_t n_q_heads, float softmax_scale, void *out, const void *gate,
                               void *workspace, int64_t workspace_bytes, int32_t flags, hs_stream_t stream);

/* Log-sum-exp merge of `n_parts` partial results: o_parts fp32 [n_parts, n_rows, head_dim],
 * lse_parts fp32 [n_parts, n_rows] (n_rows = n_seqs * n_q_heads) -> out bf16 [n_rows, head_dim],
 * optionally times sigmoid(gate).  A part with lse = -inf contributes nothing. */
int32_t hs_attn_merge_partials(const float *o_parts, const float *lse_parts, int32_t n_parts, int64_t n_rows,
                               int32_t head_dim, void *out, const void *gate, hs_stream_t stream);
/* The same with the parts `part_stride_o` / `part_stride_lse` floats apart (>= n_rows * head_dim / n_rows), so that
 * each GPU's (o, lse) message of an all-gather can be merged where it landed, without repacking. */
int32_t hs_attn_merge_partials_strided(const float *o_parts, const float *lse_parts, int32_t n_parts, int64_t part_stride_o,
                                       int64_t part_stride_lse, int64_t n_rows, int32_t head_dim, void *out, const void *gate,
                                       hs_stream_t stream);

/* ---- causal prefill attention ---------------------------------------------------------------
 * compute_attention_masked for q_len > 1 (architectures/llama.rs:1023-1119, single shot and the 1024-row
 * chunked loop), fused with GQA expansion (llama.rs:847-872), and Qwen3_5FullAttention's prefill branch
 * (qwen3_5.rs:1012-1059) when `gate` is given.
 *   q    bf16 [n_seqs, q_len, n_q_heads, head_dim]     k, v  bf16 [n_seqs, kv_len, n_kv_heads, head_dim]
 *   out  bf16 [n_seqs, q_len, n_q_heads, head_dim]     gate  optional bf16 like out: out *= sigmoid(gate)
 * Query row i sits at absolute position (kv_len - q_len) + i and sees keys 0 .. (kv_len - q_len) + i, the
 * reference's tril(k_len - q_len) offset for a cached prefix (llama.rs:1074-1084); kv_len >= q_len.
 * K/V are the post-RoPE tensors the reference hands to attention (cache.get() or the fresh k, v). */
int32_t hs_attn_prefill_causal(const void *q, const void *k, const void *v, void *out, const void *gate, int32_t n_seqs,
                               int32_t q_len, int32_t kv_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                               float softmax_scale, hs_stream_t stream);

/* ---- gated DeltaNet ------------------------------------------------------------------------
 * The recurrent delta rule of GatedDeltaNetLayer::forward (architectures/qwen3_5.rs:725-751) for n_tokens >= 1
 * tokens per sequence, state updated in place:
 *   S <- exp(g) S;  m = k^T S;  delta = beta (v - m);  S <- S + k delta^T;  o = q^T S
 *   q, k   f32 [n_seqs, n_tokens, n_k_heads, head_k_dim]  (already L2-normalised; q already scaled, :679-682)
 *   v      f32 [n_seqs, n_tokens, n_v_heads, head_v_dim]
 *   g,beta f32 [n_seqs, n_tokens, n_v_heads]              (log-decay <= 0 and write strength, :687-701)
 *   state  f32 [n_seqs, n_v_heads, head_k_dim, head_v_dim] in/out (rec_state, :697-699)
 *   out    f32 [n_seqs, n_tokens, n_v_heads, head_v_dim]
 * k/q head i feeds value heads [i*r, (i+1)*r), r = n_v_heads / n_k_heads (:704-720). */
int32_t hs_gdn_recurrent(const float *q, const float *k, const float *v, const float *g, const float *beta, float *state,
                         float *out, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads,
                         int32_t head_k_dim, int32_t head_v_dim, hs_stream_t stream);

/* The prefill branch of the same layer: chunked_delta_rule (architectures/qwen3_5.rs:342-498, called at :753-769) on
 * the tensor cores.  Same arguments, layouts and in-place state update as hs_gdn_recurrent, same mathematics (the chunked
 * form is an exact re-association of the rule; the chunk length is internal), but the operands of the S-dependent
 * products are rounded to bf16 (state, accumulation and the per-chunk triangular solve stay fp32): results agree with
 * hs_gdn_recurrent / the fp32 reference to ~1e-3, inside the path's tolerance (max-abs 2e-2, mean-abs 2e-3).  Head dims
 * 128 x 128.  Use hs_gdn_recurrent where fp32-exact results are wanted or for single decode tokens. */
int32_t hs_gdn_chunk_prefill(const float *q, const float *k, const float *v, const float *g, const float *beta, float *state,
                             float *out, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads,
                             int32_t head_k_dim, int32_t head_v_dim, hs_stream_t stream);

/* The elementwise steps either side of the rule in GatedDeltaNetLayer::forward, one pass over HBM each.
 *
 * hs_gdn_prologue (architectures/qwen3_5.rs:627-701, after the fused input projection): depthwise causal conv1d over
 * time with `kernel_size` taps (left context: conv_state, or zeros when has_state == 0) in bf16, SiLU, split into
 * q | k | v, q and k to fp32 and divided by max(||.||_2, 1e-3) per head, q times 1/sqrt(head_k_dim), v to fp32,
 * g = neg_a_exp * softplus(a_in + dt_bias), beta = sigmoid(b_in); conv_state is replaced by the last kernel_size-1 frames.
 *   mixed_qkv   bf16 [n_seqs, n_tokens, 2*n_k_heads*head_k_dim + n_v_heads*head_v_dim]     (qwen3_5.rs:622)
 *   conv_weight bf16 [conv_dim, kernel_size]  (the reference's [conv_dim, 1, kernel_size])  (qwen3_5.rs:655-662)
 *   conv_state  bf16 [n_seqs, conv_dim, kernel_size-1] in/out, always kernel_size-1 frames   (qwen3_5.rs:633-653)
 *   a_in, b_in  bf16 [n_seqs, n_tokens, n_v_heads];  neg_a_exp = -exp(A_log), dt_bias  f32 [n_v_heads]  (:687-689,701)
 *   q, k  f32 [n_seqs, n_tokens, n_k_heads, head_k_dim];  v f32 [n_seqs, n_tokens, n_v_heads, head_v_dim]
 *   g, beta  f32 [n_seqs, n_tokens, n_v_heads]                 -> the inputs of hs_gdn_recurrent
 *
 * hs_gdn_epilogue (RMSNormGated, qwen3_5.rs:305-313 as called at :771-784): per (token, value head) row of head_v_dim:
 *   y = bf16( o * rsqrt(mean(o^2) + eps) * norm_weight * silu(z) )
 *   o f32 [n_rows, head_v_dim] (the rule's output), z bf16 [n_rows, head_v_dim], norm_weight f32 [head_v_dim]. */
int32_t hs_gdn_prologue(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in,
                        const void *b_in, const float *neg_a_exp, const float *dt_bias, float *q, float *k, float *v, float *g,
                        float *beta, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads,
                        int32_t head_k_dim, int32_t head_v_dim, int32_t kernel_size, hs_stream_t stream);
int32_t hs_gdn_epilogue(const float *o, const void *z, const float *norm_weight, float eps, void *y, int64_t n_rows,
                        int32_t head_v_dim, hs_stream_t stream);

/* ---- Qwen3.5 hybrid layers, batched -----------------------------------------------------------
 * What GatedDeltaNetLayer::forward (architectures/qwen3_5.rs:606-802) and Qwen3_5FullAttention::forward
 * (qwen3_5.rs:902-1075) do between their input and output projections, for a batch of sequences, one call per layer;
 * and a run of DeltaNet layers followed by one full-attention layer as one call.  The reference has no batched entry
 * for this architecture (ModelOperations::forward_batched is Llama-only, the trait default errors:
 * architectures/mod.rs:268-280; its layer dispatch qwen3_5.rs:1864-1933 keeps one rec_state / conv_state slot per
 * layer): here the states are batch-major tensors of the caller, one row per sequence, updated in place, and row s of a
 * batch computes exactly what the unbatched call computes for sequence s.  The projections (GEMMs) stay with the host.
 *
 * DeltaNet layer: hs_gdn_prologue -> hs_gdn_recurrent (n_tokens == 1, the decode step) or hs_gdn_chunk_prefill
 * (n_tokens > 1, the prompt; qwen3_5.rs:725-769) -> hs_gdn_epilogue.
 *   mixed_qkv, a_in, b_in, conv_state  as for hs_gdn_prologue;  z bf16 [n_seqs, n_tokens, n_v_heads, head_v_dim]
 *   rec_state  f32 [n_seqs, n_v_heads, head_k_dim, head_v_dim] in/out; has_state == 0 starts conv_state and rec_state at zero
 *   y          bf16 [n_seqs, n_tokens, n_v_heads, head_v_dim] -> the input of out_proj
 * Full-attention layer: hs_qk_norm_rope on q (gate split, (1 + w) norm, partial RoPE) -> hs_kv_norm_rope_quantize_write
 * (k normed, rotated at its cache position dst_pos[s] + t, quantised and stored in one pass) ->
 * hs_attn_decode over the cache (n_tokens == 1) or hs_attn_prefill_causal over the fresh K/V (n_tokens > 1: a prompt
 * that starts at position 0; a continued prompt goes through hs_kv_gather_dequantize and hs_attn_prefill_causal with
 * kv_len > q_len), with the output gate.
 *   q_proj bf16 [n_seqs * n_tokens, n_q_heads * 2 * head_dim] (per head: query | gate, qwen3_5.rs:965-967)
 *   k_proj bf16 [n_seqs * n_tokens, n_kv_heads * head_dim];  v_proj bf16 [n_seqs, n_tokens, n_kv_heads, head_dim]
 *   positions device int32 [n_seqs * n_tokens] (RoPE rows); dst_pos device int32 [n_seqs] (cache position of each
 *   sequence's first new token); seq_lens device int32 [n_seqs] (length attended by a decode step, dst_pos + 1)
 *   out bf16 [n_seqs, n_tokens, n_q_heads, head_dim] -> the input of o_proj
 * Workspaces: 256-byte aligned device memory of at least the *_workspace_bytes() figure; nothing is allocated. */
typedef struct hs_gdn_layer_params {
    const void *conv_weight;   /* bf16 [conv_dim, kernel_size] */
    const float *neg_a_exp;    /* f32 [n_v_heads] = -exp(A_log) */
    const float *dt_bias;      /* f32 [n_v_heads] */
    const float *norm_weight;  /* f32 [head_v_dim] */
    float norm_eps;
    int32_t n_k_heads, n_v_heads, head_k_dim, head_v_dim, kernel_size;
} hs_gdn_layer_params;
typedef struct hs_gdn_layer_io {
    const void *mixed_qkv, *z, *a_in, *b_in;
    void *conv_state;
    float *rec_state;
    void *y;
} hs_gdn_layer_io;
typedef struct hs_qwen_attn_params {
    const float *q_norm_weight, *k_norm_weight; /* f32 [head_dim], applied as (1 + w) */
    float norm_eps;
    const void *sin, *cos;                      /* bf16 [n_positions, rotary_dim / 2] */
    int32_t n_positions, rotary_dim;
    int32_t n_q_heads, n_kv_heads, head_dim;
    float softmax_scale;
} hs_qwen_attn_params;
typedef struct hs_qwen_attn_io {
    const void *q_proj, *k_proj, *v_proj;
    const hs_kv_view *view;
    const int32_t *positions, *dst_pos, *seq_lens;
    void *out;
} hs_qwen_attn_io;
int64_t hs_gdn_layer_workspace_bytes(const hs_gdn_layer_params *params, int32_t n_seqs, int32_t n_tokens);
int32_t hs_gdn_layer_forward(const hs_gdn_layer_params *params, const void *mixed_qkv, const void *z, const void *a_in,
                             const void *b_in, void *conv_state, float *rec_state, int32_t has_state, int32_t n_seqs,
                             int32_t n_tokens, void *y, void *workspace, int64_t workspace_bytes, hs_stream_t stream);
int64_t hs_qwen_attn_layer_workspace_bytes(const hs_qwen_attn_params *params, int32_t n_seqs, int32_t n_tokens);
int32_t hs_qwen_attn_layer_forward(const hs_qwen_attn_params *params, const void *q_proj, const void *k_proj,
                                   const void *v_proj, const hs_kv_view *view, const int32_t *positions,
                                   const int32_t *dst_pos, const int32_t *seq_lens, int32_t n_seqs, int32_t n_tokens,
                                   void *out, void *workspace, int64_t workspace_bytes, hs_stream_t stream);
/* n_gdn DeltaNet layers (parameters gdn[i], tensors gdn_io[i]) and then, if attn is non-NULL, one full-attention layer,
 * all for the same batch and token count, sharing one workspace (hs_qwen_block_workspace_bytes: the largest need). */
int64_t hs_qwen_block_workspace_bytes(const hs_gdn_layer_params *gdn, int32_t n_gdn, const hs_qwen_attn_params *attn,
                                      int32_t n_seqs, int32_t n_tokens);
int32_t hs_qwen_block_forward(const hs_gdn_layer_params *gdn, const hs_gdn_layer_io *gdn_io, int32_t n_gdn,
                              const hs_qwen_attn_params *attn, const hs_qwen_attn_io *attn_io, int32_t has_state,
                              int32_t n_seqs, int32_t n_tokens, void *workspace, int64_t workspace_bytes,
                              hs_stream_t stream);

/* ---- host-side cache objects ------------------------------------------------------------------
 * C++ mirror of the reference's per-layer cache (crates/hyprstream/src/runtime/kv_cache.rs): LayerKVCache
 * (:1029-1900: new / new_paged / update / get / clear / truncate_to / seq_pos / memory_usage) and BlockPool
 * (:477-680: fixed 256-token pages, LIFO free list, owner tags, typed exhaustion with roll-back).  Storage is
 * device-resident and token-granular for every kind (quantised + paged allowed).  These objects own device
 * memory (cudaMalloc on the device current at creation, or the allocator installed with
 * hs_host_set_allocator, e.g. libtorch's caching allocator); the kernels above never allocate.
 * Handles are opaque; all calls on one cache must come from one thread at a time, like the reference's
 * (inference/local.rs:84-85).  */
typedef struct hs_pool hs_pool;
typedef struct hs_cache hs_cache;
typedef struct hs_view hs_view;
typedef void *(*hs_alloc_fn)(size_t bytes);  /* returns device memory or NULL */
typedef void (*hs_free_fn)(void *ptr);
int32_t hs_host_set_allocator(hs_alloc_fn alloc_fn, hs_free_fn free_fn); /* NULL, NULL restores cudaMalloc / cudaFree */

int32_t hs_pool_create(int32_t n_blocks, int32_t page_tokens, int32_t kind, int32_t block, int32_t scale_dtype,
                       int32_t n_kv_heads, int32_t head_dim, hs_pool **out);
/* Drops the handle.  Caches created from the pool keep its storage alive (the reference's caches hold an Arc<BlockPool>,
 * kv_cache.rs:1111-1130): it is freed when the handle and the last such cache are gone, in either order. */
void hs_pool_destroy(hs_pool *pool);
int32_t hs_pool_num_free(const hs_pool *pool);

int32_t hs_cache_create(int32_t max_seq_len, int32_t kind, int32_t block, int32_t scale_dtype, int32_t n_kv_heads,
                        int32_t head_dim, hs_cache **out);                                  /* LayerKVCache::new */
int32_t hs_cache_create_paged(int32_t max_seq_len, hs_pool *pool, int64_t owner, hs_cache **out); /* ::new_paged */
void hs_cache_destroy(hs_cache *cache); /* returns pages to the pool (Drop, kv_cache.rs:1889-1898) */
/* k_new, v_new: bf16 [1, n_tokens, n_kv_heads, head_dim] on the device; sin/cos optional (fused K RoPE). */
int32_t hs_cache_update(hs_cache *cache, const void *k_new, const void *v_new, int32_t n_tokens, int32_t start_pos,
                        const void *sin, const void *cos, int32_t rotary_dim, int32_t n_positions, hs_stream_t stream);
/* k_out, v_out: bf16 [1, seq_pos, n_kv_heads, head_dim] device buffers of the caller. */
int32_t hs_cache_get(hs_cache *cache, void *k_out, void *v_out, hs_stream_t stream);
int32_t hs_cache_reserve(hs_cache *cache, int32_t n_tokens); /* grow capacity (1024-token chunks / pages) */
int32_t hs_cache_clear(hs_cache *cache);
int32_t hs_cache_truncate_to(hs_cache *cache, int32_t n_tokens);
int32_t hs_cache_seq_pos(const hs_cache *cache);
int32_t hs_cache_set_seq_pos(hs_cache *cache, int32_t n_tokens); /* after writing through a view directly */
int32_t hs_cache_capacity(const hs_cache *cache);
int32_t hs_cache_num_pages(const hs_cache *cache);
int64_t hs_cache_memory_usage(const hs_cache *cache);
/* CPU offload / restore (LayerKVCache::to_device, kv_cache.rs:1838-1858; there a no-op for quantised and paged
 * storage, here available for every kind).  hs_cache_offload copies the seq_pos used token rows - K data, V data,
 * K scales, V scales, in that order, hs_cache_offload_bytes() bytes - into the caller's host buffer (pinned memory
 * makes the copies asynchronous up to the call's final synchronise), then releases the device storage or returns
 * the pages to the pool and leaves the cache empty.  hs_cache_restore refills an empty cache from such an image
 * (n_tokens = the seq_pos it was taken at); codes and scales come back byte for byte. */
int64_t hs_cache_offload_bytes(const hs_cache *cache);
int32_t hs_cache_offload(hs_cache *cache, void *host_buf, int64_t host_bytes, hs_stream_t stream);
int32_t hs_cache_restore(hs_cache *cache, const void *host_buf, int64_t host_bytes, int32_t n_tokens, hs_stream_t stream);
/* The same image as hs_cache_offload writes (codes and scales as stored), but the cache keeps its contents: for
 * checkpointing a sequence's cache and for checking stored codes (QuantizedTensor's data / absmax, kv_cache.rs:721-732). */
int32_t hs_cache_snapshot(const hs_cache *cache, void *host_buf, int64_t host_bytes, hs_stream_t stream);
/* One hs_kv_view over the caches of a batch (one sequence each); the handle owns the device pointer tables.
 * The tables hold the addresses the caches had when the view was built.  These calls release or replace storage and so
 * INVALIDATE every view built on the cache before them: hs_cache_update / hs_cache_reserve when they grow a contiguous
 * cache past its capacity (a new, larger slab replaces the old one: 1024-token chunks) or add pages to a paged one
 * (the new pages are not in the tables), hs_cache_clear, hs_cache_truncate_to (paged: whole pages go back to the
 * pool), hs_cache_offload / hs_cache_restore, hs_cache_destroy.  A kernel given a stale view reads or writes memory
 * that may belong to somebody else and cannot notice.  Reserve the capacity a decode loop will need before building
 * its view, or check with hs_view_is_current (host-only, cheap: HS_OK, or HS_ERR_ARG naming the cache that changed)
 * and rebuild.  The caches must outlive the view, and a pool its caches.  Growth copies on the legacy default stream
 * and synchronises the device, so writes in flight on other streams are complete before the old slab is released. */
int32_t hs_view_create(hs_cache *const *caches, int32_t n_caches, hs_view **out);
const hs_kv_view *hs_view_get(const hs_view *view);
int32_t hs_view_is_current(const hs_view *view);
void hs_view_destroy(hs_view *view);

/* ---- continuous-batching scheduler ---------------------------------------------------------------
 * The loop around the batched decode step that the reference leaves open: its engine has the batched step
 * (crates/hyprstream/src/runtime/torch_engine.rs:1475-1501 forward_batched_step) and two settings
 * (crates/hyprstream/src/config/mod.rs:2146-2152: continuous_batching, continuous_batch_max = 16) but no caller, and
 * its pool's typed exhaustion error says what a scheduler is to do with it (kv_cache.rs:482-505: defer admission and
 * retry once other sequences release blocks).  One scheduler serves one layer stack's pool; the host drives it from
 * the engine's single thread:
 *     hs_sched_submit(...)                                  any time: queue a sequence (prompt length, token budget)
 *     loop:  hs_sched_plan_step(..., &plan)                 admit while pages last (FIFO; a sequence whose prompt does not
 *                                                           fit is DEFERRED, not failed), plan the decode batch
 *            run the plan: prefill plan.prefill_caches[i] with its prompt (hs_cache_update + prefill attention), and
 *            one batched decode step over plan.view with plan.dst_pos / plan.seq_lens (hs_kv_quantize_write +
 *            hs_attn_decode, or hs_attn_decode_step)
 *            hs_sched_commit_step(..., finished ids)        positions advance, finished sequences are retired and their
 *                                                           pages go back to the pool for the deferred ones
 * Running sequences come before new ones: a running sequence that cannot get a page for its next token sits the step
 * out (n_stalled) and keeps its pages; there is no preemption, so when nothing at all can move the plan call returns
 * HS_ERR_POOL_EXHAUSTED and the host must retire something.  Sequence ids are >= 0 and tag the pool's pages.
 * Pointers in a plan belong to the scheduler and are valid until the next plan or commit; dst_pos / seq_lens / view
 * are device objects, built only with HS_SCHED_DEVICE_OBJECTS (without it the call is pure host logic). */
typedef struct hs_sched hs_sched;
#define HS_SCHED_DEVICE_OBJECTS 1
typedef struct hs_sched_plan {
    int32_t n_prefill;                 /* sequences admitted by this plan: prefill them before the decode step */
    const int64_t *prefill_ids;
    const int32_t *prefill_lens;
    hs_cache *const *prefill_caches;
    int32_t n_decode;                  /* the decode batch, in admission order */
    const int64_t *decode_ids;
    hs_cache *const *decode_caches;
    const int32_t *host_dst_pos;       /* host copy of dst_pos */
    const hs_kv_view *view;            /* device objects (NULL without HS_SCHED_DEVICE_OBJECTS or with an empty batch) */
    const int32_t *dst_pos, *seq_lens; /* device int32 [n_decode]: cache position of the new token, length attended */
    int32_t n_deferred, n_stalled, n_waiting, n_running;
} hs_sched_plan;
typedef struct hs_sched_stats_t {
    int32_t n_waiting, n_running, pages_free, reserved;
    int64_t n_admitted, n_retired, n_deferred, n_stalled, n_steps;
} hs_sched_stats_t;
int32_t hs_sched_create(hs_pool *pool, int32_t continuous_batch_max, int32_t max_seq_len, hs_sched **out);
void hs_sched_destroy(hs_sched *sched);
int32_t hs_sched_submit(hs_sched *sched, int64_t seq_id, int32_t prompt_len, int32_t max_new_tokens);
int32_t hs_sched_plan_step(hs_sched *sched, int32_t flags, hs_sched_plan *plan, hs_stream_t stream);
int32_t hs_sched_commit_step(hs_sched *sched, const int64_t *finished_ids, int32_t n_finished);
/* Between steps: drop a queued sequence, or retire a running one and return its pages (a client that went away; the way
 * out when hs_sched_plan_step reports that nothing can make progress). */
int32_t hs_sched_cancel(hs_sched *sched, int64_t seq_id);
int32_t hs_sched_stats(const hs_sched *sched, hs_sched_stats_t *out);

#ifdef __cplusplus
}
#endif
#endif /* HS_ATTN_H */
