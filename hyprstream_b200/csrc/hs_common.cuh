// Shared host/device helpers for the sm_100a attention + KV-cache kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/hs_attn.h"

namespace hs {

// ---- host-side status plumbing --------------------------------------------------------------
void set_error(const char *fmt, ...);
int32_t fail(int32_t code, const char *fmt, ...);
int32_t check_device();             // HS_OK on compute capability 10.x, else HS_ERR_DEVICE
int32_t check_launch(const char *what);  // cudaGetLastError -> status
int sm_count();
int current_device();  // ordinal of the current device, -1 if there is none
// Address (on the current device) of the error words: word 0 holds the HS_DEVERR_* flags that kernels set instead of
// faulting (hs_attn_take_device_error() reads and clears it); word 1 holds the id of the latest launch in which a bounded
// wait ran out, so that the remaining CTAs of THAT launch can return at once (later launches carry another id and are
// not affected by it).  The address is looked up once per device.
int *device_error_word();
uint32_t next_launch_id();  // never 0

// Internal forms of hs_gdn_prologue / hs_gdn_chunk_prefill with bf16 q, k, v between them (gdn_edges.cu, gdn_chunk.cu).
int32_t gdn_prologue_impl(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in,
                          const void *b_in, const float *neg_a_exp, const float *dt_bias, void *q, void *k, void *v, bool out_bf16, float *g,
                          float *beta, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                          int32_t head_v_dim, int32_t kernel_size, hs_stream_t stream);
int32_t gdn_conv_state_shift(const void *mixed_qkv, const void *state_in, void *state_out, int32_t n_seqs, int32_t n_tokens, int32_t conv_dim,
                             int32_t kernel_size, hs_stream_t stream);
// One decode step of a DeltaNet layer in one kernel (gdn_step.cu); conv_state is read (when has_state) and shifted in place.
int32_t gdn_step_fused(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in, const void *b_in,
                       const float *neg_a_exp, const float *dt_bias, const void *z, const float *norm_weight, float eps, float *state, void *y,
                       int32_t n_seqs, int32_t n_k_heads, int32_t n_v_heads, int32_t kernel_size, hs_stream_t stream);
// hs_attn_prefill_causal with the gate's strides given (elements between tokens / between heads); prefill.cu
int32_t prefill_causal_impl(const void *q, const void *k, const void *v, void *out, const void *gate, int64_t gate_ts, int64_t gate_hs,
                            int32_t n_seqs, int32_t q_len, int32_t kv_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                            float softmax_scale, hs_stream_t stream);
int32_t gdn_chunk_impl(const void *q, const void *k, const void *v, bool in_bf16, const float *g, const float *beta, float *state, float *out,
                       int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim, int32_t head_v_dim, hs_stream_t stream);

// Launch configuration is per device (cudaFuncSetAttribute, occupancy, whether cooperative launches are accepted): a
// process that drives several GPUs configures each kernel once on each.  One int of state per device ordinal, 0 = not
// configured yet.  Two threads may both configure a device; the calls are idempotent.
constexpr int kMaxDevices = 64;
struct PerDeviceState {
    std::atomic<int> v[kMaxDevices];
    int get(int dev) const { return dev >= 0 && dev < kMaxDevices ? v[dev].load(std::memory_order_acquire) : 0; }
    void set(int dev, int x) { if (dev >= 0 && dev < kMaxDevices) v[dev].store(x, std::memory_order_release); }
};

static inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline cudaStream_t as_stream(hs_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

int32_t validate_view(const hs_kv_view *v);
// Bracket the dominant kernel of an entry point; records CUDA events only while profiling is on.
void prof_begin(cudaStream_t s);
void prof_end(cudaStream_t s);

// Kernel-argument copy of hs_kv_view (passed by value).
struct ViewDev {
    void *const *k_pages, *const *v_pages, *const *k_scale_pages, *const *v_scale_pages;
    int kind, scale_dtype, block, n_kv_heads, head_dim, page_tokens, pages_per_seq;
};

static inline ViewDev to_dev(const hs_kv_view *v) {
    ViewDev d;
    d.k_pages = v->k_pages; d.v_pages = v->v_pages; d.k_scale_pages = v->k_scale_pages; d.v_scale_pages = v->v_scale_pages;
    d.kind = v->kind; d.scale_dtype = v->scale_dtype; d.block = v->kind == HS_KV_BF16 ? v->head_dim : v->block;
    d.n_kv_heads = v->n_kv_heads; d.head_dim = v->head_dim; d.page_tokens = v->page_tokens; d.pages_per_seq = v->pages_per_seq;
    return d;
}

// ---- exchange of KV-length-shard results between GPUs inside the decode kernel -----------------------
// Every rank owns an "inbox" that all ranks can address (its own memory for itself, a peer mapping for the others).
// A value travels as one 8-byte word {value, epoch}: 8-byte stores and loads are single transactions, so a reader that
// sees this step's epoch in a word also sees its value - no fence and no separate flag are needed, and the latency of an
// exchange is one trip over NVLink plus the reader's poll.  Layout in 8-byte words, with W = world, R = rows_cap,
// D = head_dim and h = epoch & 1 (two halves, so that a rank that is one step ahead never overwrites what a slower
// rank still reads): row `row` of source s in half h starts at ((h * W + s) * R + row) * (D + 2); words 0 .. D-1 hold the
// normalised output, word D the log-sum-exp, word D+1 pads the row to 16 bytes.
constexpr int kShardMaxWorld = 8;
struct ShardArgs {
    unsigned long long *inbox[kShardMaxWorld];
    int rank, world;          // world == 0: no exchange
    unsigned int epoch;       // never 0 (a cleared inbox holds epoch 0)
    int push_only;            // deliver this rank's part, do not wait for the others, write no output
    long long wait_cycles;    // limit of the wait for the other ranks' parts
    long long rows_cap;
};

// One new token per sequence that the decode kernel writes into the cache itself (int8 caches) before it attends:
// k_new == NULL: off.  The token of sequence s goes to position seq_lens[s] - 1.
struct AppendArgs {
    const uint16_t *k_new, *v_new;  // bf16 [n_seqs, 1, n_kv_heads, head_dim]
    const uint16_t *sin, *cos;      // optional fused K rotation
    int rotary_dim, n_positions;
};
int32_t kv_write_at_end(const hs_kv_view *view, const void *k_new, const void *v_new, int32_t n_seqs, const int32_t *seq_lens, const void *sin,
                        const void *cos, int32_t rotary_dim, int32_t n_positions, hs_stream_t stream);

// ---- device helpers --------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    return static_cast<uint32_t>(f32_to_bf16_bits(lo)) | (static_cast<uint32_t>(f32_to_bf16_bits(hi)) << 16);
}
// a (op) b rounded to bf16, as libtorch's bf16 elementwise kernels do (f32 op, then round).
__device__ __forceinline__ float bf16_round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
// x * sigmoid(x) on the approximate exponential and reciprocal: the values of __fdividef(x, 1 + __expf(-x)) without the
// denormal handling of the two intrinsics (three more instructions per value; 1 + tiny is 1 either way)
// 1 / max(sqrt(ss), 1e-3) = min(rsqrt(ss), 1e3) on the approximate reciprocal square root (relative error 2^-22; ss = 0 gives 1e3)
__device__ __forceinline__ float inv_l2_norm(float ss) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(ss));
    return fminf(r, 1e3f);
}
__device__ __forceinline__ float silu_fast(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return x * r;
}

__device__ __forceinline__ float load_scale(const void *p, int64_t idx, int scale_dtype) {
    return scale_dtype == HS_SCALE_F16 ? __half2float(reinterpret_cast<const __half *>(p)[idx])
                                       : reinterpret_cast<const float *>(p)[idx];
}

// NF4 / FP4 codebooks (bitsandbytes-sys/src/lib.rs:131-148,152-169)
static __device__ __constant__ float c_nf4[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230945587158f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
static __device__ __constant__ float c_fp4[16] = {0.0f,  0.0625f, 0.125f, 0.1875f, 0.25f,  0.3125f, 0.375f, 0.4375f,
                                                  0.5f,  0.5625f, 0.625f, 0.6875f, 0.75f,  0.8125f, 0.875f, 1.0f};

// ---- flat split-KV partition -------------------------------------------------------------------
// The KV tokens of all sequences are cut into tiles of `tile` tokens; the concatenated tile list is
// divided evenly over `n_ctas` CTAs.  CTA c owns tiles [c*total/n_ctas, (c+1)*total/n_ctas).  A
// (cta, sequence) pair that overlaps writes one partial into slot cta + sequence (unique because
// both indices are non-decreasing along the tile list).
__device__ __forceinline__ int64_t part_begin(int64_t c, int64_t total, int64_t n_ctas) { return c * total / n_ctas; }

}  // namespace hs
