// Batched layer-level entry points for the Qwen3.5 hybrid architecture: everything GatedDeltaNetLayer::forward and
// Qwen3_5FullAttention::forward do between their input and output projections, for a batch of sequences, as one call
// each, and a block-level call that runs a run of DeltaNet layers followed by one full-attention layer.
//
// The reference has no batched entry for this architecture: ModelOperations::forward_batched is implemented for Llama
// only and the trait default returns an error (architectures/mod.rs:268-280); Qwen3.5 decodes one sequence at a time
// through the layer dispatch (qwen3_5.rs:1864-1933) with one rec_state / conv_state slot per layer.  Here the states are
// batch-major tensors the caller owns ([n_seqs, ...]: one row per sequence, updated in place), the KV cache is a view
// over the batch's per-sequence caches, and a batch row computes exactly what the unbatched call computes for it.
//
// This file is host code: it chains the library's own entry points and only carves their intermediates out of the
// caller's workspace.
#include "hs_common.cuh"

namespace hs {

static inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }

struct GdnScratch {  // intermediates of one DeltaNet layer call, carved from the workspace
    float *q, *k, *v, *g, *beta, *o;
    size_t total;
};

static GdnScratch gdn_scratch(const hs_gdn_layer_params *p, int64_t n_seqs, int64_t n_tokens, unsigned char *base) {
    const size_t rows = static_cast<size_t>(n_seqs) * n_tokens;
    const size_t qk = up256(rows * p->n_k_heads * p->head_k_dim * 4), vv = up256(rows * p->n_v_heads * p->head_v_dim * 4);
    const size_t gb = up256(rows * p->n_v_heads * 4);
    GdnScratch s;
    size_t off = 0;
    auto take = [&](size_t bytes) { float *r = reinterpret_cast<float *>(base + off); off += bytes; return r; };
    s.q = take(qk); s.k = take(qk); s.v = take(vv); s.g = take(gb); s.beta = take(gb); s.o = take(vv);
    s.total = off;
    return s;
}

static int32_t check_gdn_params(const hs_gdn_layer_params *p, const char *who) {
    if (!p) return fail(HS_ERR_ARG, "%s: NULL layer parameters", who);
    if (p->n_k_heads <= 0 || p->n_v_heads <= 0 || p->n_v_heads % p->n_k_heads != 0)
        return fail(HS_ERR_ARG, "%s: n_v_heads %d must be a positive multiple of n_k_heads %d", who, p->n_v_heads, p->n_k_heads);
    if (p->head_k_dim != 128 || p->head_v_dim != 128) return fail(HS_ERR_UNSUPPORTED, "%s: head dims %d x %d (supported: 128 x 128)", who, p->head_k_dim, p->head_v_dim);
    if (!p->conv_weight || !p->neg_a_exp || !p->dt_bias || !p->norm_weight) return fail(HS_ERR_ARG, "%s: NULL weight", who);
    return HS_OK;
}

static int32_t check_attn_params(const hs_qwen_attn_params *p, const char *who) {
    if (!p) return fail(HS_ERR_ARG, "%s: NULL layer parameters", who);
    if (p->n_q_heads <= 0 || p->n_kv_heads <= 0 || p->n_q_heads % p->n_kv_heads != 0)
        return fail(HS_ERR_ARG, "%s: n_q_heads %d must be a positive multiple of n_kv_heads %d", who, p->n_q_heads, p->n_kv_heads);
    if (p->head_dim != 64 && p->head_dim != 128 && p->head_dim != 256) return fail(HS_ERR_UNSUPPORTED, "%s: head_dim %d", who, p->head_dim);
    return HS_OK;
}

}  // namespace hs

using namespace hs;

extern "C" {

int64_t hs_gdn_layer_workspace_bytes(const hs_gdn_layer_params *params, int32_t n_seqs, int32_t n_tokens) {
    if (!params || n_seqs < 0 || n_tokens < 0) return HS_ERR_ARG;
    return static_cast<int64_t>(gdn_scratch(params, n_seqs, n_tokens, nullptr).total);
}

int32_t hs_gdn_layer_forward(const hs_gdn_layer_params *params, const void *mixed_qkv, const void *z, const void *a_in, const void *b_in,
                             void *conv_state, float *rec_state, int32_t has_state, int32_t n_seqs, int32_t n_tokens, void *y,
                             void *workspace, int64_t workspace_bytes, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = check_gdn_params(params, "hs_gdn_layer_forward")) return st;
    if (n_seqs < 0 || n_tokens < 0) return fail(HS_ERR_ARG, "hs_gdn_layer_forward: negative sizes");
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (!mixed_qkv || !z || !a_in || !b_in || !conv_state || !rec_state || !y || !workspace) return fail(HS_ERR_ARG, "hs_gdn_layer_forward: NULL pointer");
    if (!aligned(workspace, 256)) return fail(HS_ERR_ARG, "hs_gdn_layer_forward: the workspace must be 256-byte aligned");
    GdnScratch s = gdn_scratch(params, n_seqs, n_tokens, static_cast<unsigned char *>(workspace));
    if (workspace_bytes < static_cast<int64_t>(s.total))
        return fail(HS_ERR_WORKSPACE, "hs_gdn_layer_forward: workspace %lld < %lld bytes", static_cast<long long>(workspace_bytes), static_cast<long long>(s.total));
    // a state that is being started is zero
    if (!has_state) {
        cudaError_t e = cudaMemsetAsync(rec_state, 0, static_cast<size_t>(n_seqs) * params->n_v_heads * params->head_k_dim * params->head_v_dim * 4, as_stream(stream));
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_gdn_layer_forward: %s", cudaGetErrorString(e));
    }
    if (n_tokens == 1 && n_seqs <= 65535) {
        // a decode step: conv (with the conv_state shift), gates, the recurrent rule and RMSNormGated in one kernel
        return gdn_step_fused(mixed_qkv, params->conv_weight, conv_state, has_state, a_in, b_in, params->neg_a_exp, params->dt_bias, z, params->norm_weight,
                              params->norm_eps, rec_state, y, n_seqs, params->n_k_heads, params->n_v_heads, params->kernel_size, stream);
    }
    // conv1d + SiLU + split + L2 norm + gates (qwen3_5.rs:627-701).  For a prompt q, k, v go to the chunked rule as bf16: that kernel
    // rounds q and k to bf16 first thing and v is a bf16 value already, so the results are the same and half the bytes move.
    const bool chunked = n_tokens > 1;
    if (int32_t st = gdn_prologue_impl(mixed_qkv, params->conv_weight, conv_state, has_state, a_in, b_in, params->neg_a_exp, params->dt_bias, s.q, s.k, s.v,
                                       chunked, s.g, s.beta, n_seqs, n_tokens, params->n_k_heads, params->n_v_heads, params->head_k_dim, params->head_v_dim,
                                       params->kernel_size, stream))
        return st;
    // the rule: recurrent for a decode step, chunked for a prompt (qwen3_5.rs:725-769)
    int32_t st;
    if (n_tokens == 1)
        st = hs_gdn_recurrent(s.q, s.k, s.v, s.g, s.beta, rec_state, s.o, n_seqs, 1, params->n_k_heads, params->n_v_heads, params->head_k_dim,
                              params->head_v_dim, stream);
    else
        st = gdn_chunk_impl(s.q, s.k, s.v, true, s.g, s.beta, rec_state, s.o, n_seqs, n_tokens, params->n_k_heads, params->n_v_heads, params->head_k_dim,
                            params->head_v_dim, stream);
    if (st != HS_OK) return st;
    // RMSNormGated (qwen3_5.rs:305-313,771-784)
    return hs_gdn_epilogue(s.o, z, params->norm_weight, params->norm_eps, y, static_cast<int64_t>(n_seqs) * n_tokens * params->n_v_heads, params->head_v_dim,
                           stream);
}

int64_t hs_qwen_attn_layer_workspace_bytes(const hs_qwen_attn_params *params, int32_t n_seqs, int32_t n_tokens) {
    if (!params || n_seqs < 0 || n_tokens < 0) return HS_ERR_ARG;
    const size_t rows = static_cast<size_t>(n_seqs) * n_tokens;
    const size_t qb = up256(rows * params->n_q_heads * params->head_dim * 2), kb = up256(rows * params->n_kv_heads * params->head_dim * 2);
    const int64_t dec = n_tokens == 1 ? hs_attn_decode_workspace_bytes(n_seqs, params->n_q_heads, params->head_dim) : 0;
    return static_cast<int64_t>(2 * qb + kb) + (dec > 0 ? static_cast<int64_t>(up256(static_cast<size_t>(dec))) : 0);
}

int32_t hs_qwen_attn_layer_forward(const hs_qwen_attn_params *params, const void *q_proj, const void *k_proj, const void *v_proj,
                                   const hs_kv_view *view, const int32_t *positions, const int32_t *dst_pos, const int32_t *seq_lens, int32_t n_seqs,
                                   int32_t n_tokens, void *out, void *workspace, int64_t workspace_bytes, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (int32_t st = check_attn_params(params, "hs_qwen_attn_layer_forward")) return st;
    if (int32_t st = validate_view(view)) return st;
    if (n_seqs < 0 || n_tokens < 0) return fail(HS_ERR_ARG, "hs_qwen_attn_layer_forward: negative sizes");
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (view->n_kv_heads != params->n_kv_heads || view->head_dim != params->head_dim)
        return fail(HS_ERR_ARG, "hs_qwen_attn_layer_forward: the cache view's geometry differs from the layer's");
    if (!q_proj || !k_proj || !v_proj || !positions || !dst_pos || !out || !workspace) return fail(HS_ERR_ARG, "hs_qwen_attn_layer_forward: NULL pointer");
    if (n_tokens == 1 && !seq_lens) return fail(HS_ERR_ARG, "hs_qwen_attn_layer_forward: a decode step needs seq_lens");
    if (!aligned(workspace, 256)) return fail(HS_ERR_ARG, "hs_qwen_attn_layer_forward: the workspace must be 256-byte aligned");
    const int64_t need = hs_qwen_attn_layer_workspace_bytes(params, n_seqs, n_tokens);
    if (workspace_bytes < need)
        return fail(HS_ERR_WORKSPACE, "hs_qwen_attn_layer_forward: workspace %lld < %lld bytes", static_cast<long long>(workspace_bytes), static_cast<long long>(need));
    const int hq = params->n_q_heads, hkv = params->n_kv_heads, d = params->head_dim;
    const int64_t rows = static_cast<int64_t>(n_seqs) * n_tokens;
    unsigned char *w = static_cast<unsigned char *>(workspace);
    const size_t qb = up256(static_cast<size_t>(rows) * hq * d * 2), kb = up256(static_cast<size_t>(rows) * hkv * d * 2);
    void *query = w, *gate = w + qb, *k_rot = w + 2 * qb, *dec_ws = w + 2 * qb + kb;
    // q_proj rows are [n_q_heads, 2 * head_dim]: query half | gate half (qwen3_5.rs:965-967); (1 + w) QK-norm, partial RoPE.
    // A decode step copies the gate halves out (its kernel wants them dense); a prompt's attention reads them in place.
    if (int32_t st = hs_qk_norm_rope(q_proj, static_cast<int64_t>(hq) * 2 * d, 2 * d, query, n_tokens == 1 ? gate : nullptr, params->q_norm_weight, params->norm_eps, 1, params->sin,
                                     params->cos, positions, params->n_positions, params->rotary_dim, rows, hq, d, stream))
        return st;
    // K: norm + rotation + cache update in one pass over the new keys (qwen3_5.rs:971-999); a prompt also keeps the normed,
    // rotated keys in bf16 for its own attention.  The keys' RoPE rows are their cache positions dst_pos[s] + t, which is
    // what `positions` holds for the queries.
    if (int32_t st = hs_kv_norm_rope_quantize_write(view, k_proj, v_proj, n_seqs, n_tokens, dst_pos, params->k_norm_weight, params->norm_eps, 1, params->sin,
                                                    params->cos, params->rotary_dim, params->n_positions, n_tokens == 1 ? nullptr : k_rot, stream))
        return st;
    if (n_tokens == 1)
        return hs_attn_decode(query, view, seq_lens, n_seqs, hq, params->softmax_scale, out, gate, dec_ws,
                              hs_attn_decode_workspace_bytes(n_seqs, hq, d), nullptr, nullptr, stream);
    return hs::prefill_causal_impl(query, k_rot, v_proj, out, static_cast<const uint16_t *>(q_proj) + d, static_cast<int64_t>(hq) * 2 * d, 2 * d, n_seqs, n_tokens,
                                   n_tokens, hq, hkv, d, params->softmax_scale, stream);
}

int64_t hs_qwen_block_workspace_bytes(const hs_gdn_layer_params *gdn, int32_t n_gdn, const hs_qwen_attn_params *attn, int32_t n_seqs,
                                      int32_t n_tokens) {
    int64_t need = 0;
    for (int i = 0; i < n_gdn; ++i) {
        const int64_t b = hs_gdn_layer_workspace_bytes(gdn + i, n_seqs, n_tokens);
        if (b < 0) return b;
        need = b > need ? b : need;
    }
    if (attn) {
        const int64_t b = hs_qwen_attn_layer_workspace_bytes(attn, n_seqs, n_tokens);
        if (b < 0) return b;
        need = b > need ? b : need;
    }
    return need;
}

int32_t hs_qwen_block_forward(const hs_gdn_layer_params *gdn, const hs_gdn_layer_io *gdn_io, int32_t n_gdn, const hs_qwen_attn_params *attn,
                              const hs_qwen_attn_io *attn_io, int32_t has_state, int32_t n_seqs, int32_t n_tokens, void *workspace,
                              int64_t workspace_bytes, hs_stream_t stream) {
    if (n_gdn < 0 || (n_gdn > 0 && (!gdn || !gdn_io))) return fail(HS_ERR_ARG, "hs_qwen_block_forward: bad DeltaNet layer arrays");
    if ((attn == nullptr) != (attn_io == nullptr)) return fail(HS_ERR_ARG, "hs_qwen_block_forward: attention parameters and inputs go together");
    for (int i = 0; i < n_gdn; ++i) {
        const hs_gdn_layer_io &io = gdn_io[i];
        if (int32_t st = hs_gdn_layer_forward(gdn + i, io.mixed_qkv, io.z, io.a_in, io.b_in, io.conv_state, io.rec_state, has_state, n_seqs, n_tokens, io.y,
                                              workspace, workspace_bytes, stream))
            return st;
    }
    if (attn)
        return hs_qwen_attn_layer_forward(attn, attn_io->q_proj, attn_io->k_proj, attn_io->v_proj, attn_io->view, attn_io->positions, attn_io->dst_pos,
                                          attn_io->seq_lens, n_seqs, n_tokens, attn_io->out, workspace, workspace_bytes, stream);
    return HS_OK;
}

}  // extern "C"
