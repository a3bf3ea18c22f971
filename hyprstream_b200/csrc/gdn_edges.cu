// The elementwise steps either side of the gated-DeltaNet rule in GatedDeltaNetLayer::forward
// (architectures/qwen3_5.rs:627-701 before the rule, :771-784 after it), each fused into one pass over HBM:
//
//   prologue: depthwise causal conv1d (kernel ks <= 8, left context = the carried conv_state or zeros) in bf16 -> SiLU
//             (bf16) -> split into q | k | v -> q, k to fp32, x / max(||x||, 1e-3) per head, q * 1/sqrt(head_k_dim); v to
//             fp32; g = -exp(A_log) * softplus(a + dt_bias); beta = sigmoid(b); new conv_state = the last ks-1 frames
//   epilogue: RMSNormGated per value head: x * rsqrt(mean(x^2) + eps) * w * silu(z) -> bf16
//
// The reference runs these as ~25 libtorch operators (cat, permute, conv1d, silu, narrow, norm, clamp, div, mul,
// softplus, sigmoid, ...), every one a pass over the tensors.  Here a token's 2*key_dim + value_dim channels are read
// once (plus a ks-1 frame halo per token tile) and q, k, v, g, beta written once; both kernels are HBM-bound.
// Rounding follows the reference's dtypes: the conv sum is rounded to bf16, SiLU is evaluated on that bf16 value in
// fp32 and rounded to bf16 again, everything after is fp32.
#include "hs_common.cuh"

namespace hs {

constexpr int kEdgeThreads = 256;
constexpr int kEdgeTokens = 96;   // tokens per CTA tile (a multiple of the unroll of 6)
constexpr int kEdgeMaxTaps = 8;

__device__ __forceinline__ float silu_f(float x) { return silu_fast(x); }
// two values rounded to bf16 (nearest even) and back by one packed conversion and two integer operations (scalar conversions,
// one per value, kept the conversion unit 66 % busy; this form measured fastest)
__device__ __forceinline__ void bf16_round_pair(float &a, float &b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    a = __uint_as_float(r << 16);
    b = __uint_as_float(r & 0xffff0000u);
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(__expf(x)); }  // libtorch: beta 1, threshold 20

// Thread = 4 consecutive channels of one 128-channel group: a warp is one head, 8 heads per CTA; a CTA walks kEdgeTokens
// tokens keeping the last ks-1 frames of its channels in registers.
// Groups are heads: [0, nk) q heads, [nk, 2nk) k heads, [2nk, 2nk + nv) v heads (head dims are 128).
// TOut: float (the boundary's tensors) or uint16_t = bf16 bits (the layer entry's route to the chunked rule, which rounds q and k
// to bf16 itself and finds v a bf16 value already: half the bytes written here and read there, same results).
template <int KS, typename TOut>
__global__ void __launch_bounds__(kEdgeThreads, 3)
gdn_prologue_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, const uint16_t *__restrict__ state_in,
                    const uint16_t *__restrict__ a_in, const uint16_t *__restrict__ b_in, const float *__restrict__ neg_a_exp,
                    const float *__restrict__ dt_bias, TOut *__restrict__ q, TOut *__restrict__ k, TOut *__restrict__ v,
                    float *__restrict__ g, float *__restrict__ beta, int n_tokens, int nk, int nv, float q_scale) {
    constexpr int C = 4;  // channels per thread
    const int conv_dim = (2 * nk + nv) * 128;
    const int b = blockIdx.z, t0 = blockIdx.y * kEdgeTokens;
    const int group = blockIdx.x * (kEdgeThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int nt = min(kEdgeTokens, n_tokens - t0);
    // gates of this token tile (first channel block only)
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i < nt * nv; i += kEdgeThreads) {
            const int t = i / nv, h = i - t * nv;
            const int64_t idx = (static_cast<int64_t>(b) * n_tokens + t0 + t) * nv + h;
            g[idx] = neg_a_exp[h] * softplus_f(bf16_bits_to_f32(a_in[idx]) + dt_bias[h]);
            beta[idx] = 1.0f / (1.0f + __expf(-bf16_bits_to_f32(b_in[idx])));
        }
    }
    if (group >= 2 * nk + nv) return;  // (a whole warp)
    const int c0 = group * 128 + lane * C;
    float wt[C][KS];
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int j = 0; j < KS; ++j) wt[c][j] = bf16_bits_to_f32(w[static_cast<int64_t>(c0 + c) * KS + j]);
    // hist[c][j]: the last KS-1 frames of channel c as a ring: the frame at offset f from the tile start sits in slot
    // (f + KS-1) mod (KS-1) = f mod (KS-1)
    float hist[C][KS - 1];
#pragma unroll
    for (int j = 0; j < KS - 1; ++j) {
        const int tf = t0 - (KS - 1) + j;  // frame index in the token stream; negative = carried state
        if (tf >= 0) {
            const uint2 raw = *reinterpret_cast<const uint2 *>(x + (static_cast<int64_t>(b) * n_tokens + tf) * conv_dim + c0);
            hist[0][j] = bf16lo(raw.x); hist[1][j] = bf16hi(raw.x); hist[2][j] = bf16lo(raw.y); hist[3][j] = bf16hi(raw.y);
        } else {
#pragma unroll
            for (int c = 0; c < C; ++c)
                hist[c][j] = state_in ? bf16_bits_to_f32(state_in[(static_cast<int64_t>(b) * conv_dim + c0 + c) * (KS - 1) + (KS - 1) + tf]) : 0.0f;
        }
    }
    const bool is_v = group >= 2 * nk;
    const bool is_q = group < nk;
    TOut *dst = is_q ? q + (static_cast<int64_t>(b) * n_tokens * nk + group) * 128
               : (is_v ? v + (static_cast<int64_t>(b) * n_tokens * nv + (group - 2 * nk)) * 128
                       : k + (static_cast<int64_t>(b) * n_tokens * nk + (group - nk)) * 128);
    const int64_t tok_stride = static_cast<int64_t>(is_v ? nv : nk) * 128;
    // U tokens' loads are in flight together; U is a multiple of KS-1 so that the ring is indexed by constants after unrolling
    constexpr int U = (KS - 1) * (KS == 4 ? 2 : 6);  // (deeper batches measured no faster: 9 tokens the same, 12 slower)
    // ... and the next U tokens' loads are issued before this batch is worked on: the kernel is bound by bytes in flight
    // (a batch that lies wholly inside the tile is loaded and stored without per-token tests)
    const uint16_t *xt = x + (static_cast<int64_t>(b) * n_tokens + t0) * conv_dim + c0;
    auto load_batch = [&](int tb, uint2 (&r)[U]) {
        if (tb + U <= nt) {
#pragma unroll
            for (int u = 0; u < U; ++u) r[u] = *reinterpret_cast<const uint2 *>(xt + static_cast<int64_t>(tb + u) * conv_dim);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u)
                r[u] = tb + u < nt ? *reinterpret_cast<const uint2 *>(xt + static_cast<int64_t>(tb + u) * conv_dim) : make_uint2(0u, 0u);
        }
    };
    uint2 rawn[U];
    load_batch(0, rawn);
    for (int tb = 0; tb < nt; tb += U) {
        uint2 rawu[U];
#pragma unroll
        for (int u = 0; u < U; ++u) rawu[u] = rawn[u];
        if (tb + U < nt) load_batch(tb + U, rawn);
        // the conv sum of token u of the batch, rounded to bf16
        auto conv_token = [&](int u, float (&acc)[C]) {
            const float cur[C] = {bf16lo(rawu[u].x), bf16hi(rawu[u].x), bf16lo(rawu[u].y), bf16hi(rawu[u].y)};
#pragma unroll
            for (int c = 0; c < C; ++c) {
                acc[c] = 0.0f;
#pragma unroll
                for (int j = 0; j < KS - 1; ++j) acc[c] = fmaf(wt[c][j], hist[c][(u + j) % (KS - 1)], acc[c]);  // frame t - (KS-1) + j
                acc[c] = fmaf(wt[c][KS - 1], cur[c], acc[c]);
                hist[c][u % (KS - 1)] = cur[c];  // replaces the oldest frame
            }
            bf16_round_pair(acc[0], acc[1]);
            bf16_round_pair(acc[2], acc[3]);
        };
        const int n_store = min(U, nt - tb);
        if constexpr (sizeof(TOut) == 2) {
            if (is_v) {  // (warp-uniform) v as bf16 is SiLU's output rounded once: the packed conversion's result is what is stored
                uint2 yw[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float acc[C];
                    conv_token(u, acc);
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(silu_f(acc[0]), silu_f(acc[1])), hi = __floats2bfloat162_rn(silu_f(acc[2]), silu_f(acc[3]));
                    yw[u] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (u >= n_store) break;
                    *reinterpret_cast<uint2 *>(dst + (t0 + tb + u) * tok_stride + lane * C) = yw[u];
                }
                continue;
            }
        }
        float y[U][C], ss[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {  // (tokens past the end compute on zeros and are not stored)
            ss[u] = 0.0f;
            float acc[C];
            conv_token(u, acc);
#pragma unroll
            for (int c = 0; c < C; ++c) y[u][c] = silu_f(acc[c]);
            bf16_round_pair(y[u][0], y[u][1]);
            bf16_round_pair(y[u][2], y[u][3]);
#pragma unroll
            for (int c = 0; c < C; ++c) ss[u] = fmaf(y[u][c], y[u][c], ss[u]);
        }
        if (!is_v) {  // L2 norm over the 128 channels of the head = this warp (warp-uniform branch); the U reductions interleave
#pragma unroll
            for (int off = 1; off < 32; off <<= 1)
#pragma unroll
                for (int u = 0; u < U; ++u) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], off);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = tb + u;
            if (u >= n_store) break;
            float mul = 1.0f;
            if (!is_v) {
                mul = inv_l2_norm(ss[u]);  // x / clamp_min(norm, 1e-3), as a multiply by the reciprocal
                if (is_q) mul *= q_scale;
            }
            if constexpr (sizeof(TOut) == 4) {
                __stcs(reinterpret_cast<float4 *>(dst + (t0 + t) * tok_stride + lane * C),
                       make_float4(y[u][0] * mul, y[u][1] * mul, y[u][2] * mul, y[u][3] * mul));
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(y[u][0] * mul, y[u][1] * mul), hi = __floats2bfloat162_rn(y[u][2] * mul, y[u][3] * mul);
                *reinterpret_cast<uint2 *>(dst + (t0 + t) * tok_stride + lane * C) =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
            }
        }
    }
}

// new conv_state[b][c][j] = frame n_tokens - (KS-1) + j of the padded stream (old state, then the tokens).  Runs after the
// main kernel has read the old state; a thread owns one channel and reads all it needs before it writes (in place).
__global__ void gdn_conv_state_kernel(const uint16_t *__restrict__ x, const uint16_t *state_in, uint16_t *state_out, int n_tokens,
                                      int conv_dim, int ks1, int64_t total) {
    const int64_t bc = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // (sequence, channel)
    if (bc >= total) return;
    const int c = static_cast<int>(bc % conv_dim);
    const int64_t b = bc / conv_dim;
    uint16_t val[kEdgeMaxTaps - 1];
#pragma unroll
    for (int j = 0; j < kEdgeMaxTaps - 1; ++j) {
        val[j] = 0;
        if (j < ks1) {
            const int tf = n_tokens - ks1 + j;
            if (tf >= 0) val[j] = x[(b * n_tokens + tf) * conv_dim + c];
            else if (state_in) val[j] = state_in[bc * ks1 + ks1 + tf];
        }
    }
#pragma unroll
    for (int j = 0; j < kEdgeMaxTaps - 1; ++j)
        if (j < ks1) state_out[bc * ks1 + j] = val[j];
}

// RMSNormGated: thread = 8 values of one (token, head) row of 128, 16 threads per row
__global__ void __launch_bounds__(kEdgeThreads)
gdn_epilogue_kernel(const float *__restrict__ o, const uint16_t *__restrict__ z, const float *__restrict__ weight, float eps,
                    uint16_t *__restrict__ y, int64_t n_rows) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 16 + (threadIdx.x >> 4);
    const int l16 = threadIdx.x & 15;
    if (row >= n_rows) return;  // (whole 16-lane groups leave together; the shuffles below stay inside a group)
    const float4 a0 = *reinterpret_cast<const float4 *>(o + row * 128 + l16 * 8), a1 = *reinterpret_cast<const float4 *>(o + row * 128 + l16 * 8 + 4);
    const float xv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < 8; ++c) ss = fmaf(xv[c], xv[c], ss);
    const unsigned mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) ss += __shfl_xor_sync(mask, ss, off);
    const float rrms = rsqrtf(ss * (1.0f / 128.0f) + eps);
    const uint4 zr = *reinterpret_cast<const uint4 *>(z + row * 128 + l16 * 8);
    const uint32_t zw[4] = {zr.x, zr.y, zr.z, zr.w};
    const float4 w0 = *reinterpret_cast<const float4 *>(weight + l16 * 8), w1 = *reinterpret_cast<const float4 *>(weight + l16 * 8 + 4);
    const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    uint32_t out[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float r0 = xv[2 * c] * rrms * wv[2 * c] * silu_f(bf16lo(zw[c]));
        const float r1 = xv[2 * c + 1] * rrms * wv[2 * c + 1] * silu_f(bf16hi(zw[c]));
        out[c] = pack_bf16(r0, r1);
    }
    *reinterpret_cast<uint4 *>(y + row * 128 + l16 * 8) = make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace hs

using namespace hs;

namespace hs {

// The body of hs_gdn_prologue; `out_bf16`: q, k, v are written as bf16.
int32_t gdn_prologue_impl(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in,
                          const void *b_in, const float *neg_a_exp, const float *dt_bias, void *q, void *k, void *v, bool out_bf16, float *g,
                          float *beta, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                          int32_t head_v_dim, int32_t kernel_size, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_seqs < 0 || n_tokens < 0 || n_k_heads <= 0 || n_v_heads <= 0) return fail(HS_ERR_ARG, "hs_gdn_prologue: bad sizes");
    if (head_k_dim != 128 || head_v_dim != 128) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_prologue: head dims %d x %d (supported: 128 x 128)", head_k_dim, head_v_dim);
    if (kernel_size != 4 && kernel_size != 2) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_prologue: conv kernel size %d (supported: 2, 4)", kernel_size);
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (!mixed_qkv || !conv_weight || !conv_state || !a_in || !b_in || !neg_a_exp || !dt_bias || !q || !k || !v || !g || !beta)
        return fail(HS_ERR_ARG, "hs_gdn_prologue: NULL pointer");
    if (!aligned(mixed_qkv, 8) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16))
        return fail(HS_ERR_ARG, "hs_gdn_prologue: mixed_qkv, q, k, v must be 16-byte aligned");
    if (n_seqs > 65535) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_prologue: more than 65535 sequences");
    const int groups = 2 * n_k_heads + n_v_heads, conv_dim = groups * 128;
    cudaStream_t s = as_stream(stream);
    const uint16_t *st_in = has_state ? reinterpret_cast<const uint16_t *>(conv_state) : nullptr;
    dim3 grid((groups + kEdgeThreads / 32 - 1) / (kEdgeThreads / 32), (n_tokens + kEdgeTokens - 1) / kEdgeTokens, n_seqs);
    const float q_scale = 1.0f / sqrtf(static_cast<float>(head_k_dim));
    prof_begin(s);
#define HS_GDN_PRO(KS, T)                                                                                                           \
    gdn_prologue_kernel<KS, T><<<grid, kEdgeThreads, 0, s>>>(                                                                       \
        reinterpret_cast<const uint16_t *>(mixed_qkv), reinterpret_cast<const uint16_t *>(conv_weight), st_in,                      \
        reinterpret_cast<const uint16_t *>(a_in), reinterpret_cast<const uint16_t *>(b_in), neg_a_exp, dt_bias,                     \
        reinterpret_cast<T *>(q), reinterpret_cast<T *>(k), reinterpret_cast<T *>(v), g, beta, n_tokens, n_k_heads, n_v_heads, q_scale)
    if (out_bf16) {
        if (kernel_size == 4) HS_GDN_PRO(4, uint16_t); else HS_GDN_PRO(2, uint16_t);
    } else {
        if (kernel_size == 4) HS_GDN_PRO(4, float); else HS_GDN_PRO(2, float);
    }
#undef HS_GDN_PRO
    prof_end(s);
    if (int32_t e = check_launch("hs_gdn_prologue")) return e;
    // the new state is written by a second, stream-ordered launch: the first one still reads the old state
    return gdn_conv_state_shift(mixed_qkv, has_state ? conv_state : nullptr, conv_state, n_seqs, n_tokens, conv_dim, kernel_size, stream);
}

// conv_state <- the last kernel_size - 1 frames of (old state | the new tokens); state_in == NULL: the old state is zeros.
int32_t gdn_conv_state_shift(const void *mixed_qkv, const void *state_in, void *state_out, int32_t n_seqs, int32_t n_tokens, int32_t conv_dim,
                             int32_t kernel_size, hs_stream_t stream) {
    const int ks1 = kernel_size - 1;
    const int64_t total = static_cast<int64_t>(n_seqs) * conv_dim;
    gdn_conv_state_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint16_t *>(mixed_qkv), reinterpret_cast<const uint16_t *>(state_in), reinterpret_cast<uint16_t *>(state_out), n_tokens,
        conv_dim, ks1, total);
    return check_launch("hs_gdn_prologue (conv state)");
}

}  // namespace hs

extern "C" {

int32_t hs_gdn_prologue(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in,
                        const void *b_in, const float *neg_a_exp, const float *dt_bias, float *q, float *k, float *v, float *g,
                        float *beta, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                        int32_t head_v_dim, int32_t kernel_size, hs_stream_t stream) {
    return hs::gdn_prologue_impl(mixed_qkv, conv_weight, conv_state, has_state, a_in, b_in, neg_a_exp, dt_bias, q, k, v, false, g, beta, n_seqs, n_tokens,
                                 n_k_heads, n_v_heads, head_k_dim, head_v_dim, kernel_size, stream);
}

int32_t hs_gdn_epilogue(const float *o, const void *z, const float *norm_weight, float eps, void *y, int64_t n_rows, int32_t head_v_dim,
                        hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_rows < 0) return fail(HS_ERR_ARG, "hs_gdn_epilogue: bad sizes");
    if (head_v_dim != 128) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_epilogue: head dim %d (supported: 128)", head_v_dim);
    if (n_rows == 0) return HS_OK;
    if (!o || !z || !norm_weight || !y) return fail(HS_ERR_ARG, "hs_gdn_epilogue: NULL pointer");
    if (!aligned(o, 16) || !aligned(z, 16) || !aligned(y, 16) || !aligned(norm_weight, 16))
        return fail(HS_ERR_ARG, "hs_gdn_epilogue: o, z, y, norm_weight must be 16-byte aligned");
    const int64_t blocks = (n_rows + 15) / 16;
    if (blocks > 0x7fffffffLL) return fail(HS_ERR_ARG, "hs_gdn_epilogue: too many rows");
    cudaStream_t s = as_stream(stream);
    prof_begin(s);
    gdn_epilogue_kernel<<<static_cast<unsigned>(blocks), kEdgeThreads, 0, s>>>(o, reinterpret_cast<const uint16_t *>(z), norm_weight, eps,
                                                                              reinterpret_cast<uint16_t *>(y), n_rows);
    prof_end(s);
    return check_launch("hs_gdn_epilogue");
}

}  // extern "C"
