// One decode step of a gated-DeltaNet layer between its projections, in one kernel: GatedDeltaNetLayer::forward with
// seq_len == 1 (architectures/qwen3_5.rs:627-784) - depthwise causal conv1d over the carried conv_state + SiLU, split into
// q | k | v, L2 norm of q and k, the gates, the recurrent rule on the fp32 state, RMSNormGated - for one (sequence, value
// head) per CTA.  The separate kernels of the same steps (gdn_edges.cu, gdn.cu) cost a launch each and at a batch of 64 the
// launches, not the bytes, are most of a layer's time; here the state moves once in and once out (2 * hk * hv * 4 bytes per
// sequence and head: the kernel is HBM-bound on the state) and everything else stays in shared memory.
//
// The arithmetic is the separate kernels', operation for operation and in the same order (conv sum by fmaf over the taps,
// rounded to bf16; SiLU in fp32, rounded to bf16; sums of squares by fmaf over a lane's values and a xor tree; the rule's
// partial sums per warp over rows w, w + 8, ... and then over the warps in order), so the results are the same bit for bit.
// A CTA owns a key head's q / k channels and all of its value heads, so every conv channel has one reader and its carried
// frames are shifted in place by that thread: no second launch.  Two CTAs per SM hide each other's latencies; a persistent CTA per SM moving the state by bulk copies through a ring of
// shared-memory buffers was measured slower (64-74 us against 61.5 us for batch 64 x 32 heads): with 8 warps the per-item
// chain of conv, rule and output row is longer than the item's transfer time.
#include "hs_common.cuh"

namespace hs {

constexpr int kGsThreads = 256;
constexpr int kGsWarps = kGsThreads / 32;
constexpr int kGsD = 128;  // head_k_dim = head_v_dim

__device__ __forceinline__ float gs_silu(float x) { return silu_fast(x); }
__device__ __forceinline__ float gs_softplus(float x) { return x > 20.0f ? x : log1pf(__expf(x)); }  // libtorch: beta 1, threshold 20

// grid (n_k_heads, n_seqs): a CTA takes a key head's q / k channels once and then its value heads one after the other - so every
// conv channel is read and its carried frames are shifted by one thread, in place.
// Thread (warp w, lane l) holds S[k][v] of the current value head for k = w + 8 i (i < 16), v = 4 l .. 4 l + 3.
template <int KS>
__global__ void __launch_bounds__(kGsThreads, 2)
gdn_step_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, uint16_t *__restrict__ conv_state, int has_state,
                const uint16_t *__restrict__ a_in, const uint16_t *__restrict__ b_in, const float *__restrict__ neg_a_exp,
                const float *__restrict__ dt_bias, const uint16_t *__restrict__ z, const float *__restrict__ norm_weight, float eps,
                float *__restrict__ state, uint16_t *__restrict__ y, int nk, int nv, float q_scale) {
    constexpr int R = kGsD / kGsWarps;  // state rows per thread
    __shared__ __align__(16) float s_qk[2][kGsD];                         // q, k (normalised)
    __shared__ __align__(16) float s_vv[2][kGsD];                         // v of the current value head (two buffers by head parity)
    __shared__ __align__(16) float s_pm[kGsWarps][kGsD], s_pr[kGsWarps][kGsD];
    __shared__ __align__(16) float s_o[kGsD];
    __shared__ float s_gb[2][2];
    const int b = blockIdx.y, kh = blockIdx.x, rr = nv / nk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int conv_dim = (2 * nk + nv) * kGsD;

    // conv1d + SiLU of 4 consecutive channels of head `group` (q | k | v order), the carried frames shifted in place; returns the
    // lane's sum of squares (a lane = 4 channels, as in the prologue kernel)
    auto conv4 = [&](int group, float (&yv)[4]) -> float {
        const int c0 = group * kGsD + 4 * lane;
        const uint2 raw = *reinterpret_cast<const uint2 *>(x + static_cast<int64_t>(b) * conv_dim + c0);
        const uint16_t xb[4] = {static_cast<uint16_t>(raw.x & 0xffffu), static_cast<uint16_t>(raw.x >> 16), static_cast<uint16_t>(raw.y & 0xffffu),
                                static_cast<uint16_t>(raw.y >> 16)};
        uint16_t *hp = conv_state + (static_cast<int64_t>(b) * conv_dim + c0) * (KS - 1);
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint16_t hist[KS - 1];
#pragma unroll
            for (int j = 0; j < KS - 1; ++j) hist[j] = has_state ? hp[c * (KS - 1) + j] : static_cast<uint16_t>(0);
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < KS - 1; ++j) acc = fmaf(bf16_bits_to_f32(w[static_cast<int64_t>(c0 + c) * KS + j]), bf16_bits_to_f32(hist[j]), acc);
            acc = fmaf(bf16_bits_to_f32(w[static_cast<int64_t>(c0 + c) * KS + KS - 1]), bf16_bits_to_f32(xb[c]), acc);
            yv[c] = bf16_round(gs_silu(bf16_round(acc)));
            ss = fmaf(yv[c], yv[c], ss);
            // the carried frames: drop the oldest, append this token (GatedDeltaNetLayer's conv_state, qwen3_5.rs:639-651)
#pragma unroll
            for (int j = 0; j < KS - 2; ++j) hp[c * (KS - 1) + j] = hist[j + 1];
            hp[c * (KS - 1) + KS - 2] = xb[c];
        }
        return ss;
    };

    // ---- q and k of the key head: warps 0 and 1 ----
    if (warp < 2) {
        float yv[4];
        float ss = conv4(warp == 0 ? kh : nk + kh, yv);
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        float mul = inv_l2_norm(ss);
        if (warp == 0) mul *= q_scale;
        *reinterpret_cast<float4 *>(&s_qk[warp][4 * lane]) = make_float4(yv[0] * mul, yv[1] * mul, yv[2] * mul, yv[3] * mul);
    }
    for (int hh = 0; hh < rr; ++hh) {
        const int h = kh * rr + hh, par = hh & 1;
        // the state first: its loads are in flight under the conv of v and the gates
        float4 S[R];
        float *sp = state + (static_cast<int64_t>(b) * nv + h) * kGsD * kGsD;
#pragma unroll
        for (int i = 0; i < R; ++i) S[i] = *reinterpret_cast<const float4 *>(sp + (warp + kGsWarps * i) * kGsD + 4 * lane);
        if (warp == 2) {
            float yv[4];
            conv4(2 * nk + h, yv);
            *reinterpret_cast<float4 *>(&s_vv[par][4 * lane]) = make_float4(yv[0], yv[1], yv[2], yv[3]);
        } else if (warp == 3 && lane == 0) {
            const int64_t idx = static_cast<int64_t>(b) * nv + h;
            s_gb[par][0] = neg_a_exp[h] * gs_softplus(bf16_bits_to_f32(a_in[idx]) + dt_bias[h]);
            s_gb[par][1] = 1.0f / (1.0f + __expf(-bf16_bits_to_f32(b_in[idx])));
        }
        __syncthreads();  // q, k, this head's v and gates are in shared memory; the previous head's partial sums have been read

        // ---- the rule: S <- exp(g) S; m = k^T S; delta = beta (v - m); S <- S + k delta^T; o = q^T (exp(g) S) + (q.k) delta ----
        const float *s_q = s_qk[0], *s_k = s_qk[1], *s_v = s_vv[par];
        const float decay = __expf(s_gb[par][0]), bt = s_gb[par][1];
        // (k and q of the thread's rows are read from shared memory where they are used - broadcast loads, 32 registers fewer; three
        // CTAs per SM, which that would allow with the state spilling a little, measured slower: 64.0 against 57.4 us)
        float qk = 0.0f;
        for (int i = lane; i < kGsD; i += 32) qk = fmaf(s_q[i], s_k[i], qk);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) qk += __shfl_xor_sync(0xffffffffu, qk, off);
        float4 pm = make_float4(0, 0, 0, 0), pr = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const float kr = s_k[warp + kGsWarps * i], qr = s_q[warp + kGsWarps * i];
            S[i].x *= decay; S[i].y *= decay; S[i].z *= decay; S[i].w *= decay;
            pm.x = fmaf(kr, S[i].x, pm.x); pm.y = fmaf(kr, S[i].y, pm.y); pm.z = fmaf(kr, S[i].z, pm.z); pm.w = fmaf(kr, S[i].w, pm.w);
            pr.x = fmaf(qr, S[i].x, pr.x); pr.y = fmaf(qr, S[i].y, pr.y); pr.z = fmaf(qr, S[i].z, pr.z); pr.w = fmaf(qr, S[i].w, pr.w);
        }
        *reinterpret_cast<float4 *>(&s_pm[warp][4 * lane]) = pm;
        *reinterpret_cast<float4 *>(&s_pr[warp][4 * lane]) = pr;
        __syncthreads();
        float4 m = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int ww = 0; ww < kGsWarps; ++ww) {
            const float4 a = *reinterpret_cast<const float4 *>(&s_pm[ww][4 * lane]);
            m.x += a.x; m.y += a.y; m.z += a.z; m.w += a.w;
        }
        const float4 vt = *reinterpret_cast<const float4 *>(&s_v[4 * lane]);
        const float4 d = make_float4((vt.x - m.x) * bt, (vt.y - m.y) * bt, (vt.z - m.z) * bt, (vt.w - m.w) * bt);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const float kr = s_k[warp + kGsWarps * i];
            S[i].x = fmaf(kr, d.x, S[i].x); S[i].y = fmaf(kr, d.y, S[i].y); S[i].z = fmaf(kr, d.z, S[i].z); S[i].w = fmaf(kr, d.w, S[i].w);
        }
#pragma unroll
        for (int i = 0; i < R; ++i) *reinterpret_cast<float4 *>(sp + (warp + kGsWarps * i) * kGsD + 4 * lane) = S[i];
        if (warp == 0) {
            float4 r = make_float4(0, 0, 0, 0);
#pragma unroll
            for (int ww = 0; ww < kGsWarps; ++ww) {
                const float4 a = *reinterpret_cast<const float4 *>(&s_pr[ww][4 * lane]);
                r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
            }
            *reinterpret_cast<float4 *>(&s_o[4 * lane]) = make_float4(fmaf(qk, d.x, r.x), fmaf(qk, d.y, r.y), fmaf(qk, d.z, r.z), fmaf(qk, d.w, r.w));
            __syncwarp();
            // ---- RMSNormGated of the row (16 lanes, 8 values each: the epilogue kernel's order) ----
            if (lane < 16) {
                const int64_t row = static_cast<int64_t>(b) * nv + h;
                const float4 a0 = *reinterpret_cast<const float4 *>(&s_o[lane * 8]), a1 = *reinterpret_cast<const float4 *>(&s_o[lane * 8 + 4]);
                const float xv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                float ss = 0.0f;
#pragma unroll
                for (int c = 0; c < 8; ++c) ss = fmaf(xv[c], xv[c], ss);
#pragma unroll
                for (int off = 1; off < 16; off <<= 1) ss += __shfl_xor_sync(0x0000ffffu, ss, off);
                const float rrms = rsqrtf(ss * (1.0f / 128.0f) + eps);
                const uint4 zr = *reinterpret_cast<const uint4 *>(z + row * kGsD + lane * 8);
                const uint32_t zw[4] = {zr.x, zr.y, zr.z, zr.w};
                const float4 w0 = *reinterpret_cast<const float4 *>(norm_weight + lane * 8), w1 = *reinterpret_cast<const float4 *>(norm_weight + lane * 8 + 4);
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint32_t o4[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float r0 = xv[2 * c] * rrms * wv[2 * c] * gs_silu(bf16lo(zw[c]));
                    const float r1 = xv[2 * c + 1] * rrms * wv[2 * c + 1] * gs_silu(bf16hi(zw[c]));
                    o4[c] = pack_bf16(r0, r1);
                }
                *reinterpret_cast<uint4 *>(y + row * kGsD + lane * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
            __syncwarp();
        }
    }
}

// One decode step of a DeltaNet layer for every sequence of a batch (see the kernel).  conv_state: the carried frames, read when
// `has_state` (zeros for a sequence's very first token) and shifted in place; `state` is updated in place.
int32_t gdn_step_fused(const void *mixed_qkv, const void *conv_weight, void *conv_state, int32_t has_state, const void *a_in, const void *b_in,
                       const float *neg_a_exp, const float *dt_bias, const void *z, const float *norm_weight, float eps, float *state, void *y,
                       int32_t n_seqs, int32_t n_k_heads, int32_t n_v_heads, int32_t kernel_size, hs_stream_t stream) {
    if (kernel_size != 4 && kernel_size != 2) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_layer_forward: conv kernel size %d (supported: 2, 4)", kernel_size);
    if (!aligned(mixed_qkv, 8) || !aligned(z, 16) || !aligned(y, 16) || !aligned(norm_weight, 16) || !aligned(state, 16))
        return fail(HS_ERR_ARG, "hs_gdn_layer_forward: mixed_qkv must be 8-byte, z, y, norm_weight and rec_state 16-byte aligned");
    cudaStream_t s = as_stream(stream);
    dim3 grid(n_k_heads, n_seqs);
    const float q_scale = 1.0f / sqrtf(static_cast<float>(kGsD));
    prof_begin(s);
#define HS_GS(KS)                                                                                                                  \
    gdn_step_kernel<KS><<<grid, kGsThreads, 0, s>>>(                                                                               \
        reinterpret_cast<const uint16_t *>(mixed_qkv), reinterpret_cast<const uint16_t *>(conv_weight),                            \
        reinterpret_cast<uint16_t *>(conv_state), has_state, reinterpret_cast<const uint16_t *>(a_in),                             \
        reinterpret_cast<const uint16_t *>(b_in), neg_a_exp, dt_bias, reinterpret_cast<const uint16_t *>(z), norm_weight, eps, state,  \
        reinterpret_cast<uint16_t *>(y), n_k_heads, n_v_heads, q_scale)
    if (kernel_size == 4) HS_GS(4); else HS_GS(2);
#undef HS_GS
    prof_end(s);
    return check_launch("hs_gdn_layer_forward (step)");
}

}  // namespace hs
