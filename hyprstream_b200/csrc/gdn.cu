// Gated DeltaNet state update on sm_100a: the recurrent rule of GatedDeltaNetLayer::forward
// (architectures/qwen3_5.rs:725-751), applied to 1 token (decode) or to a run of tokens.
//
//   per token and value head, fp32 state S[hk][hv]:
//     S <- exp(g) S;  m = k^T S;  delta = beta (v - m);  S <- S + k delta^T;  o = q^T S
//   (o is evaluated as q^T(exp(g)S) + (q.k) delta, so S is read once and written once per token)
//
// One CTA owns one (sequence, value head) pair and keeps the whole 128 x hv state in registers
// (64 floats per thread at 128 x 128), so a decode step moves exactly the state once in and once out:
// 2 * hk * hv * 4 bytes per (sequence, head) — the kernel is HBM-bound on the state.
// k/q head i feeds value heads [i*r, (i+1)*r), r = n_v_heads / n_k_heads (qwen3_5.rs:704-720).
#include "hs_common.cuh"

namespace hs {

constexpr int kGdnThreads = 256;
constexpr int kGdnWarps = kGdnThreads / 32;
constexpr int kGdnHV = 128;  // value head dim handled per CTA (one float4 per lane)

// HK: key head dim.  Thread (warp w, lane l) holds S[k][v] for k = w + 8*i (i < HK/8), v = 4l .. 4l+3.
template <int HK>
__global__ void __launch_bounds__(kGdnThreads)
gdn_recurrent_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                     const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state,
                     float *__restrict__ out, int n_tokens, int n_k_heads, int n_v_heads) {
    constexpr int R = HK / kGdnWarps;  // rows per thread
    __shared__ __align__(16) float s_k[2][HK], s_q[2][HK], s_v[2][kGdnHV];
    __shared__ __align__(16) float s_pm[2][kGdnWarps][kGdnHV], s_pr[2][kGdnWarps][kGdnHV];
    __shared__ float s_gb[2][2];
    const int b = blockIdx.y, h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = h / (n_v_heads / n_k_heads);
    float4 S[R];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * HK * kGdnHV;
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = *reinterpret_cast<const float4 *>(sp + (warp + kGdnWarps * i) * kGdnHV + 4 * lane);

    auto load_token = [&](int t, int buf) {
        const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
        const float *kp = k + (tok * n_k_heads + kh) * HK, *qp = q + (tok * n_k_heads + kh) * HK;
        const float *vp = v + (tok * n_v_heads + h) * kGdnHV;
        for (int i = threadIdx.x; i < HK; i += kGdnThreads) { s_k[buf][i] = kp[i]; s_q[buf][i] = qp[i]; }
        for (int i = threadIdx.x; i < kGdnHV; i += kGdnThreads) s_v[buf][i] = vp[i];
        if (threadIdx.x == 0) { s_gb[buf][0] = g[tok * n_v_heads + h]; s_gb[buf][1] = beta[tok * n_v_heads + h]; }
    };
    load_token(0, 0);
    __syncthreads();
    for (int t = 0; t < n_tokens; ++t) {
        const int buf = t & 1;
        if (t + 1 < n_tokens) load_token(t + 1, buf ^ 1);  // overlaps with this token's arithmetic
        const float decay = __expf(s_gb[buf][0]), bt = s_gb[buf][1];
        float kr[R], qr[R];
        float qk = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) { kr[i] = s_k[buf][warp + kGdnWarps * i]; qr[i] = s_q[buf][warp + kGdnWarps * i]; }
        // q.k over all HK rows: every warp computes it from shared memory
        for (int i = lane; i < HK; i += 32) qk = fmaf(s_q[buf][i], s_k[buf][i], qk);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) qk += __shfl_xor_sync(0xffffffffu, qk, off);
        float4 pm = make_float4(0, 0, 0, 0), pr = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            S[i].x *= decay; S[i].y *= decay; S[i].z *= decay; S[i].w *= decay;
            pm.x = fmaf(kr[i], S[i].x, pm.x); pm.y = fmaf(kr[i], S[i].y, pm.y); pm.z = fmaf(kr[i], S[i].z, pm.z); pm.w = fmaf(kr[i], S[i].w, pm.w);
            pr.x = fmaf(qr[i], S[i].x, pr.x); pr.y = fmaf(qr[i], S[i].y, pr.y); pr.z = fmaf(qr[i], S[i].z, pr.z); pr.w = fmaf(qr[i], S[i].w, pr.w);
        }
        const float4 vt = *reinterpret_cast<const float4 *>(&s_v[buf][4 * lane]);  // read before the barrier: the
        // buffer is refilled for token t + 2 by threads that are already one barrier ahead
        *reinterpret_cast<float4 *>(&s_pm[buf][warp][4 * lane]) = pm;
        *reinterpret_cast<float4 *>(&s_pr[buf][warp][4 * lane]) = pr;
        __syncthreads();  // partials of this token visible; next token's inputs loaded
        float4 m = make_float4(0, 0, 0, 0), r = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int w = 0; w < kGdnWarps; ++w) {
            const float4 a = *reinterpret_cast<const float4 *>(&s_pm[buf][w][4 * lane]);
            m.x += a.x; m.y += a.y; m.z += a.z; m.w += a.w;
        }
        const float4 d = make_float4((vt.x - m.x) * bt, (vt.y - m.y) * bt, (vt.z - m.z) * bt, (vt.w - m.w) * bt);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            S[i].x = fmaf(kr[i], d.x, S[i].x); S[i].y = fmaf(kr[i], d.y, S[i].y);
            S[i].z = fmaf(kr[i], d.z, S[i].z); S[i].w = fmaf(kr[i], d.w, S[i].w);
        }
        if (warp == 0) {
#pragma unroll
            for (int w = 0; w < kGdnWarps; ++w) {
                const float4 a = *reinterpret_cast<const float4 *>(&s_pr[buf][w][4 * lane]);
                r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
            }
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
            *reinterpret_cast<float4 *>(out + (tok * n_v_heads + h) * kGdnHV + 4 * lane) =
                make_float4(fmaf(qk, d.x, r.x), fmaf(qk, d.y, r.y), fmaf(qk, d.z, r.z), fmaf(qk, d.w, r.w));
        }
        // the buffers of token t are overwritten by load_token(t + 2) during token t + 1, i.e. after the next
        // barrier; the partial buffers alternate, so one barrier per token is enough
    }
#pragma unroll
    for (int i = 0; i < R; ++i) *reinterpret_cast<float4 *>(sp + (warp + kGdnWarps * i) * kGdnHV + 4 * lane) = S[i];
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_gdn_recurrent(const float *q, const float *k, const float *v, const float *g, const float *beta, float *state,
                         float *out, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                         int32_t head_v_dim, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_seqs < 0 || n_tokens < 0 || n_k_heads <= 0 || n_v_heads <= 0) return fail(HS_ERR_ARG, "hs_gdn_recurrent: bad sizes");
    if (n_v_heads % n_k_heads != 0) return fail(HS_ERR_ARG, "hs_gdn_recurrent: n_v_heads %d not a multiple of n_k_heads %d", n_v_heads, n_k_heads);
    if (head_v_dim != kGdnHV || (head_k_dim != 64 && head_k_dim != 128))
        return fail(HS_ERR_UNSUPPORTED, "hs_gdn_recurrent: head dims %d x %d (supported: key 64 or 128, value 128)", head_k_dim, head_v_dim);
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (!q || !k || !v || !g || !beta || !state || !out) return fail(HS_ERR_ARG, "hs_gdn_recurrent: NULL pointer");
    if (!aligned(state, 16) || !aligned(out, 16) || !aligned(q, 4) || !aligned(k, 4) || !aligned(v, 4))
        return fail(HS_ERR_ARG, "hs_gdn_recurrent: state and out must be 16-byte aligned");
    if (n_seqs > 65535) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_recurrent: more than 65535 sequences");
    dim3 grid(n_v_heads, n_seqs);
    cudaStream_t s = as_stream(stream);
    prof_begin(s);
    if (head_k_dim == 128) gdn_recurrent_kernel<128><<<grid, kGdnThreads, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
    else gdn_recurrent_kernel<64><<<grid, kGdnThreads, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
    prof_end(s);
    return check_launch("hs_gdn_recurrent");
}

}  // extern "C"
