// Gated DeltaNet state update on sm_100a: the recurrent rule of GatedDeltaNetLayer::forward
// (architectures/qwen3_5.rs:725-751), applied to 1 token (decode) or to a run of tokens.
//
//   per token and value head, fp32 state S[hk][hv]:
//     S <- exp(g) S;  m = k^T S;  delta = beta (v - m);  S <- S + k delta^T;  o = q^T S
//   (o is evaluated as q^T(exp(g)S) + (q.k) delta, so S is read once and written once per token)
//
// One CTA owns 64 of the 128 value columns of one (sequence, value head) pair — the rule is independent per
// value column — and keeps its 128 x 64 slice of the state in registers (32 floats per thread), several CTAs
// per SM, so a decode step moves exactly the state once in and once out:
// 2 * hk * hv * 4 bytes per (sequence, head) — the kernel is HBM-bound on the state.
// k/q head i feeds value heads [i*r, (i+1)*r), r = n_v_heads / n_k_heads (qwen3_5.rs:704-720).
#include "hs_common.cuh"

namespace hs {

constexpr int kGdnThreads = 256;
constexpr int kGdnWarps = kGdnThreads / 32;
constexpr int kGdnHV = 128;    // value head dim
constexpr int kGdnCols = 64;   // state columns per CTA: the rule is independent per value column, so a head is cut in two

// HK: key head dim.  Thread (warp w, lane l) of column block c holds S[k][v] for k = w + 8*i (i < HK/8), v = 64c + 2l, 2l+1.
template <int HK>
__global__ void __launch_bounds__(kGdnThreads)
gdn_recurrent_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                     const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state,
                     float *__restrict__ out, int n_tokens, int n_k_heads, int n_v_heads) {
    constexpr int R = HK / kGdnWarps;  // rows per thread
    __shared__ __align__(16) float s_k[2][HK], s_q[2][HK], s_v[2][kGdnCols];
    __shared__ __align__(16) float s_pm[2][kGdnWarps][kGdnCols], s_pr[2][kGdnWarps][kGdnCols];
    __shared__ float s_gb[2][2];
    const int b = blockIdx.y, h = blockIdx.x >> 1, c0 = (blockIdx.x & 1) * kGdnCols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = h / (n_v_heads / n_k_heads);
    float2 S[R];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * HK * kGdnHV + c0;
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = *reinterpret_cast<const float2 *>(sp + (warp + kGdnWarps * i) * kGdnHV + 2 * lane);

    auto load_token = [&](int t, int buf) {
        const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
        const float *kp = k + (tok * n_k_heads + kh) * HK, *qp = q + (tok * n_k_heads + kh) * HK;
        const float *vp = v + (tok * n_v_heads + h) * kGdnHV + c0;
        for (int i = threadIdx.x; i < HK; i += kGdnThreads) { s_k[buf][i] = kp[i]; s_q[buf][i] = qp[i]; }
        for (int i = threadIdx.x; i < kGdnCols; i += kGdnThreads) s_v[buf][i] = vp[i];
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
        float2 pm = make_float2(0, 0), pr = make_float2(0, 0);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            S[i].x *= decay; S[i].y *= decay;
            pm.x = fmaf(kr[i], S[i].x, pm.x); pm.y = fmaf(kr[i], S[i].y, pm.y);
            pr.x = fmaf(qr[i], S[i].x, pr.x); pr.y = fmaf(qr[i], S[i].y, pr.y);
        }
        const float2 vt = *reinterpret_cast<const float2 *>(&s_v[buf][2 * lane]);  // read before the barrier: the
        // buffer is refilled for token t + 2 by threads that are already one barrier ahead
        *reinterpret_cast<float2 *>(&s_pm[buf][warp][2 * lane]) = pm;
        *reinterpret_cast<float2 *>(&s_pr[buf][warp][2 * lane]) = pr;
        __syncthreads();  // partials of this token visible; next token's inputs loaded
        float2 m = make_float2(0, 0), r = make_float2(0, 0);
#pragma unroll
        for (int w = 0; w < kGdnWarps; ++w) {
            const float2 a = *reinterpret_cast<const float2 *>(&s_pm[buf][w][2 * lane]);
            m.x += a.x; m.y += a.y;
        }
        const float2 d = make_float2((vt.x - m.x) * bt, (vt.y - m.y) * bt);
#pragma unroll
        for (int i = 0; i < R; ++i) { S[i].x = fmaf(kr[i], d.x, S[i].x); S[i].y = fmaf(kr[i], d.y, S[i].y); }
        if (warp == 0) {
#pragma unroll
            for (int w = 0; w < kGdnWarps; ++w) {
                const float2 a = *reinterpret_cast<const float2 *>(&s_pr[buf][w][2 * lane]);
                r.x += a.x; r.y += a.y;
            }
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
            *reinterpret_cast<float2 *>(out + (tok * n_v_heads + h) * kGdnHV + c0 + 2 * lane) = make_float2(fmaf(qk, d.x, r.x), fmaf(qk, d.y, r.y));
        }
        // the buffers of token t are overwritten by load_token(t + 2) during token t + 1, i.e. after the next
        // barrier; the partial buffers alternate, so one barrier per token is enough
    }
#pragma unroll
    for (int i = 0; i < R; ++i) *reinterpret_cast<float2 *>(sp + (warp + kGdnWarps * i) * kGdnHV + 2 * lane) = S[i];
}

// ---- column-owner form for runs of tokens --------------------------------------------------------------------
// The rule is independent per value column: m[v], delta[v], S[:,v] and o[v] never mix columns.  Here a pair of lanes owns
// one column of the state (HK/2 floats each in registers), so a token needs one shuffle for m and one for o and no barrier: S <- decay S; m = k.S; delta = beta (v - m); S <- S + k delta; o = q.S, all in-lane.  The
// four warps of a CTA are the four column groups of one (sequence, value head) and share k, q, v, g, beta of a batch
// of 8 tokens staged in shared memory (double buffered with cp.async; one barrier per 8 tokens).
constexpr int kGdnColTokens = 8;

// A column is shared by two adjacent lanes (rows [0, HK/2) and [HK/2, HK)): 256 threads per CTA, HK/2 state floats per
// thread, one shuffle each for m and o per token.
template <int HK>
__global__ void __launch_bounds__(256)
gdn_column_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                  const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state,
                  float *__restrict__ out, int n_tokens, int n_k_heads, int n_v_heads) {
    constexpr int R = HK / 2;
    __shared__ __align__(16) float s_k[2][kGdnColTokens][HK], s_q[2][kGdnColTokens][HK], s_v[2][kGdnColTokens][kGdnHV];
    __shared__ float s_g[2][kGdnColTokens], s_b[2][kGdnColTokens];
    const int b = blockIdx.y, h = blockIdx.x, kh = h / (n_v_heads / n_k_heads);
    const int col = threadIdx.x >> 1, r0 = (threadIdx.x & 1) * R;
    float S[R];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * HK * kGdnHV + static_cast<int64_t>(r0) * kGdnHV + col;
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = sp[i * kGdnHV];

    auto stage = [&](int t0, int buf) {
        const int nt = min(kGdnColTokens, n_tokens - t0);
        // HK/4 16-byte chunks of k and of q per token, 32 chunks of v per token
        for (int i = threadIdx.x; i < nt * (HK / 4); i += 256) {
            const int t = i / (HK / 4), c = i - t * (HK / 4);
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + t;
            const uint32_t dk = static_cast<uint32_t>(__cvta_generic_to_shared(&s_k[buf][t][4 * c]));
            const uint32_t dq = static_cast<uint32_t>(__cvta_generic_to_shared(&s_q[buf][t][4 * c]));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk), "l"(k + (tok * n_k_heads + kh) * HK + 4 * c) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dq), "l"(q + (tok * n_k_heads + kh) * HK + 4 * c) : "memory");
        }
        for (int i = threadIdx.x; i < nt * (kGdnHV / 4); i += 256) {
            const int t = i / (kGdnHV / 4), c = i - t * (kGdnHV / 4);
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + t;
            const uint32_t dv = static_cast<uint32_t>(__cvta_generic_to_shared(&s_v[buf][t][4 * c]));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dv), "l"(v + (tok * n_v_heads + h) * kGdnHV + 4 * c) : "memory");
        }
        if (threadIdx.x < nt) {
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + threadIdx.x;
            s_g[buf][threadIdx.x] = g[tok * n_v_heads + h];
            s_b[buf][threadIdx.x] = beta[tok * n_v_heads + h];
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    for (int t0 = 0, it = 0; t0 < n_tokens; t0 += kGdnColTokens, ++it) {
        const int buf = it & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this batch has landed; everyone is done with the other buffer
        if (t0 + kGdnColTokens < n_tokens) stage(t0 + kGdnColTokens, buf ^ 1);
        const int nt = min(kGdnColTokens, n_tokens - t0);
        for (int t = 0; t < nt; ++t) {
            const float decay = __expf(s_g[buf][t]), bt = s_b[buf][t];
            const float *kt = &s_k[buf][t][r0], *qt = &s_q[buf][t][r0];
            float m0 = 0.0f, m1 = 0.0f, m2 = 0.0f, m3 = 0.0f;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 kk = *reinterpret_cast<const float4 *>(kt + i);  // two addresses per warp: broadcast
                S[i] *= decay; S[i + 1] *= decay; S[i + 2] *= decay; S[i + 3] *= decay;
                m0 = fmaf(kk.x, S[i], m0); m1 = fmaf(kk.y, S[i + 1], m1); m2 = fmaf(kk.z, S[i + 2], m2); m3 = fmaf(kk.w, S[i + 3], m3);
            }
            float m = (m0 + m1) + (m2 + m3);
            m += __shfl_xor_sync(0xffffffffu, m, 1);
            const float d = (s_v[buf][t][col] - m) * bt;
            float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 kk = *reinterpret_cast<const float4 *>(kt + i);
                const float4 qq = *reinterpret_cast<const float4 *>(qt + i);
                S[i] = fmaf(kk.x, d, S[i]); S[i + 1] = fmaf(kk.y, d, S[i + 1]); S[i + 2] = fmaf(kk.z, d, S[i + 2]); S[i + 3] = fmaf(kk.w, d, S[i + 3]);
                o0 = fmaf(qq.x, S[i], o0); o1 = fmaf(qq.y, S[i + 1], o1); o2 = fmaf(qq.z, S[i + 2], o2); o3 = fmaf(qq.w, S[i + 3], o3);
            }
            float o = (o0 + o1) + (o2 + o3);
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            if ((threadIdx.x & 1) == 0) {
                const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + t;
                out[(tok * n_v_heads + h) * kGdnHV + col] = o;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) sp[i * kGdnHV] = S[i];
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
    cudaStream_t s = as_stream(stream);
    if (n_tokens >= 4 && aligned(q, 16) && aligned(k, 16) && aligned(v, 16)) {
        // runs of tokens: one lane per state column, no per-token synchronisation
        dim3 cgrid(n_v_heads, n_seqs);
        prof_begin(s);
        if (head_k_dim == 128) gdn_column_kernel<128><<<cgrid, 256, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
        else gdn_column_kernel<64><<<cgrid, 256, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
        prof_end(s);
        return check_launch("hs_gdn_recurrent");
    }
    dim3 grid(2 * n_v_heads, n_seqs);
    prof_begin(s);
    if (head_k_dim == 128) gdn_recurrent_kernel<128><<<grid, kGdnThreads, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
    else gdn_recurrent_kernel<64><<<grid, kGdnThreads, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
    prof_end(s);
    return check_launch("hs_gdn_recurrent");
}

}  // extern "C"
