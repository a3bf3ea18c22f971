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

// ---- register-tile form for runs of tokens ---------------------------------------------------------------------
// The rule is independent per value column: m[v], delta[v], S[:,v] and o[v] never mix columns.  One CTA of 8 warps owns a
// whole (sequence, value head) state; warp w owns value columns [16w, 16w+16) and a thread an (HK/RG rows) x (CPT columns)
// tile of the state in registers (head_k_dim 128: 32 x 2), row pairs packed for the two-wide fp32 FMA (which saves issue
// slots; the fp32 rate itself, ~125 FMA per clock per SM measured, is the same packed or not).  Per token a thread reads
// its rows of k and q (shared memory, rows of a group padded so that the groups of a warp hit distinct banks) and its
// values of v, and the RG row groups of a column add their partial k.S and q.S with log2(RG) shuffle rounds; no barrier.
// k, q, v, g, beta of 8 tokens are staged per barrier (cp.async, double buffered).
//
// The decay is carried as a scalar: with G the product of the decays since the last renormalisation and S^ = S / G,
//   m = G (k.S^);  delta = beta (v - m);  S^ <- S^ + k (delta / G);  o = G (q.S^)
// which is the reference's S <- exp(g) S; m = k.S; S <- S + k delta; o = q.S with one multiply-add per state element
// less.  S^ is multiplied back (S = G S^, G = 1) every 8 tokens and whenever G would drop below 2^-60; a single
// decay below that is applied to the state directly.
constexpr int kGdnColTokens = 8;

__device__ __forceinline__ uint64_t gdn_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void gdn_unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t gdn_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t gdn_mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// RG: row groups (lanes of a warp that share a column), CPT: columns per thread; a warp covers (32 / RG) * CPT columns and
// the CTA has as many warps as cover the 128 columns.
template <int HK, int RG, int CPT>
__global__ void __launch_bounds__(32 * 128 / ((32 / RG) * CPT))
gdn_tile_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state,
                float *__restrict__ out, int n_tokens, int n_k_heads, int n_v_heads) {
    static_assert(CPT == 2 || CPT == 4, "columns are moved in pairs");
    constexpr int WC = (32 / RG) * CPT;        // columns per warp
    constexpr int NT = 32 * kGdnHV / WC;       // threads per CTA
    constexpr int R = HK / RG;       // rows per thread
    constexpr int RP = R / 2;        // row pairs per thread
    constexpr int GS = R + 4;        // padded stride of a row group in shared memory (floats): the groups hit distinct banks
    __shared__ __align__(16) float s_k[2][kGdnColTokens][RG * GS], s_q[2][kGdnColTokens][RG * GS], s_v[2][kGdnColTokens][kGdnHV];
    __shared__ float s_g[2][kGdnColTokens], s_b[2][kGdnColTokens];
    const int b = blockIdx.y, h = blockIdx.x, kh = h / (n_v_heads / n_k_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = lane / (32 / RG), cg = lane % (32 / RG);
    const int r0 = rg * R, c0 = warp * WC + cg * CPT;
    // S2[p][c] = (S[r0 + 2p][c0 + c], S[r0 + 2p + 1][c0 + c])
    uint64_t S2[RP][CPT];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * HK * kGdnHV + static_cast<int64_t>(r0) * kGdnHV + c0;
#pragma unroll
    for (int p = 0; p < RP; ++p)
#pragma unroll
        for (int c = 0; c < CPT; c += 2) {
            const float2 a = *reinterpret_cast<const float2 *>(sp + (2 * p) * kGdnHV + c), e = *reinterpret_cast<const float2 *>(sp + (2 * p + 1) * kGdnHV + c);
            S2[p][c] = gdn_pack2(a.x, e.x);
            S2[p][c + 1] = gdn_pack2(a.y, e.y);
        }

    auto stage = [&](int t0, int buf) {
        const int nt = min(kGdnColTokens, n_tokens - t0);
        // HK/4 16-byte chunks of k and of q per token (chunk c lands in row group c / (R/4)), 32 chunks of v per token
        for (int i = threadIdx.x; i < nt * (HK / 4); i += NT) {
            const int t = i / (HK / 4), c = i - t * (HK / 4);
            const int dst = (c / (R / 4)) * GS + (c % (R / 4)) * 4;
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + t;
            const uint32_t dk = static_cast<uint32_t>(__cvta_generic_to_shared(&s_k[buf][t][dst]));
            const uint32_t dq = static_cast<uint32_t>(__cvta_generic_to_shared(&s_q[buf][t][dst]));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk), "l"(k + (tok * n_k_heads + kh) * HK + 4 * c) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dq), "l"(q + (tok * n_k_heads + kh) * HK + 4 * c) : "memory");
        }
        for (int i = threadIdx.x; i < nt * (kGdnHV / 4); i += NT) {
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
    auto renormalise = [&](float f) {
        const uint64_t f2 = gdn_pack2(f, f);
#pragma unroll
        for (int p = 0; p < RP; ++p)
#pragma unroll
            for (int c = 0; c < CPT; ++c) S2[p][c] = gdn_mul2(S2[p][c], f2);
    };
    constexpr float kTiny = 8.673617379884035e-19f;  // 2^-60
    float G = 1.0f;  // product of the decays since the state was last multiplied back
    stage(0, 0);
    for (int t0 = 0, it = 0; t0 < n_tokens; t0 += kGdnColTokens, ++it) {
        const int buf = it & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // this batch has landed; everyone is done with the other buffer
        if (t0 + kGdnColTokens < n_tokens) stage(t0 + kGdnColTokens, buf ^ 1);
        const int nt = min(kGdnColTokens, n_tokens - t0);
        for (int t = 0; t < nt; ++t) {
            const float decay = __expf(s_g[buf][t]), bt = s_b[buf][t];
            if (G * decay < kTiny) {  // (uniform over the CTA)
                renormalise(G);
                G = 1.0f;
                if (decay < kTiny) renormalise(decay); else G = decay;
            } else {
                G *= decay;
            }
            const float *kt = &s_k[buf][t][rg * GS], *qt = &s_q[buf][t][rg * GS];
            uint64_t k2[RP], m2[2][CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) m2[0][c] = m2[1][c] = 0ull;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const ulonglong2 kk = *reinterpret_cast<const ulonglong2 *>(kt + 4 * i);  // rows 4i, 4i+1 | 4i+2, 4i+3
                k2[2 * i] = kk.x;
                k2[2 * i + 1] = kk.y;
            }
#pragma unroll
            for (int p = 0; p < RP; ++p)
#pragma unroll
                for (int c = 0; c < CPT; ++c) m2[p & 1][c] = gdn_fma2(k2[p], S2[p][c], m2[p & 1][c]);
            float m[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float a0, a1, b0, b1;
                gdn_unpack2(m2[0][c], a0, a1);
                gdn_unpack2(m2[1][c], b0, b1);
                m[c] = (a0 + a1) + (b0 + b1);
            }
#pragma unroll
            for (int off = 32 / RG; off < 32; off <<= 1)
#pragma unroll
                for (int c = 0; c < CPT; ++c) m[c] += __shfl_xor_sync(0xffffffffu, m[c], off);
            float vin[CPT];
#pragma unroll
            for (int c = 0; c < CPT; c += 2) {
                const float2 vv = *reinterpret_cast<const float2 *>(&s_v[buf][t][c0 + c]);
                vin[c] = vv.x;
                vin[c + 1] = vv.y;
            }
            const float invG = 1.0f / G;
            uint64_t d2[CPT], o2[2][CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float d = (vin[c] - G * m[c]) * bt * invG;  // delta / G
                d2[c] = gdn_pack2(d, d);
                o2[0][c] = o2[1][c] = 0ull;
            }
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const ulonglong2 qq = *reinterpret_cast<const ulonglong2 *>(qt + 4 * i);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    S2[2 * i][c] = gdn_fma2(k2[2 * i], d2[c], S2[2 * i][c]);
                    o2[0][c] = gdn_fma2(qq.x, S2[2 * i][c], o2[0][c]);
                    S2[2 * i + 1][c] = gdn_fma2(k2[2 * i + 1], d2[c], S2[2 * i + 1][c]);
                    o2[1][c] = gdn_fma2(qq.y, S2[2 * i + 1][c], o2[1][c]);
                }
            }
            float o[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float a0, a1, b0, b1;
                gdn_unpack2(o2[0][c], a0, a1);
                gdn_unpack2(o2[1][c], b0, b1);
                o[c] = (a0 + a1) + (b0 + b1);
            }
#pragma unroll
            for (int off = 32 / RG; off < 32; off <<= 1)
#pragma unroll
                for (int c = 0; c < CPT; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], off);
            if (rg == 0) {
                const int64_t tok = static_cast<int64_t>(b) * n_tokens + t0 + t;
                float *op = out + (tok * n_v_heads + h) * kGdnHV + c0;
#pragma unroll
                for (int c = 0; c < CPT; c += 2) *reinterpret_cast<float2 *>(op + c) = make_float2(o[c] * G, o[c + 1] * G);
            }
        }
        renormalise(G);  // back to the true state at the end of every batch
        G = 1.0f;
    }
#pragma unroll
    for (int p = 0; p < RP; ++p)
#pragma unroll
        for (int c = 0; c < CPT; c += 2) {
            float a0, e0, a1, e1;
            gdn_unpack2(S2[p][c], a0, e0);
            gdn_unpack2(S2[p][c + 1], a1, e1);
            *reinterpret_cast<float2 *>(sp + (2 * p) * kGdnHV + c) = make_float2(a0, a1);
            *reinterpret_cast<float2 *>(sp + (2 * p + 1) * kGdnHV + c) = make_float2(e0, e1);
        }
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
        // runs of tokens: the whole state of a (sequence, head) in one CTA's registers, no per-token barrier
        dim3 cgrid(n_v_heads, n_seqs);
        prof_begin(s);
        if (head_k_dim == 128) gdn_tile_kernel<128, 4, 2><<<cgrid, 256, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
        else gdn_tile_kernel<64, 8, 4><<<cgrid, 256, 0, s>>>(q, k, v, g, beta, state, out, n_tokens, n_k_heads, n_v_heads);
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
