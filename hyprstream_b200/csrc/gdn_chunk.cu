// Gated DeltaNet prefill in chunked (WY / UT-transform) form on the tensor cores: chunked_delta_rule
// (architectures/qwen3_5.rs:342-498) re-cut for one CTA per (sequence, value head) with the state in registers.
//
// For a chunk of C tokens with G = cumsum(g), Gamma = exp(G), the rule  S <- e^g S; u = beta (v - S^T k); S <- S + k u^T;
// o = S^T q  is equivalent to (qwen3_5.rs:394-485, same algebra):
//   A'[t][s] = beta_t (k_t.k_s) exp(G_t - G_s), s < t;   T = (I + A')^-1;   U = T (beta V - beta Gamma K S0)
//   o_t = Gamma_t q_t^T S0 + sum_{s<=t} exp(G_t - G_s)(q_t.k_s) u_s;   S = Gamma_C S0 + sum_s exp(G_C - G_s) k_s u_s^T
// (the reference forms W = T (beta Gamma K) and V' = T (beta V) first and U = V' - W S0; applying T last is the same
// product and leaves no per-chunk matrix products outside the tensor cores)
// The reference uses C = 64; the result does not depend on C, and C = 16 keeps the triangular inverse (16 x 16: the
// product (I + M)(I + M^2)(I + M^4)(I + M^8), M = -A', six small MMAs) and the other per-chunk set-up short enough to sit
// in front of every chunk.
//
// Layout: warp w of 8 owns value columns [16w, 16w+16) and keeps S^T[v][k] (16 x 128 fp32) in its mma accumulator
// registers; every S-dependent product of the chunk is warp-local, with the state or U^T as the A operand straight from
// those accumulators (fp32 -> bf16 pairs), mma.sync.m16n8k16 bf16 x bf16 -> fp32:
//   [K S0 | Q S0]^T = S^T . [K | Q]^T     (32 MMAs)      R^T = beta (V^T - Gamma (K S0)^T)      U^T = R^T . T^T   (2 MMAs)
//   O^T = Gamma (Q S0)^T + U^T . P^T      (2 MMAs)       S^T = Gamma_C S^T + (U^T diag(exp(G_C - G))) . K   (16 MMAs)
// The per-chunk set-up that does not depend on S belongs to three more warps: one scans the decay, forms k.k on the tensor
// cores (bf16 k), applies the decay and computes T in its own fragments, one forms q.k and P, one stages the next chunk's
// fp32 inputs (three TMA tensor copies), all while the eight state warps already run the first product.  Gamma and exp(G_C - G) are folded
// into accumulator columns, so the only operand tiles in shared memory are k and q as bf16.  Only MMA operands are rounded
// to bf16; the state and all accumulation stay fp32.
// Bound: latency of the per-chunk dependency chain (3 block barriers); FLOPs are far below the tensor peak.
//
// Accuracy: bf16 operand rounding (2^-9 relative) enters every S-dependent product, so outputs agree with the fp32 rule
// to ~1e-3, inside the path's stated tolerance (max-abs 2e-2, mean-abs 2e-3); hs_gdn_recurrent remains the fp32-exact form.
#include <cuda.h>
#include <cuda_bf16.h>

#include "hs_common.cuh"

namespace hs {

constexpr int kGcC = 16;          // tokens per chunk
constexpr int kGcD = 128;         // head_k_dim = head_v_dim
constexpr int kGcThreads = 352;   // warps 0-7: one 16-column slice of the state each; 8: decay scan, k.k, T; 9: q.k, P; 10: staging
constexpr int kGcRS = kGcD;       // fp32 row stride of the staged inputs (floats): dense, as the tensor copies write them
constexpr int kGcBS = kGcD + 8;   // bf16 row stride of the [16][128] operand tiles
constexpr int kGcPS = kGcC + 8;   // bf16 row stride of P, T and of Kd^T

struct GcSmem {
    __align__(128) float raw[2][3][kGcC][kGcRS];  // k, q, v of a chunk (fp32), double buffered
    float g[2][kGcC], b[2][kGcC];
    float G[kGcC], gam[kGcC], dec[kGcC];  // cumulative log-decay, exp(G), exp(G_C - G)
    __nv_bfloat16 Tb[kGcC][kGcPS];      // (I + A')^-1 (lower)
    __nv_bfloat16 Kb[kGcC][kGcBS], Qb[kGcC][kGcBS];    // k, q
    __nv_bfloat16 P[kGcC][kGcPS];       // (q.k) exp(G_t - G_s), s <= t
    __align__(8) uint64_t full[2];      // mbarriers: the bulk copies of a raw buffer have landed
};

constexpr long long kGcWaitCycles = 4000000000LL;  // ~2 s: bound of the wait on the copies

__device__ __forceinline__ uint32_t gc_s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool gc_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool gc_wait(uint32_t bar, uint32_t parity) {  // bounded
    if (gc_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!gc_try_wait(bar, parity))
        if (clock64() - t0 > kGcWaitCycles) return false;
    return true;
}
// one [16 tokens][128] fp32 box of a 4-D tensor (d, head, token, sequence); tokens past the tensor's end arrive as zeros
__device__ __forceinline__ void gc_tma_box(uint32_t dst, const CUtensorMap *map, int head, int token, int seq, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(0), "r"(head), "r"(token), "r"(seq), "r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t gc_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void gc_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t gc_ld32(const __nv_bfloat16 *p) { return *reinterpret_cast<const uint32_t *>(p); }


__global__ void __launch_bounds__(kGcThreads, 1)
gdn_chunk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state, float *__restrict__ out, int n_tokens, int n_k_heads,
                 int n_v_heads, int *__restrict__ err) {
    extern __shared__ unsigned char gc_smem_raw[];
    GcSmem &sm = *reinterpret_cast<GcSmem *>((reinterpret_cast<uintptr_t>(gc_smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    const int b = blockIdx.y, h = blockIdx.x, kh = h / (n_v_heads / n_k_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, jq = lane & 3;
    const bool chain_warp = warp < 8;
    const int v0 = (warp & 7) * 16;  // a chain warp's value columns

    // S^T accumulators: tile i covers k columns [8i, 8i+8): St[i] = {S^T[v0+gq][8i+2jq], [..+1], S^T[v0+gq+8][8i+2jq], [..+1]}
    float St[16][4];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * kGcD * kGcD;  // [k][v]
    if (chain_warp) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            St[i][0] = sp[(8 * i + 2 * jq) * kGcD + v0 + gq];
            St[i][1] = sp[(8 * i + 2 * jq + 1) * kGcD + v0 + gq];
            St[i][2] = sp[(8 * i + 2 * jq) * kGcD + v0 + gq + 8];
            St[i][3] = sp[(8 * i + 2 * jq + 1) * kGcD + v0 + gq + 8];
        }
    }

    // Staging (warp 10): one lane issues three TMA tensor copies per chunk (the [16 tokens][128] boxes of k, q and v; rows
    // of a head are 512 bytes, strided by the number of heads); they complete on the buffer's mbarrier.  Tokens past the
    // end of the sequence arrive as zeros (beta = 0, g = 0, k = q = v = 0 leave state and outputs untouched).
    // g and beta of a chunk are loaded one stage call ahead (registers gb_g, gb_b), so their global-memory latency is never
    // waited for: stage(c) stores the values fetched during stage(c - 1) and fetches those of chunk c + 1.
    float gb_g = 0.0f, gb_b = 0.0f;
    auto fetch_gates = [&](int c) {
        const int t = c * kGcC + lane;
        const bool in = lane < kGcC && t < n_tokens;
        const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
        gb_g = in ? g[tok * n_v_heads + h] : 0.0f;
        gb_b = in ? beta[tok * n_v_heads + h] : 0.0f;
    };
    auto stage = [&](int c, int buf) {  // called by warp 10 only
        const int t0 = c * kGcC;
        const uint32_t bar = gc_s32(&sm.full[buf]);
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(3u * kGcC * kGcD * 4u) : "memory");
            gc_tma_box(gc_s32(&sm.raw[buf][0][0][0]), &map_k, kh, t0, b, bar);
            gc_tma_box(gc_s32(&sm.raw[buf][1][0][0]), &map_q, kh, t0, b, bar);
            gc_tma_box(gc_s32(&sm.raw[buf][2][0][0]), &map_v, h, t0, b, bar);
        }
        if (lane < kGcC) {
            sm.g[buf][lane] = gb_g;
            sm.b[buf][lane] = gb_b;
        }
        fetch_gates(c + 1);
    };

    const int n_chunks = (n_tokens + kGcC - 1) / kGcC;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gc_s32(&sm.full[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gc_s32(&sm.full[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 10) {
        fetch_gates(0);
        stage(0, 0);
    }
    bool failed = false;
    for (int c = 0; c < n_chunks; ++c) {
        const int buf = c & 1;
        const bool landed = gc_wait(gc_s32(&sm.full[buf]), (c >> 1) & 1);
        // chunk c has landed (and its zero-fill / g / beta stores are visible); every warp is done with the previous chunk's
        // set-up buffers.  A wait that ran out ends the loop for the whole CTA.
        if (!__syncthreads_and(landed)) { failed = true; break; }

        // ---- Pa: k, q -> bf16 (warps 0-7) | cumulative decay (warp 8) ----
        if (chain_warp) {
            const int t = threadIdx.x >> 4, c8 = (threadIdx.x & 15) * 8;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const float4 x0 = *reinterpret_cast<const float4 *>(&sm.raw[buf][which][t][c8]);
                const float4 x1 = *reinterpret_cast<const float4 *>(&sm.raw[buf][which][t][c8 + 4]);
                *reinterpret_cast<uint4 *>(which ? &sm.Qb[t][c8] : &sm.Kb[t][c8]) =
                    make_uint4(gc_pack(x0.x, x0.y), gc_pack(x0.z, x0.w), gc_pack(x1.x, x1.y), gc_pack(x1.z, x1.w));
            }
        } else if (warp == 8) {
            float x = lane < kGcC ? sm.g[buf][lane] : 0.0f;
#pragma unroll
            for (int off = 1; off < kGcC; off <<= 1) {
                const float y = __shfl_up_sync(0xffffffffu, x, off);
                if (lane >= off) x += y;
            }
            const float G_last = __shfl_sync(0xffffffffu, x, kGcC - 1);
            if (lane < kGcC) { sm.G[lane] = x; sm.gam[lane] = __expf(x); sm.dec[lane] = __expf(G_last - x); }
        }
        __syncthreads();
        // ---- C: k.k, decay, T = (I + A')^-1, all in its registers (warp 8) | q.k, decay, P (warp 9) | the next chunk's copies
        //          (warp 10) | [K S0 | Q S0]^T and R^T (warps 0-7) ----
        float X[4][4];
        uint32_t r[4];
        if (warp == 9) {
            // P[t][s] = (q_t . k_s) exp(G_t - G_s), s <= t: tiles nt = columns s in [8nt, 8nt+8), two accumulators each
            float acc[2][2][4];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i >> 3][(i >> 2) & 1][i & 3] = 0.0f;
#pragma unroll
            for (int kk8 = 0; kk8 < 8; ++kk8) {
                const int col = 16 * kk8 + 2 * jq;
                const uint32_t k0 = gc_ld32(&sm.Kb[gq][col]), k1 = gc_ld32(&sm.Kb[gq + 8][col]), k2 = gc_ld32(&sm.Kb[gq][col + 8]), k3 = gc_ld32(&sm.Kb[gq + 8][col + 8]);
                const uint32_t q0 = gc_ld32(&sm.Qb[gq][col]), q1 = gc_ld32(&sm.Qb[gq + 8][col]), q2 = gc_ld32(&sm.Qb[gq][col + 8]), q3 = gc_ld32(&sm.Qb[gq + 8][col + 8]);
                gc_mma(acc[kk8 & 1][0], q0, q1, q2, q3, k0, k2);
                gc_mma(acc[kk8 & 1][1], q0, q1, q2, q3, k1, k3);
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float pv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = gq + 8 * (e >> 1), col = 8 * nt + 2 * jq + (e & 1);
                    pv[e] = col <= row ? (acc[0][nt][e] + acc[1][nt][e]) * __expf(sm.G[row] - sm.G[col]) : 0.0f;
                }
                *reinterpret_cast<uint32_t *>(&sm.P[gq][8 * nt + 2 * jq]) = gc_pack(pv[0], pv[1]);
                *reinterpret_cast<uint32_t *>(&sm.P[gq + 8][8 * nt + 2 * jq]) = gc_pack(pv[2], pv[3]);
            }
        } else if (warp == 10) {
            if (c + 1 < n_chunks) stage(c + 1, buf ^ 1);
        } else if (!chain_warp) {
            // k_t . k_s: tiles nt = columns s in [8nt, 8nt+8); the A fragments of the k rows are the B fragments of the two tiles
            float acc[2][2][4];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i >> 3][(i >> 2) & 1][i & 3] = 0.0f;
#pragma unroll
            for (int kk8 = 0; kk8 < 8; ++kk8) {
                const int col = 16 * kk8 + 2 * jq;
                const uint32_t k0 = gc_ld32(&sm.Kb[gq][col]), k1 = gc_ld32(&sm.Kb[gq + 8][col]), k2 = gc_ld32(&sm.Kb[gq][col + 8]), k3 = gc_ld32(&sm.Kb[gq + 8][col + 8]);
                gc_mma(acc[kk8 & 1][0], k0, k1, k2, k3, k0, k2);
                gc_mma(acc[kk8 & 1][1], k0, k1, k2, k3, k1, k3);
            }
            // (I + A')^-1 = (I + M)(I + M^2)(I + M^4)(I + M^8) with M = -A' (strictly lower 16 x 16, so M^16 = 0): three
            // squarings and three products on the tensor cores, all in this warp's fragments.  m, pm: accumulator layout,
            // tile nt = columns [8nt, 8nt+8): {(row gq, cols 2jq, 2jq+1), (row gq+8, same cols)}.
            float m[2][4], pm[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = gq + 8 * (e >> 1), col = 8 * nt + 2 * jq + (e & 1);
                    m[nt][e] = col < row ? -sm.b[buf][row] * (acc[0][nt][e] + acc[1][nt][e]) * __expf(sm.G[row] - sm.G[col]) : 0.0f;  // -A'
                    pm[nt][e] = m[nt][e] + (row == col ? 1.0f : 0.0f);
                }
            // A-form of a 16 x 16 matrix held in accumulator layout: its four 8 x 8 blocks as bf16 pairs; the B-form of the
            // same matrix is each block transposed across the warp
            auto a_form = [&](const float (&x)[2][4], uint32_t (&a)[4]) {
                a[0] = gc_pack(x[0][0], x[0][1]); a[1] = gc_pack(x[0][2], x[0][3]); a[2] = gc_pack(x[1][0], x[1][1]); a[3] = gc_pack(x[1][2], x[1][3]);
            };
            auto b_form = [&](const uint32_t (&a)[4], uint32_t (&bf)[4]) {
#pragma unroll
                for (int i = 0; i < 4; ++i) asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(bf[i]) : "r"(a[i]));
            };
            uint32_t ma[4], mb[4], pa[4];
            a_form(m, ma);
            b_form(ma, mb);
#pragma unroll
            for (int step = 0; step < 3; ++step) {
                // m <- m . m: the B operand of column tile nt is the blocks (rows 0-7, nt), (rows 8-15, nt) transposed
                float m2[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    m2[nt][0] = m2[nt][1] = m2[nt][2] = m2[nt][3] = 0.0f;
                    gc_mma(m2[nt], ma[0], ma[1], ma[2], ma[3], mb[2 * nt], mb[2 * nt + 1]);
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) m[nt][e] = m2[nt][e];
                a_form(m, ma);
                b_form(ma, mb);
                // pm <- pm + pm . m
                a_form(pm, pa);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) gc_mma(pm[nt], pa[0], pa[1], pa[2], pa[3], mb[2 * nt], mb[2 * nt + 1]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                *reinterpret_cast<uint32_t *>(&sm.Tb[gq][8 * nt + 2 * jq]) = gc_pack(pm[nt][0], pm[nt][1]);
                *reinterpret_cast<uint32_t *>(&sm.Tb[gq + 8][8 * nt + 2 * jq]) = gc_pack(pm[nt][2], pm[nt][3]);
            }
        } else {
            // rows = this warp's 16 value columns, columns = 16 tokens of k then 16 tokens of q
#pragma unroll
            for (int n = 0; n < 4; ++n) X[n][0] = X[n][1] = X[n][2] = X[n][3] = 0.0f;
#pragma unroll
            for (int kk8 = 0; kk8 < 8; ++kk8) {
                const uint32_t a0 = gc_pack(St[2 * kk8][0], St[2 * kk8][1]), a1 = gc_pack(St[2 * kk8][2], St[2 * kk8][3]);
                const uint32_t a2 = gc_pack(St[2 * kk8 + 1][0], St[2 * kk8 + 1][1]), a3 = gc_pack(St[2 * kk8 + 1][2], St[2 * kk8 + 1][3]);
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const __nv_bfloat16 *row = n < 2 ? &sm.Kb[8 * n + gq][0] : &sm.Qb[8 * (n - 2) + gq][0];
                    gc_mma(X[n], a0, a1, a2, a3, gc_ld32(row + 16 * kk8 + 2 * jq), gc_ld32(row + 16 * kk8 + 2 * jq + 8));
                }
            }
            // R^T = beta (V^T - Gamma (K S0)^T) in the accumulator layout = the A operand (k = tokens) of U^T = R^T . T^T;
            // (Gamma Q S0)^T = (Q S0)^T scaled per token column
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int s0 = 8 * n + 2 * jq;
                const float b0 = sm.b[buf][s0], b1 = sm.b[buf][s0 + 1], g0 = sm.gam[s0], g1 = sm.gam[s0 + 1];
                const float r00 = b0 * (sm.raw[buf][2][s0][v0 + gq] - g0 * X[n][0]), r01 = b1 * (sm.raw[buf][2][s0 + 1][v0 + gq] - g1 * X[n][1]);
                const float r10 = b0 * (sm.raw[buf][2][s0][v0 + gq + 8] - g0 * X[n][2]), r11 = b1 * (sm.raw[buf][2][s0 + 1][v0 + gq + 8] - g1 * X[n][3]);
                r[2 * n] = gc_pack(r00, r01);
                r[2 * n + 1] = gc_pack(r10, r11);
                X[2 + n][0] *= g0; X[2 + n][1] *= g1; X[2 + n][2] *= g0; X[2 + n][3] *= g1;
            }
        }
        __syncthreads();  // T and P are ready
        if (chain_warp) {
            // ---- D: U^T = R^T . T^T; O^T = (Gamma Q S0)^T + U^T . P^T; S^T = Gamma_C S^T + (U^T diag(exp(G_C - G))) . K ----
            float U[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                U[n][0] = U[n][1] = U[n][2] = U[n][3] = 0.0f;
                gc_mma(U[n], r[0], r[1], r[2], r[3], gc_ld32(&sm.Tb[8 * n + gq][2 * jq]), gc_ld32(&sm.Tb[8 * n + gq][2 * jq + 8]));
            }
            const uint32_t u0 = gc_pack(U[0][0], U[0][1]), u1 = gc_pack(U[0][2], U[0][3]), u2 = gc_pack(U[1][0], U[1][1]), u3 = gc_pack(U[1][2], U[1][3]);
#pragma unroll
            for (int n = 0; n < 2; ++n)
                gc_mma(X[2 + n], u0, u1, u2, u3, gc_ld32(&sm.P[8 * n + gq][2 * jq]), gc_ld32(&sm.P[8 * n + gq][2 * jq + 8]));
            // token columns of U scaled by exp(G_C - G_s); k itself is the B operand, its 8 x 8 blocks transposed on load
            const float d00 = sm.dec[2 * jq], d01 = sm.dec[2 * jq + 1], d10 = sm.dec[8 + 2 * jq], d11 = sm.dec[8 + 2 * jq + 1];
            const uint32_t w0 = gc_pack(U[0][0] * d00, U[0][1] * d01), w1 = gc_pack(U[0][2] * d00, U[0][3] * d01);
            const uint32_t w2 = gc_pack(U[1][0] * d10, U[1][1] * d11), w3 = gc_pack(U[1][2] * d10, U[1][3] * d11);
            const float gC = sm.gam[kGcC - 1];
            // lane -> row address of ldmatrix.x4.trans: matrix (lane >> 3): rows s = (lane & 7) + 8 (matrix & 1), column block + (matrix >> 1)
            const uint32_t kb_lane = gc_s32(&sm.Kb[(lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(kb_lane + 16u * i));
                St[i][0] *= gC; St[i][1] *= gC; St[i][2] *= gC; St[i][3] *= gC;
                gc_mma(St[i], w0, w1, w2, w3, b0, b1);
                St[i + 1][0] *= gC; St[i + 1][1] *= gC; St[i + 1][2] *= gC; St[i + 1][3] *= gC;
                gc_mma(St[i + 1], w0, w1, w2, w3, b2, b3);
            }
            // outputs: X[2 + n] = O^T rows v0+gq (+8), tokens 8n + 2jq (+1)
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int t = c * kGcC + 8 * n + 2 * jq + e;
                    if (t < n_tokens) {
                        float *op = out + ((static_cast<int64_t>(b) * n_tokens + t) * n_v_heads + h) * kGcD + v0 + gq;
                        op[0] = X[2 + n][e];
                        op[8] = X[2 + n][2 + e];
                    }
                }
        }
    }
    if (failed) {
        if (threadIdx.x == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        return;  // the state is left as it was
    }
    if (chain_warp) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            sp[(8 * i + 2 * jq) * kGcD + v0 + gq] = St[i][0];
            sp[(8 * i + 2 * jq + 1) * kGcD + v0 + gq] = St[i][1];
            sp[(8 * i + 2 * jq) * kGcD + v0 + gq + 8] = St[i][2];
            sp[(8 * i + 2 * jq + 1) * kGcD + v0 + gq + 8] = St[i][3];
        }
    }
}

}  // namespace hs

namespace hs {

typedef CUresult (*GcEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static GcEncodeTiledFn gc_encode_fn() {
    static GcEncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<GcEncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// [n_seqs, n_tokens, n_heads, 128] fp32 -> 4-D map (d, head, token, sequence), box 128 x 1 x 16 x 1, no swizzle
static bool gc_make_map(CUtensorMap *map, const float *base, int n_seqs, int n_tokens, int n_heads) {
    GcEncodeTiledFn fn = gc_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {kGcD, static_cast<cuuint64_t>(n_heads), static_cast<cuuint64_t>(n_tokens), static_cast<cuuint64_t>(n_seqs)};
    const cuuint64_t strides[3] = {kGcD * 4ull, static_cast<cuuint64_t>(n_heads) * kGcD * 4ull,
                                   static_cast<cuuint64_t>(n_tokens) * n_heads * kGcD * 4ull};
    const cuuint32_t box[4] = {kGcD, 1, kGcC, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_gdn_chunk_prefill(const float *q, const float *k, const float *v, const float *g, const float *beta, float *state,
                             float *out, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                             int32_t head_v_dim, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_seqs < 0 || n_tokens < 0 || n_k_heads <= 0 || n_v_heads <= 0) return fail(HS_ERR_ARG, "hs_gdn_chunk_prefill: bad sizes");
    if (n_v_heads % n_k_heads != 0) return fail(HS_ERR_ARG, "hs_gdn_chunk_prefill: n_v_heads %d not a multiple of n_k_heads %d", n_v_heads, n_k_heads);
    if (head_k_dim != kGcD || head_v_dim != kGcD)
        return fail(HS_ERR_UNSUPPORTED, "hs_gdn_chunk_prefill: head dims %d x %d (supported: 128 x 128; use hs_gdn_recurrent)", head_k_dim, head_v_dim);
    if (n_seqs == 0 || n_tokens == 0) return HS_OK;
    if (!q || !k || !v || !g || !beta || !state || !out) return fail(HS_ERR_ARG, "hs_gdn_chunk_prefill: NULL pointer");
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(state, 4) || !aligned(out, 4))
        return fail(HS_ERR_ARG, "hs_gdn_chunk_prefill: q, k, v must be 16-byte aligned");
    if (n_seqs > 65535) return fail(HS_ERR_UNSUPPORTED, "hs_gdn_chunk_prefill: more than 65535 sequences");
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "hs_gdn_chunk_prefill: device error word unavailable");
    CUtensorMap mq, mk, mv;
    if (!gc_make_map(&mq, q, n_seqs, n_tokens, n_k_heads) || !gc_make_map(&mk, k, n_seqs, n_tokens, n_k_heads) ||
        !gc_make_map(&mv, v, n_seqs, n_tokens, n_v_heads))
        return fail(HS_ERR_UNSUPPORTED, "hs_gdn_chunk_prefill: the driver refused the tensor maps (use hs_gdn_recurrent)");
    static PerDeviceState configured;
    const int dev = current_device();
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(GcSmem) + 128));
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_gdn_chunk_prefill: %s", cudaGetErrorString(e));
        configured.set(dev, 1);
    }
    cudaStream_t s = as_stream(stream);
    dim3 grid(n_v_heads, n_seqs);
    prof_begin(s);
    gdn_chunk_kernel<<<grid, kGcThreads, sizeof(GcSmem) + 128, s>>>(mq, mk, mv, g, beta, state, out, n_tokens, n_k_heads, n_v_heads, err);
    prof_end(s);
    return check_launch("hs_gdn_chunk_prefill");
}

}  // extern "C"
