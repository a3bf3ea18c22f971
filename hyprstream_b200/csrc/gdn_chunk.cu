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
// Layout: four state warps, one per scheduler; warp w owns value columns [32w, 32w+32) as two 16-row MMA tiles and keeps
// S^T[v][k] (32 x 128 fp32, 128 registers a thread) in its mma accumulators.  Every S-dependent product of the chunk is
// warp-local, with the state or U^T as the A operand straight from those accumulators (fp32 -> bf16 pairs) and every B operand
// shared by the warp's two tiles, mma.sync.m16n8k16 bf16 x bf16 -> fp32, per warp and chunk:
//   [K S0 | Q S0]^T = S^T . [K | Q]^T     (64 MMAs)      R^T = beta (V^T - Gamma (K S0)^T)      U^T = R^T . T^T   (4 MMAs)
//   O^T = Gamma (Q S0)^T + U^T . P^T      (4 MMAs)       S^T = Gamma_C S^T + (U^T diag(exp(G_C - G))) . K   (32 MMAs)
// The per-chunk set-up that does not depend on S runs ahead of the state warps in a ring of chunk slots: a staging warp issues
// each chunk's three TMA tensor copies (k, q, v boxes of [16 tokens][128]; fp32 from the boundary, bf16 from the layer entry's
// own prologue) as soon as the slot's previous chunk is done with; three set-up warps take a whole chunk each, round-robin (k, q
// to bf16 tiles, the decay scan, k.k and q.k on the tensor cores, T in the warp's own fragments, P), and hand the slot to the
// state warps through an mbarrier.  The state warps never meet a block barrier: each waits for the slot, runs its products and
// signals the slot free.  Eight warps in all: two per scheduler, so that a state warp can have its ~250 registers.  Gamma and
// exp(G_C - G) are folded into accumulator columns, so the only operand tiles in shared memory are k and q as bf16.  Only MMA
// operands are rounded to bf16; the state and all accumulation stay fp32.
// Bound: the state warps' own chain, ~2,000 cycles per chunk.  Measured on this part: mma.sync.m16n8k16 issues at one per ~5 cycles
// and scheduler when its A registers repeat (21 cycles dependent), one per ~9.4 when every MMA brings fresh A registers - as the
// state does, whether they are packed by cvt.rn.bf16x2 or by a single byte permute - so the first product alone (64 MMAs) is
// ~600 cycles and the chunk's 115 MMAs per scheduler ~1,050; HBM traffic and FLOPs are far below their peaks.
// Tried and measured slower: RMSNormGated fused in through writer warps (twelve warps with setmaxnreg: the extra warps take
// issue slots from the state warps, 14.4 -> 16.7 ms for three layers).
//
// Accuracy: bf16 operand rounding (2^-9 relative) enters every S-dependent product, so outputs agree with the fp32 rule
// to ~1e-3, inside the path's stated tolerance (max-abs 2e-2, mean-abs 2e-3); hs_gdn_recurrent remains the fp32-exact form.
#include <cuda.h>
#include <cuda_bf16.h>

#include "hs_common.cuh"

namespace hs {

constexpr int kGcC = 16;          // tokens per chunk
constexpr int kGcD = 128;         // head_k_dim = head_v_dim
constexpr int kGcChain = 4;       // warps 0-3: a 32-column slice of the state each, one warp per scheduler
// set-up warps (after the state warps): the S-independent set-up of a chunk, a whole chunk per warp, chunks dealt round-robin; then one
// staging warp.  Whole-head CTAs (MT = 2): three, eight warps in all - two per scheduler, so that a state warp may hold its 128 state
// registers.  Half-head CTAs (MT = 1): the state warps' chain is shorter and they need fewer registers: six set-up warps keep up.
template <int MT> constexpr int gc_prep() { return MT == 2 ? 3 : 6; }
template <int MT> constexpr int gc_threads() { return (kGcChain + gc_prep<MT>() + 1) * 32; }
// chunks in flight between the copies and the state warps: what fits beside fp32 (bf16) inputs
template <typename TIn> constexpr int gc_slots() { return sizeof(TIn) == 4 ? 6 : 9; }
constexpr int kGcRS = kGcD;       // fp32 row stride of the staged inputs (floats): dense, as the tensor copies write them
constexpr int kGcBS = kGcD + 8;   // bf16 row stride of the [16][128] operand tiles
constexpr int kGcPS = kGcC + 8;   // bf16 row stride of P, T and of Kd^T

template <typename TIn>
struct GcSlot {
    __align__(128) TIn raw[3][kGcC][kGcRS];             // k, q, v of the chunk, as the tensor copies deliver them
    __nv_bfloat16 Kb[kGcC][kGcBS], Qb[kGcC][kGcBS];     // k, q
    __nv_bfloat16 Tb[kGcC][kGcPS];                      // (I + A')^-1 (lower)
    __nv_bfloat16 P[kGcC][kGcPS];                       // (q.k) exp(G_t - G_s), s <= t
    float g[kGcC], b[kGcC];
    float G[kGcC], gam[kGcC], dec[kGcC];                // cumulative log-decay, exp(G), exp(G_C - G)
};
template <typename TIn>
struct GcSmem {
    GcSlot<TIn> slot[gc_slots<TIn>()];
    __align__(8) uint64_t full[gc_slots<TIn>()];   // the tensor copies (and g, beta) of the slot's chunk have landed
    uint64_t ready[gc_slots<TIn>()];               // its set-up (Kb, Qb, T, P, decays) is complete
    uint64_t done[gc_slots<TIn>()];                // all state warps are through with it
    int abort;                                     // a wait ran out somewhere in the CTA
};
static_assert(sizeof(GcSmem<float>) + 128 <= 227 * 1024 && sizeof(GcSmem<__nv_bfloat16>) + 128 <= 227 * 1024, "one CTA's shared memory");

constexpr long long kGcWaitCycles = 4000000000LL;  // ~2 s: bound of every wait

__device__ __forceinline__ uint32_t gc_s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool gc_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded; a wait that runs out raises the CTA's abort flag, which ends every other wait of the CTA at once
// (the helper warps sleep `nap` ns between polls so that their waiting takes no issue slots from the state warp of their scheduler)
__device__ __forceinline__ bool gc_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned nap = 0) {
    if (gc_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!gc_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > kGcWaitCycles) { *abort_flag = 1; return false; }
        if (nap) __nanosleep(nap);
    }
    return true;
}
constexpr unsigned kGcNap = 200;
__device__ __forceinline__ void gc_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ float gc_f32(float x) { return x; }
__device__ __forceinline__ float gc_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ uint32_t gc_ld32(const __nv_bfloat16 *p) { return *reinterpret_cast<const uint32_t *>(p); }


// MT: 16-row MMA tiles per state warp.  2: a CTA holds a whole head (4 warps x 32 value columns).  1: a head is cut over two
// CTAs of 64 columns (4 warps x 16): each repeats the set-up, and the state warps' chain per chunk is about half as long - for
// launches that would leave more than half of the SMs idle (few sequences, or a head group per GPU).
template <typename TIn, int MT>
__global__ void __launch_bounds__(gc_threads<MT>(), 1)
gdn_chunk_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const float *__restrict__ g, const float *__restrict__ beta, float *__restrict__ state, float *__restrict__ out, int n_tokens, int n_k_heads,
                 int n_v_heads, int *__restrict__ err) {
    extern __shared__ unsigned char gc_smem_raw[];
    constexpr int kGcSlots = gc_slots<TIn>();
    using Slot = GcSlot<TIn>;
    GcSmem<TIn> &sm = *reinterpret_cast<GcSmem<TIn> *>((reinterpret_cast<uintptr_t>(gc_smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    const int b = blockIdx.y, h = blockIdx.x / (2 / MT), kh = h / (n_v_heads / n_k_heads);
    const int col0 = (blockIdx.x % (2 / MT)) * 64;  // first value column of this CTA
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, jq = lane & 3;
    const int n_chunks = (n_tokens + kGcC - 1) / kGcC;
    volatile int *abort_flag = &sm.abort;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kGcSlots; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gc_s32(&sm.full[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gc_s32(&sm.ready[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gc_s32(&sm.done[i])), "r"(kGcChain));
        }
        sm.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    constexpr int kGcPrep = gc_prep<MT>();
    if (warp == kGcChain + kGcPrep) {
        // ================================ staging (one warp) ================================
        // Chunk c goes into slot c mod kGcSlots once the state warps are through with the chunk that used the slot before: one
        // lane issues three TMA tensor copies (the [16 tokens][128] boxes of k, q and v; rows of a head are 512 bytes, strided by
        // the number of heads); they complete on the slot's `full` barrier.  Tokens past the end of the sequence arrive as zeros
        // (beta = 0, g = 0, k = q = v = 0 leave state and outputs untouched).  g and beta of a chunk are loaded one chunk ahead
        // (registers), so their global-memory latency is never waited for.
        float gb_g = 0.0f, gb_b = 0.0f;
        auto fetch_gates = [&](int c) {
            const int t = c * kGcC + lane;
            const bool in = lane < kGcC && c < n_chunks && t < n_tokens;
            const int64_t tok = static_cast<int64_t>(b) * n_tokens + t;
            gb_g = in ? g[tok * n_v_heads + h] : 0.0f;
            gb_b = in ? beta[tok * n_v_heads + h] : 0.0f;
        };
        fetch_gates(0);
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c % kGcSlots, use = c / kGcSlots;
            Slot &sl = sm.slot[s];
            if (use > 0 && !gc_wait(gc_s32(&sm.done[s]), (use - 1) & 1, abort_flag, kGcNap)) break;
            if (lane < kGcC) {
                sl.g[lane] = gb_g;
                sl.b[lane] = gb_b;
            }
            __syncwarp();
            if (lane == 0) {
                const uint32_t bar = gc_s32(&sm.full[s]);
                const int t0 = c * kGcC;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(3u * kGcC * kGcD * static_cast<uint32_t>(sizeof(TIn))) : "memory");
                gc_tma_box(gc_s32(&sl.raw[0][0][0]), &map_k, kh, t0, b, bar);
                gc_tma_box(gc_s32(&sl.raw[1][0][0]), &map_q, kh, t0, b, bar);
                gc_tma_box(gc_s32(&sl.raw[2][0][0]), &map_v, h, t0, b, bar);
            }
            fetch_gates(c + 1);
        }
        // (every copy issued is waited for by a set-up warp, or the CTA has given up: then a bounded pause lets them land)
        if (*abort_flag) {
            const long long t0c = clock64();
            while (clock64() - t0c < 2000000LL) {}
            if (lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        }
        return;
    }

    if (warp >= kGcChain) {
        // ================================ set-up (three warps, a whole chunk each) ================================
        // Everything of a chunk that does not depend on the state: k, q -> bf16; the cumulative decay; k.k on the tensor cores,
        // the decay applied, T = (I + A')^-1 in the warp's own fragments; q.k, the decay applied, P.  Warp p takes chunks
        // p, p + 3, ...: the warps never talk to each other, and the state warps never wait for any of this unless all three
        // fall behind.
        for (int c = warp - kGcChain; c < n_chunks; c += kGcPrep) {
            const int s = c % kGcSlots, use = c / kGcSlots;
            Slot &sl = sm.slot[s];
            if (!gc_wait(gc_s32(&sm.full[s]), use & 1, abort_flag, kGcNap)) break;
            // ---- k, q -> bf16 ----
#pragma unroll
            for (int which = 0; which < 2; ++which)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int idx = i * 32 + lane, t = idx >> 4, c8 = (idx & 15) * 8;
                    uint4 packed;
                    if constexpr (sizeof(TIn) == 4) {
                        const float4 x0 = *reinterpret_cast<const float4 *>(&sl.raw[which][t][c8]);
                        const float4 x1 = *reinterpret_cast<const float4 *>(&sl.raw[which][t][c8 + 4]);
                        packed = make_uint4(gc_pack(x0.x, x0.y), gc_pack(x0.z, x0.w), gc_pack(x1.x, x1.y), gc_pack(x1.z, x1.w));
                    } else {
                        packed = *reinterpret_cast<const uint4 *>(&sl.raw[which][t][c8]);  // already bf16: into the padded rows
                    }
                    *reinterpret_cast<uint4 *>(which ? &sl.Qb[t][c8] : &sl.Kb[t][c8]) = packed;
                }
            // ---- cumulative decay ----
            {
                float x = lane < kGcC ? sl.g[lane] : 0.0f;
#pragma unroll
                for (int off = 1; off < kGcC; off <<= 1) {
                    const float y = __shfl_up_sync(0xffffffffu, x, off);
                    if (lane >= off) x += y;
                }
                const float G_last = __shfl_sync(0xffffffffu, x, kGcC - 1);
                if (lane < kGcC) { sl.G[lane] = x; sl.gam[lane] = __expf(x); sl.dec[lane] = __expf(G_last - x); }
            }
            __syncwarp();
            // ---- k_t . k_s and q_t . k_s: tiles nt = columns s in [8nt, 8nt+8), two accumulators each; the A fragments of the k
            //      rows are the B fragments of the two tiles ----
            float acc[2][2][4], acq[2][2][4];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i >> 3][(i >> 2) & 1][i & 3] = acq[i >> 3][(i >> 2) & 1][i & 3] = 0.0f;
#pragma unroll
            for (int kk8 = 0; kk8 < 8; ++kk8) {
                const int col = 16 * kk8 + 2 * jq;
                const uint32_t k0 = gc_ld32(&sl.Kb[gq][col]), k1 = gc_ld32(&sl.Kb[gq + 8][col]), k2 = gc_ld32(&sl.Kb[gq][col + 8]), k3 = gc_ld32(&sl.Kb[gq + 8][col + 8]);
                const uint32_t q0 = gc_ld32(&sl.Qb[gq][col]), q1 = gc_ld32(&sl.Qb[gq + 8][col]), q2 = gc_ld32(&sl.Qb[gq][col + 8]), q3 = gc_ld32(&sl.Qb[gq + 8][col + 8]);
                gc_mma(acc[kk8 & 1][0], k0, k1, k2, k3, k0, k2);
                gc_mma(acc[kk8 & 1][1], k0, k1, k2, k3, k1, k3);
                gc_mma(acq[kk8 & 1][0], q0, q1, q2, q3, k0, k2);
                gc_mma(acq[kk8 & 1][1], q0, q1, q2, q3, k1, k3);
            }
            // P[t][s] = (q_t . k_s) exp(G_t - G_s), s <= t
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                float pv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = gq + 8 * (e >> 1), col = 8 * nt + 2 * jq + (e & 1);
                    pv[e] = col <= row ? (acq[0][nt][e] + acq[1][nt][e]) * __expf(sl.G[row] - sl.G[col]) : 0.0f;
                }
                *reinterpret_cast<uint32_t *>(&sl.P[gq][8 * nt + 2 * jq]) = gc_pack(pv[0], pv[1]);
                *reinterpret_cast<uint32_t *>(&sl.P[gq + 8][8 * nt + 2 * jq]) = gc_pack(pv[2], pv[3]);
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
                    m[nt][e] = col < row ? -sl.b[row] * (acc[0][nt][e] + acc[1][nt][e]) * __expf(sl.G[row] - sl.G[col]) : 0.0f;  // -A'
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
                *reinterpret_cast<uint32_t *>(&sl.Tb[gq][8 * nt + 2 * jq]) = gc_pack(pm[nt][0], pm[nt][1]);
                *reinterpret_cast<uint32_t *>(&sl.Tb[gq + 8][8 * nt + 2 * jq]) = gc_pack(pm[nt][2], pm[nt][3]);
            }
            __syncwarp();
            if (lane == 0) gc_arrive(gc_s32(&sm.ready[s]));
        }
        if (*abort_flag && lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        return;
    }

    // ================================ state (four warps, 32 value columns each) ================================
    // One state warp per scheduler: its 32 value columns are two 16-row MMA tiles (mt) that share every B operand (k, q, T, P)
    // and give the tensor pipe eight independent accumulators to work on.
    const int v0 = col0 + warp * 16 * MT;
    // S^T accumulators: tile (mt, i) covers rows v0 + 16 mt + gq (+8), k columns [8i, 8i+8):
    // St[mt][i] = {S^T[row][8i+2jq], [..+1], S^T[row+8][8i+2jq], [..+1]}
    float St[MT][16][4];
    float *sp = state + (static_cast<int64_t>(b) * n_v_heads + h) * kGcD * kGcD;  // [k][v]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int vr = v0 + 16 * mt + gq;
            St[mt][i][0] = sp[(8 * i + 2 * jq) * kGcD + vr];
            St[mt][i][1] = sp[(8 * i + 2 * jq + 1) * kGcD + vr];
            St[mt][i][2] = sp[(8 * i + 2 * jq) * kGcD + vr + 8];
            St[mt][i][3] = sp[(8 * i + 2 * jq + 1) * kGcD + vr + 8];
        }
    bool failed = false;
    for (int c = 0; c < n_chunks; ++c) {
        const int s = c % kGcSlots, use = c / kGcSlots;
        Slot &sl = sm.slot[s];
        if (!gc_wait(gc_s32(&sm.ready[s]), use & 1, abort_flag)) { failed = true; break; }
        // ---- [K S0 | Q S0]^T = S^T . [K | Q]^T: rows = this warp's value columns, columns = 16 tokens of k then 16 tokens of q ----
        float X[MT][4][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int n = 0; n < 4; ++n) X[mt][n][0] = X[mt][n][1] = X[mt][n][2] = X[mt][n][3] = 0.0f;
        // B operands: one ldmatrix.x4 per 16 state columns brings the four 8 x 8 blocks (tokens 0-7 / 8-15) x (columns +0 / +8) of k
        // (and one of q): lane -> row address of matrix (lane >> 3) = token 8 (lane >> 4) + (lane & 7), column block (lane >> 3) & 1
        const uint32_t xk_lane = gc_s32(&sl.Kb[8 * (lane >> 4) + (lane & 7)][8 * ((lane >> 3) & 1)]);
        const uint32_t xq_lane = gc_s32(&sl.Qb[8 * (lane >> 4) + (lane & 7)][8 * ((lane >> 3) & 1)]);
#pragma unroll
        for (int kk8 = 0; kk8 < 8; ++kk8) {
            uint32_t kb[4], qb[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(kb[0]), "=r"(kb[1]), "=r"(kb[2]), "=r"(kb[3]) : "r"(xk_lane + 32u * kk8));
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(qb[0]), "=r"(qb[1]), "=r"(qb[2]), "=r"(qb[3]) : "r"(xq_lane + 32u * kk8));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint32_t a0 = gc_pack(St[mt][2 * kk8][0], St[mt][2 * kk8][1]), a1 = gc_pack(St[mt][2 * kk8][2], St[mt][2 * kk8][3]);
                const uint32_t a2 = gc_pack(St[mt][2 * kk8 + 1][0], St[mt][2 * kk8 + 1][1]), a3 = gc_pack(St[mt][2 * kk8 + 1][2], St[mt][2 * kk8 + 1][3]);
                gc_mma(X[mt][0], a0, a1, a2, a3, kb[0], kb[1]);
                gc_mma(X[mt][1], a0, a1, a2, a3, kb[2], kb[3]);
                gc_mma(X[mt][2], a0, a1, a2, a3, qb[0], qb[1]);
                gc_mma(X[mt][3], a0, a1, a2, a3, qb[2], qb[3]);
            }
        }
        // R^T = beta (V^T - Gamma (K S0)^T) in the accumulator layout = the A operand (k = tokens) of U^T = R^T . T^T;
        // (Gamma Q S0)^T = (Q S0)^T scaled per token column
        uint32_t r[MT][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const int s0 = 8 * n + 2 * jq;
            const float b0 = sl.b[s0], b1 = sl.b[s0 + 1], g0 = sl.gam[s0], g1 = sl.gam[s0 + 1];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int vr = v0 + 16 * mt + gq;
                const float r00 = b0 * (gc_f32(sl.raw[2][s0][vr]) - g0 * X[mt][n][0]), r01 = b1 * (gc_f32(sl.raw[2][s0 + 1][vr]) - g1 * X[mt][n][1]);
                const float r10 = b0 * (gc_f32(sl.raw[2][s0][vr + 8]) - g0 * X[mt][n][2]), r11 = b1 * (gc_f32(sl.raw[2][s0 + 1][vr + 8]) - g1 * X[mt][n][3]);
                r[mt][2 * n] = gc_pack(r00, r01);
                r[mt][2 * n + 1] = gc_pack(r10, r11);
                X[mt][2 + n][0] *= g0; X[mt][2 + n][1] *= g1; X[mt][2 + n][2] *= g0; X[mt][2 + n][3] *= g1;
            }
        }
        // ---- U^T = R^T . T^T; O^T = (Gamma Q S0)^T + U^T . P^T; S^T = Gamma_C S^T + (U^T diag(exp(G_C - G))) . K ----
        float U[MT][2][4];
        {
            const uint32_t t00 = gc_ld32(&sl.Tb[gq][2 * jq]), t01 = gc_ld32(&sl.Tb[gq][2 * jq + 8]);
            const uint32_t t10 = gc_ld32(&sl.Tb[8 + gq][2 * jq]), t11 = gc_ld32(&sl.Tb[8 + gq][2 * jq + 8]);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                U[mt][0][0] = U[mt][0][1] = U[mt][0][2] = U[mt][0][3] = 0.0f;
                U[mt][1][0] = U[mt][1][1] = U[mt][1][2] = U[mt][1][3] = 0.0f;
                gc_mma(U[mt][0], r[mt][0], r[mt][1], r[mt][2], r[mt][3], t00, t01);
                gc_mma(U[mt][1], r[mt][0], r[mt][1], r[mt][2], r[mt][3], t10, t11);
            }
        }
        uint32_t w[MT][4];
        {
            const uint32_t p00 = gc_ld32(&sl.P[gq][2 * jq]), p01 = gc_ld32(&sl.P[gq][2 * jq + 8]);
            const uint32_t p10 = gc_ld32(&sl.P[8 + gq][2 * jq]), p11 = gc_ld32(&sl.P[8 + gq][2 * jq + 8]);
            // token columns of U scaled by exp(G_C - G_s) for the state update
            const float d00 = sl.dec[2 * jq], d01 = sl.dec[2 * jq + 1], d10 = sl.dec[8 + 2 * jq], d11 = sl.dec[8 + 2 * jq + 1];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint32_t u0 = gc_pack(U[mt][0][0], U[mt][0][1]), u1 = gc_pack(U[mt][0][2], U[mt][0][3]);
                const uint32_t u2 = gc_pack(U[mt][1][0], U[mt][1][1]), u3 = gc_pack(U[mt][1][2], U[mt][1][3]);
                gc_mma(X[mt][2], u0, u1, u2, u3, p00, p01);
                gc_mma(X[mt][3], u0, u1, u2, u3, p10, p11);
                w[mt][0] = gc_pack(U[mt][0][0] * d00, U[mt][0][1] * d01); w[mt][1] = gc_pack(U[mt][0][2] * d00, U[mt][0][3] * d01);
                w[mt][2] = gc_pack(U[mt][1][0] * d10, U[mt][1][1] * d11); w[mt][3] = gc_pack(U[mt][1][2] * d10, U[mt][1][3] * d11);
            }
        }
        const float gC = sl.gam[kGcC - 1];
        // k itself is the B operand of the update, its 8 x 8 blocks transposed on load.  lane -> row address of ldmatrix.x4.trans:
        // matrix (lane >> 3): rows s = (lane & 7) + 8 (matrix & 1), column block + (matrix >> 1)
        const uint32_t kb_lane = gc_s32(&sl.Kb[(lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(kb_lane + 16u * i));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                St[mt][i][0] *= gC; St[mt][i][1] *= gC; St[mt][i][2] *= gC; St[mt][i][3] *= gC;
                gc_mma(St[mt][i], w[mt][0], w[mt][1], w[mt][2], w[mt][3], b0, b1);
                St[mt][i + 1][0] *= gC; St[mt][i + 1][1] *= gC; St[mt][i + 1][2] *= gC; St[mt][i + 1][3] *= gC;
                gc_mma(St[mt][i + 1], w[mt][0], w[mt][1], w[mt][2], w[mt][3], b2, b3);
            }
        }
        // this warp is through with the slot
        __syncwarp();
        if (lane == 0) gc_arrive(gc_s32(&sm.done[s]));
        // outputs: X[mt][2 + n] = O^T rows v0 + 16 mt + gq (+8), tokens 8n + 2jq (+1)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int t = c * kGcC + 8 * n + 2 * jq + e;
                if (t < n_tokens) {
                    float *op = out + ((static_cast<int64_t>(b) * n_tokens + t) * n_v_heads + h) * kGcD + v0 + gq;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        op[16 * mt] = X[mt][2 + n][e];
                        op[16 * mt + 8] = X[mt][2 + n][2 + e];
                    }
                }
            }
    }
    if (failed) {
        if (lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        return;  // the state is left as it was
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int vr = v0 + 16 * mt + gq;
            sp[(8 * i + 2 * jq) * kGcD + vr] = St[mt][i][0];
            sp[(8 * i + 2 * jq + 1) * kGcD + vr] = St[mt][i][1];
            sp[(8 * i + 2 * jq) * kGcD + vr + 8] = St[mt][i][2];
            sp[(8 * i + 2 * jq + 1) * kGcD + vr + 8] = St[mt][i][3];
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

// [n_seqs, n_tokens, n_heads, 128] fp32 or bf16 -> 4-D map (d, head, token, sequence), box 128 x 1 x 16 x 1, no swizzle
static bool gc_make_map(CUtensorMap *map, const void *base, bool bf16, int n_seqs, int n_tokens, int n_heads) {
    GcEncodeTiledFn fn = gc_encode_fn();
    if (!fn) return false;
    const cuuint64_t es = bf16 ? 2 : 4;
    const cuuint64_t dims[4] = {kGcD, static_cast<cuuint64_t>(n_heads), static_cast<cuuint64_t>(n_tokens), static_cast<cuuint64_t>(n_seqs)};
    const cuuint64_t strides[3] = {kGcD * es, static_cast<cuuint64_t>(n_heads) * kGcD * es, static_cast<cuuint64_t>(n_tokens) * n_heads * kGcD * es};
    const cuuint32_t box[4] = {kGcD, 1, kGcC, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename TIn, int MT>
static int32_t gc_launch(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const float *g, const float *beta, float *state, float *out,
                         int n_seqs, int n_tokens, int n_k_heads, int n_v_heads, int *err, cudaStream_t s) {
    static PerDeviceState configured;
    const int dev = current_device();
    constexpr int kBytes = static_cast<int>(sizeof(GcSmem<TIn>) + 128);
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel<TIn, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_gdn_chunk_prefill: %s", cudaGetErrorString(e));
        configured.set(dev, 1);
    }
    dim3 grid(n_v_heads * (2 / MT), n_seqs);
    prof_begin(s);
    gdn_chunk_kernel<TIn, MT><<<grid, gc_threads<MT>(), kBytes, s>>>(mq, mk, mv, g, beta, state, out, n_tokens, n_k_heads, n_v_heads, err);
    prof_end(s);
    return check_launch("hs_gdn_chunk_prefill");
}

// The body of hs_gdn_chunk_prefill; `in_bf16`: q, k, v are bf16 (the layer entry's own prologue writes them so: the kernel rounds
// q and k to bf16 anyway and v is a bf16 value to begin with, so the results are the same bit for bit).
int32_t gdn_chunk_impl(const void *q, const void *k, const void *v, bool in_bf16, const float *g, const float *beta, float *state, float *out,
                       int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim, int32_t head_v_dim, hs_stream_t stream) {
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
    if (!gc_make_map(&mq, q, in_bf16, n_seqs, n_tokens, n_k_heads) || !gc_make_map(&mk, k, in_bf16, n_seqs, n_tokens, n_k_heads) ||
        !gc_make_map(&mv, v, in_bf16, n_seqs, n_tokens, n_v_heads))
        return fail(HS_ERR_UNSUPPORTED, "hs_gdn_chunk_prefill: the driver refused the tensor maps (use hs_gdn_recurrent)");
    cudaStream_t s = as_stream(stream);
    // a head over two CTAs when even so the launch fills at most one wave
    const bool split = 2LL * n_seqs * n_v_heads <= sm_count();
#define HS_GC(T, M) gc_launch<T, M>(mq, mk, mv, g, beta, state, out, n_seqs, n_tokens, n_k_heads, n_v_heads, err, s)
    const int32_t st = in_bf16 ? (split ? HS_GC(__nv_bfloat16, 1) : HS_GC(__nv_bfloat16, 2)) : (split ? HS_GC(float, 1) : HS_GC(float, 2));
#undef HS_GC
    return st;
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_gdn_chunk_prefill(const float *q, const float *k, const float *v, const float *g, const float *beta, float *state,
                             float *out, int32_t n_seqs, int32_t n_tokens, int32_t n_k_heads, int32_t n_v_heads, int32_t head_k_dim,
                             int32_t head_v_dim, hs_stream_t stream) {
    return gdn_chunk_impl(q, k, v, false, g, beta, state, out, n_seqs, n_tokens, n_k_heads, n_v_heads, head_k_dim, head_v_dim, stream);
}

}  // extern "C"
