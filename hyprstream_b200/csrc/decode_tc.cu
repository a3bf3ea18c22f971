// Int8-KV decode attention for head_dim 128: a persistent, warp-specialised kernel.
//
//   * one CTA per SM; the tokens of ALL sequences, cut into 32-token tiles, are divided evenly over the
//     CTAs (flat split-KV), so ragged batches balance without padding;
//   * a producer warp streams each tile of the [tokens, kv_heads, 128] u8 cache into a 3-stage shared
//     memory ring with bulk async copies (cp.async.bulk, one 16-byte-aligned row of all kv heads per
//     lane, completion on an mbarrier) — the HBM reads are whole contiguous rows;
//   * consumer warp h owns kv head h and the G query heads that share it: codes are widened to fp16 with
//     byte permutes (exactly: 1024 + code, minus 1151), q.K^T and P.V run on the tensor cores
//     (mma.sync m16n8k16, fp32 accumulate) with the block scales applied to the fp32 scores (K) and
//     folded into P (V); online softmax in the exp2 domain, quad shuffles for the row maximum;
//   * each (CTA, sequence) pair writes one normalised partial + log-sum-exp; the merge kernel combines.
//
// Replaces, for the q_len == 1 path, cache.get() (full-history dequantise, kv_cache.rs:1499-1643) + GQA
// expansion (llama.rs:847-872) + compute_attention_masked (llama.rs:1023-1119) + the padding/mask of
// forward_batched (llama.rs:787-826,2540-2572).
//
// Every wait on an mbarrier is bounded; on expiry the CTA records HS_DEVERR_WAIT_TIMEOUT and winds down.
#include <cuda_fp16.h>

#include "hs_common.cuh"

namespace hs {

constexpr int kTcTile = 32;    // tokens per stage
constexpr int kTcStages = 3;
constexpr int kTcRowPad = 64;  // bytes of padding per token row in shared memory (bank spread)
constexpr long long kTcWaitCycles = 4000000000LL;  // ~2 s at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another warp already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kTcWaitCycles) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8..15 of A are never used (a1 = a3 = 0): at most 8 query heads share a kv head
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
// two u8 codes (bytes `lo_sel` of w) -> fp16x2 of (code - 127): bytes become 1024 + code exactly, then - 1151
__device__ __forceinline__ uint32_t codes_to_h2(uint32_t w, uint32_t selector) {
    uint32_t h = __byte_perm(w, 0x64646464u, selector);
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h), "r"(0x647F647Fu));
    return r;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float clamp_h(float x) { return fminf(fmaxf(x, -65504.0f), 65504.0f); }

template <int HKV, int BPR, bool SF16>
struct TcLayout {
    static constexpr int kRowG = HKV * 128;            // bytes of one token row in global memory
    static constexpr int kRowS = kRowG + kTcRowPad;    // ... in shared memory
    static constexpr int kSRow = HKV * BPR * (SF16 ? 2 : 4);  // scale bytes per token
    static constexpr int kKOff = 0;
    static constexpr int kVOff = kTcTile * kRowS;
    static constexpr int kKsOff = 2 * kTcTile * kRowS;
    static constexpr int kVsOff = kKsOff + kTcTile * kSRow;
    static constexpr int kStage = (kVsOff + kTcTile * kSRow + 127) / 128 * 128;
    static constexpr int kBarOff = kTcStages * kStage;
    static constexpr int kTotal = kBarOff + 2 * kTcStages * 8 + 16;
    static constexpr uint32_t kTxBytes = 2u * kTcTile * kRowG + 2u * kTcTile * kSRow;
};

template <int HKV, int G, int BPR, bool SF16>
__global__ void __launch_bounds__((HKV + 1) * 32, 1)
decode_int8_tc_kernel(ViewDev view, const uint16_t *__restrict__ q, const int32_t *__restrict__ seq_lens, int n_seqs,
                      int n_q_heads, float kmul, float *__restrict__ o_part, float *__restrict__ lse_part,
                      int *__restrict__ err) {
    using LT = TcLayout<HKV, BPR, SF16>;
    extern __shared__ __align__(128) unsigned char smem[];
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + LT::kBarOff + 2 * kTcStages * 8);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + LT::kBarOff, bar_empty = bar_full + kTcStages * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, HKV);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int cap = view.page_tokens * view.pages_per_seq;
    const int64_t cta = blockIdx.x, n_ctas = gridDim.x;
    int64_t total = 0;
    bool over = false;
    for (int r = 0; r < n_seqs; ++r) {
        const int L = seq_lens[r];
        over |= L > cap;
        total += (min(max(L, 0), cap) + kTcTile - 1) / kTcTile;
    }
    if (over && threadIdx.x == 0 && cta == 0) atomicOr(err, HS_DEVERR_DECODE_RANGE);
    const int64_t t_begin = part_begin(cta, total, n_ctas), t_end = part_begin(cta + 1, total, n_ctas);
    if (t_begin >= t_end) return;

    if (warp == HKV) {
        // ================================ producer warp ================================
        int it = 0;
        int64_t acc = 0;
        bool ok = true;
        for (int r = 0; r < n_seqs && acc < t_end && ok; ++r) {
            const int L = min(max(seq_lens[r], 0), cap);
            const int nt = (L + kTcTile - 1) / kTcTile;
            const int64_t lo = max(t_begin, acc), hi = min(t_end, acc + nt), base = acc;
            acc += nt;
            for (int64_t tile = lo - base; tile < hi - base && ok; ++tile, ++it) {
                const int stage = it % kTcStages;
                if (it >= kTcStages) ok = mbar_wait(bar_empty + 8 * stage, ((it / kTcStages) - 1) & 1, abort_flag);
                if (!ok) break;
                const int t0 = static_cast<int>(tile) * kTcTile;
                const int page = t0 / view.page_tokens;
                const int64_t pidx = static_cast<int64_t>(r) * view.pages_per_seq + page;
                const int in_page = t0 - page * view.page_tokens;
                const uint32_t full = bar_full + 8 * stage;
                if (lane == 0) mbar_expect_tx(full, LT::kTxBytes);
                __syncwarp();
                const uint32_t sbase = smem_base + stage * LT::kStage;
                const unsigned char *kp = reinterpret_cast<const unsigned char *>(view.k_pages[pidx]);
                const unsigned char *vp = reinterpret_cast<const unsigned char *>(view.v_pages[pidx]);
                bulk_g2s(sbase + LT::kKOff + lane * LT::kRowS, kp + static_cast<int64_t>(in_page + lane) * LT::kRowG, LT::kRowG, full);
                bulk_g2s(sbase + LT::kVOff + lane * LT::kRowS, vp + static_cast<int64_t>(in_page + lane) * LT::kRowG, LT::kRowG, full);
                if (lane == 0)
                    bulk_g2s(sbase + LT::kKsOff, reinterpret_cast<const unsigned char *>(view.k_scale_pages[pidx]) + static_cast<int64_t>(in_page) * LT::kSRow,
                             kTcTile * LT::kSRow, full);
                if (lane == 1)
                    bulk_g2s(sbase + LT::kVsOff, reinterpret_cast<const unsigned char *>(view.v_scale_pages[pidx]) + static_cast<int64_t>(in_page) * LT::kSRow,
                             kTcTile * LT::kSRow, full);
            }
        }
        if (!ok) {
            // give the copies already in flight a bounded chance to land before the CTA's shared memory is released
            const long long t0c = clock64();
            while (clock64() - t0c < 2000000LL) {}
            if (lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        }
        return;
    }

    // ================================ consumer warps ================================
    const int head = warp;           // kv head
    const int g = lane >> 2, j = lane & 3;
    const float vmul = 1.0f / 127.0f;
    int it = 0;
    int64_t acc = 0;
    bool ok = true;
    for (int r = 0; r < n_seqs && acc < t_end && ok; ++r) {
        const int L = min(max(seq_lens[r], 0), cap);
        const int nt_seq = (L + kTcTile - 1) / kTcTile;
        const int64_t lo = max(t_begin, acc), hi = min(t_end, acc + nt_seq), base = acc;
        acc += nt_seq;
        if (lo >= hi) continue;

        // ---- query fragments of this sequence: fp16, d permuted so that one 16-byte K load feeds 4 k-steps ----
        uint32_t qa[2][4][2];
        if (g < G) {
            const uint16_t *qp = q + (static_cast<int64_t>(r) * n_q_heads + head * G + g) * 128;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint4 w0 = *reinterpret_cast<const uint4 *>(qp + 64 * b + 16 * j);
                const uint4 w1 = *reinterpret_cast<const uint4 *>(qp + 64 * b + 16 * j + 8);
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    qa[b][s][0] = pack_h2(clamp_h(bf16lo(ww[2 * s])), clamp_h(bf16hi(ww[2 * s])));
                    qa[b][s][1] = pack_h2(clamp_h(bf16lo(ww[2 * s + 1])), clamp_h(bf16hi(ww[2 * s + 1])));
                }
            }
        } else {
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int s = 0; s < 4; ++s) qa[b][s][0] = qa[b][s][1] = 0u;
        }
        float m = -INFINITY, l_part = 0.0f;
        float O[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.0f;

        for (int64_t tile = lo - base; tile < hi - base; ++tile, ++it) {
            const int stage = it % kTcStages;
            ok = mbar_wait(bar_full + 8 * stage, (it / kTcStages) & 1, abort_flag);
            if (!ok) break;
            const unsigned char *sK = smem + stage * LT::kStage + LT::kKOff;
            const unsigned char *sV = smem + stage * LT::kStage + LT::kVOff;
            const unsigned char *sKs = smem + stage * LT::kStage + LT::kKsOff;
            const unsigned char *sVs = smem + stage * LT::kStage + LT::kVsOff;
            const int t0 = static_cast<int>(tile) * kTcTile;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                // ---- S = q . K^T for 16 tokens (two n-tiles of 8), one accumulator per 64-wide d block ----
                float sacc[2][2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int b = 0; b < 2; ++b) sacc[nt][b][0] = sacc[nt][b][1] = sacc[nt][b][2] = sacc[nt][b][3] = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const unsigned char *krow = sK + (u * 16 + nt * 8 + g) * LT::kRowS + head * 128 + 16 * j;
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const uint4 kv = *reinterpret_cast<const uint4 *>(krow + 64 * b);
                        const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                        for (int s = 0; s < 4; ++s)
                            mma_f16(sacc[nt][b], qa[b][s][0], qa[b][s][1], codes_to_h2(kw[s], 0x4140), codes_to_h2(kw[s], 0x4342));
                    }
                }
                // ---- scales of this thread's 4 tokens, scores in the exp2 domain, masking ----
                float p[2][2], pv[2][2][2];
                float mx = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tl = u * 16 + nt * 8 + 2 * j + e;
                        const bool valid = t0 + tl < L;
                        float ks[2], vs[2];
                        if (SF16) {
                            const __half *kp = reinterpret_cast<const __half *>(sKs) + (tl * HKV + head) * BPR;
                            const __half *vp = reinterpret_cast<const __half *>(sVs) + (tl * HKV + head) * BPR;
                            ks[0] = __half2float(kp[0]); vs[0] = __half2float(vp[0]);
                            ks[1] = BPR == 2 ? __half2float(kp[BPR - 1]) : ks[0];
                            vs[1] = BPR == 2 ? __half2float(vp[BPR - 1]) : vs[0];
                        } else {
                            const float *kp = reinterpret_cast<const float *>(sKs) + (tl * HKV + head) * BPR;
                            const float *vp = reinterpret_cast<const float *>(sVs) + (tl * HKV + head) * BPR;
                            ks[0] = kp[0]; vs[0] = vp[0];
                            ks[1] = BPR == 2 ? kp[BPR - 1] : ks[0];
                            vs[1] = BPR == 2 ? vp[BPR - 1] : vs[0];
                        }
                        const float s2 = (sacc[nt][0][e] * ks[0] + sacc[nt][1][e] * ks[1]) * kmul;
                        p[nt][e] = valid ? s2 : -INFINITY;
                        pv[nt][e][0] = valid ? vs[0] * vmul : 0.0f;
                        pv[nt][e][1] = valid ? vs[1] * vmul : 0.0f;
                        mx = fmaxf(mx, p[nt][e]);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m, mx);
                const float corr = m_new == -INFINITY ? 1.0f : exp2f(m - m_new);
                m = m_new;
                float psum = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        p[nt][e] = m_new == -INFINITY ? 0.0f : exp2f(p[nt][e] - m_new);
                        psum += p[nt][e];
                    }
                l_part = l_part * corr + psum;
#pragma unroll
                for (int i = 0; i < 16; ++i) { O[i][0] *= corr; O[i][1] *= corr; }
                // ---- O += P' . V with the V block scale folded into P' ----
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t a0 = pack_h2(p[0][0] * pv[0][0][b], p[0][1] * pv[0][1][b]);
                    const uint32_t a2 = pack_h2(p[1][0] * pv[1][0][b], p[1][1] * pv[1][1][b]);
                    uint2 x[2][2];
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e)
                            x[nt][e] = *reinterpret_cast<const uint2 *>(sV + (u * 16 + nt * 8 + 2 * j + e) * LT::kRowS + head * 128 + 64 * b + 8 * g);
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t A0 = k ? x[0][0].y : x[0][0].x, B0 = k ? x[0][1].y : x[0][1].x;
                        const uint32_t A1 = k ? x[1][0].y : x[1][0].x, B1 = k ? x[1][1].y : x[1][1].x;
                        const uint32_t t01 = __byte_perm(A0, B0, 0x5140), t23 = __byte_perm(A0, B0, 0x7362);
                        const uint32_t u01 = __byte_perm(A1, B1, 0x5140), u23 = __byte_perm(A1, B1, 0x7362);
                        mma_f16(O[8 * b + 4 * k + 0], a0, a2, codes_to_h2(t01, 0x4140), codes_to_h2(u01, 0x4140));
                        mma_f16(O[8 * b + 4 * k + 1], a0, a2, codes_to_h2(t01, 0x4342), codes_to_h2(u01, 0x4342));
                        mma_f16(O[8 * b + 4 * k + 2], a0, a2, codes_to_h2(t23, 0x4140), codes_to_h2(u23, 0x4140));
                        mma_f16(O[8 * b + 4 * k + 3], a0, a2, codes_to_h2(t23, 0x4342), codes_to_h2(u23, 0x4342));
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
        }
        if (!ok) break;
        // ---- partial of this (CTA, sequence) pair ----
        float l = l_part;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (g < G) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const int64_t hrow = (cta + r) * n_q_heads + head * G + g;
            float *op = o_part + hrow * 128;
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    op[64 * b + 16 * j + i] = O[8 * b + i][0] * inv;
                    op[64 * b + 16 * j + 8 + i] = O[8 * b + i][1] * inv;
                }
            if (j == 0) lse_part[hrow] = l > 0.0f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
    }
    if (!ok && lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
}

template <int HKV, int G, int BPR, bool SF16>
static int32_t launch_tc(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads, float kmul,
                         float *o_part, float *lse_part, int *err, int n_ctas, cudaStream_t s) {
    using LT = TcLayout<HKV, BPR, SF16>;
    auto kern = decode_int8_tc_kernel<HKV, G, BPR, SF16>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LT::kTotal);
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_decode: %s", cudaGetErrorString(e));
        configured = true;
    }
    kern<<<n_ctas, (HKV + 1) * 32, LT::kTotal, s>>>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err);
    return HS_OK;
}

// Returns HS_OK and sets *n_ctas_out (> 0) when the tensor-core kernel took the launch; *n_ctas_out = 0
// when the shape is not covered and the caller should use the generic kernel.
int32_t decode_int8_tc_try(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads,
                           float softmax_scale, float *o_part, float *lse_part, int *err, cudaStream_t s, int *n_ctas_out) {
    *n_ctas_out = 0;
    if (v.kind != HS_KV_INT8 || v.head_dim != 128 || v.n_kv_heads != 8) return HS_OK;
    if (v.page_tokens % kTcTile != 0) return HS_OK;
    const int G = n_q_heads / v.n_kv_heads;
    if (G != 4) return HS_OK;
    const int bpr = 128 / v.block;
    if (bpr != 1 && bpr != 2) return HS_OK;
    const bool sf16 = v.scale_dtype == HS_SCALE_F16;
    const int n_ctas = sm_count();
    const float kmul = softmax_scale * 1.4426950408889634f / 127.0f;
    int32_t st;
    if (bpr == 2 && !sf16) st = launch_tc<8, 4, 2, false>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err, n_ctas, s);
    else if (bpr == 2 && sf16) st = launch_tc<8, 4, 2, true>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err, n_ctas, s);
    else if (bpr == 1 && !sf16) st = launch_tc<8, 4, 1, false>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err, n_ctas, s);
    else st = launch_tc<8, 4, 1, true>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err, n_ctas, s);
    if (st == HS_OK) *n_ctas_out = n_ctas;
    return st;
}

}  // namespace hs
