// Causal GQA prefill attention on the 5th-generation tensor cores (bf16; head_dim 128 first, head_dim 256 further down).
//
// One CTA = two 128-row query tiles of one head (256 rows) sharing every K/V tile.  Roles (10 warps):
//   warp 8  loader: TMA tensor loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast) of the two Q tiles
//           once and of K/V tiles of 128 keys into a 2-stage shared-memory ring; completion on mbarriers
//   warp 9  MMA issuer: the warp walks a fixed schedule with one elected lane issuing, per query tile x and key tile j,
//             S_j = Q_x . K_j^T    (both operands K-major in shared memory, accumulator 128 x 128 fp32 in TMEM)
//             O_x += P_j . V_j     (P_j read from TMEM as bf16, V_j MN-major in shared memory)
//           in the order P.V^0_j, S^0_{j+1}, P.V^1_j, S^1_{j+1} (no wait between a P.V and the S that overwrites its P: MMAs
//           execute in issue order), and tcgen05.commit to the mbarriers that hand results over; one tile's MMAs run
//           under the other tile's softmax
//   warps 0-3 / 4-7  softmax of tile 0 / 1: thread = query row (TMEM lane).  Two passes of tcgen05.ld over the
//           score row (maximum, then exp2 and P as bf16 pairs written back over the scores with tcgen05.st); the
//           output accumulator in TMEM is rescaled only when a row maximum grew by more than 2^8 (the final
//           O / l is exact either way); epilogue: O / l, optional sigmoid gate, bf16 store
//
// TMEM columns: [0,128) S/P tile 0, [128,256) S/P tile 1, [256,384) O tile 0, [384,512) O tile 1.  Shared
// memory: 2 x Q 32 KB + 2 x (K 32 KB + V 32 KB).  FLOPs per (query tile, key tile): 2 x 2 x 128^3.
// Bound: tensor pipe (and MUFU exp2).
//
// Replaces compute_attention_masked for q_len > 1 (architectures/llama.rs:1023-1119) with GQA expansion
// (llama.rs:847-872) and the cached-prefix offset tril(k_len - q_len) (llama.rs:1074-1084); with `gate`,
// Qwen3_5FullAttention's prefill branch (qwen3_5.rs:1012-1059) at head_dim 128.
//
// Every mbarrier wait is bounded; on expiry the CTA records HS_DEVERR_WAIT_TIMEOUT, frees its TMEM and returns, and CTAs that start
// while that flag is set (until the host takes it) return at once, so a failed launch ends in a fraction of a second.
#include <cuda.h>

#include "hs_common.cuh"

namespace hs {

constexpr int kT5M = 128, kT5N = 128, kT5D = 128;
constexpr int kT5Stages = 2;
constexpr int kT5BlockM = 2 * kT5M;  // two query tiles per CTA
constexpr int kT5Threads = 320;
constexpr int kT5TileBytes = kT5N * kT5D * 2;          // 32 KB: two 64-column halves of [128 rows][128 B]
constexpr int kT5HalfBytes = kT5TileBytes / 2;
constexpr int kT5SmemBytes = kT5TileBytes * (2 + 2 * kT5Stages) + 1024;  // two Q tiles, K/V ring, alignment slack
constexpr long long kT5WaitCycles = 400000000LL;  // ~0.2 s: any legitimate wait is far below a millisecond
constexpr float kT5RescaleThreshold = 8.0f;            // log2 units

__device__ __forceinline__ uint32_t t5_s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool t5_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool t5_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (t5_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (t5_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kT5WaitCycles) { *abort_flag = 1; return false; }
    }
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool t5_elect() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred)::"memory");
    return pred != 0;
}
__device__ __forceinline__ void t5_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void t5_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t t5_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFF) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void t5_mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5,%6,%7,%8}, p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
__device__ __forceinline__ void t5_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5,%6,%7,%8}, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
__device__ __forceinline__ void t5_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void t5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t5_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void t5_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
// 8-column forms for the rare rescale of O, which runs while a whole score row is held in registers
__device__ __forceinline__ void t5_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void t5_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void t5_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void t5_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void t5_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// one [128 rows x 64 columns] box of a 4-D tensor (d, head, token, sequence) -> swizzled shared memory
__device__ __forceinline__ void t5_tma_load(uint32_t dst, const CUtensorMap *map, int x, int head, int token, int seq, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(head), "r"(token), "r"(seq), "r"(bar) : "memory");
}

struct T5Bars {
    uint64_t q, kfull[kT5Stages], vfull[kT5Stages], kvempty[kT5Stages], sfull[2], pready[2], odone[2];
};

__device__ __forceinline__ uint32_t t5_pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float t5_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// packed pairs of f32 (sm_100): d = a * b + c and d = a + b on both halves
__device__ __forceinline__ uint64_t t5_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void t5_unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t t5_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t t5_add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ bool t5_test_wait(uint32_t bar, uint32_t parity) {  // non-blocking probe
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ float t5_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two 128-row query tiles (x = 0, 1) per CTA share every K/V tile.  Warps 0-3: softmax of tile 0, warps 4-7: softmax of
// tile 1, warp 8: loader, warp 9: MMA issuer.  TMEM columns: S/P of tile x at 128x, O of tile x at 256 + 128x.
__global__ void __launch_bounds__(kT5Threads, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, uint16_t *__restrict__ out, const uint16_t *__restrict__ gate, int64_t gate_ts,
                   int64_t gate_hs, int q_len, int kv_len, int n_q_heads, int n_kv_heads, float scale_log2, int *__restrict__ err, uint32_t launch_id) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) T5Bars bars;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t sQ = t5_s32(smem);                       // Q tile 0, Q tile 1
    const uint32_t sKV = sQ + 2 * kT5TileBytes;             // stage s: K at sKV + 2 s tile, V one tile later
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mb = gridDim.x - 1 - blockIdx.x;  // latest (heaviest) query blocks first
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (n_q_heads / n_kv_heads);
    const int m0 = mb * kT5BlockM, off = kv_len - q_len;
    int n_tiles[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int lo = m0 + x * kT5M;
        n_tiles[x] = lo < q_len ? (min(kv_len, off + min(lo + kT5M, q_len)) + kT5N - 1) / kT5N : 0;
    }
    const int n_max = max(n_tiles[0], n_tiles[1]);
    volatile int *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        auto init = [](uint64_t *bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(t5_s32(bar)), "r"(count)); };
        init(&bars.q, 1);
        for (int s = 0; s < kT5Stages; ++s) { init(&bars.kfull[s], 1); init(&bars.vfull[s], 1); init(&bars.kvempty[s], 1); }
        for (int i = 0; i < 2; ++i) { init(&bars.sfull[i], 1); init(&bars.pready[i], kT5M); init(&bars.odone[i], 1); }
        s_abort = *reinterpret_cast<volatile uint32_t *>(err + 1) == launch_id ? 1 : 0;  // a time-out recorded by this launch ends its later CTAs at once
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(t5_s32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const uint32_t tm = s_tmem;
    bool ok = true;

    if (warp == 8) {
        // ================================ loader ================================
        if (lane == 0) {
            t5_expect_tx(t5_s32(&bars.q), 2 * kT5TileBytes);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                t5_tma_load(sQ + x * kT5TileBytes, &map_q, 0, h, m0 + x * kT5M, b, t5_s32(&bars.q));
                t5_tma_load(sQ + x * kT5TileBytes + kT5HalfBytes, &map_q, 64, h, m0 + x * kT5M, b, t5_s32(&bars.q));
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const int s = j & 1;
                if (j >= kT5Stages) ok = t5_wait(t5_s32(&bars.kvempty[s]), ((j >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                const uint32_t sK = sKV + 2 * s * kT5TileBytes, sV = sK + kT5TileBytes;
                t5_expect_tx(t5_s32(&bars.kfull[s]), kT5TileBytes);
                t5_tma_load(sK, &map_k, 0, kvh, j * kT5N, b, t5_s32(&bars.kfull[s]));
                t5_tma_load(sK + kT5HalfBytes, &map_k, 64, kvh, j * kT5N, b, t5_s32(&bars.kfull[s]));
                t5_expect_tx(t5_s32(&bars.vfull[s]), kT5TileBytes);
                t5_tma_load(sV, &map_v, 0, kvh, j * kT5N, b, t5_s32(&bars.vfull[s]));
                t5_tma_load(sV + kT5HalfBytes, &map_v, 64, kvh, j * kT5N, b, t5_s32(&bars.vfull[s]));
            }
        }
    } else if (warp == 9) {
        // ================================ MMA issuer ================================
        // The whole warp walks a fixed schedule with blocking waits, and one elected lane issues:
        //     S^0_0, S^1_0, then per key tile j:  P.V^0_j, S^0_{j+1}, P.V^1_j, S^1_{j+1}
        // (S^x_j = Q_x K_j^T, 8 MMAs 128x128x16 from shared memory; P.V^x_j: 8 MMAs 128x128x16 with P from tensor memory).  S^x_{j+1}
        // overwrites the buffer P.V^x_j reads P from: the MMAs of one thread execute in issue order, so nothing waits in between,
        // and one tile's softmax runs under the other tile's two operations.  The loop is unrolled over the two ring stages, so
        // stage indices, most parities and all descriptor offsets are compile-time constants.
        const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((kT5N >> 3) << 17) | ((kT5M >> 4) << 24);  // bf16 x bf16 -> f32, K-major A and B
        const uint32_t idesc_pv = idesc_qk | (1u << 16);                                                         // B (V) is MN-major
        const uint64_t dq0 = t5_desc(sQ, 16, 1024), dk0 = t5_desc(sKV, 16, 1024), dv0 = t5_desc(sKV + kT5TileBytes, kT5HalfBytes, 1024);
        auto issue_s = [&](int x, int st) {  // S^x = Q_x K^T with the K tile of ring stage st
            if (t5_elect()) {
#pragma unroll
                for (int ks = 0; ks < kT5D / 16; ++ks) {
                    const uint32_t o = (ks >> 2) * kT5HalfBytes + (ks & 3) * 32;
                    t5_mma_ss(tm + x * kT5N, dq0 + ((x * kT5TileBytes + o) >> 4), dk0 + ((2 * st * kT5TileBytes + o) >> 4), idesc_qk, ks > 0);
                }
                t5_commit(t5_s32(&bars.sfull[x]));
            }
            __syncwarp();
        };
        ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.q), 0, abort_flag) && (n_max == 0 || t5_wait(t5_s32(&bars.kfull[0]), 0, abort_flag)));
        if (ok) {
            t5_fence_after();
            if (n_tiles[0] > 0) issue_s(0, 0);
            if (n_tiles[1] > 0) issue_s(1, 0);
        }
        for (int j0 = 0; j0 < n_max && ok; j0 += 2) {
            const uint32_t p2 = (j0 >> 1) & 1;  // phase parity of the ring stages for tiles j0 and j0 + 1
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j = j0 + i;
                if (j >= n_max || !ok) break;
                // tile j sits in stage i in phase j >> 1 (parity p2); tile j + 1 in stage i ^ 1, in phase (j + 1) >> 1 = parity p2 ^ i
                bool k_next_ready = false;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (j >= n_tiles[x]) continue;
                    ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.pready[x]), i, abort_flag) &&
                                                     t5_wait(t5_s32(&bars.vfull[i]), p2, abort_flag));
                    if (!ok) break;
                    t5_fence_after();
                    const bool last_user = x == 1 || j >= n_tiles[1];  // the stage of tile j is free once this P.V has completed
                    if (t5_elect()) {
#pragma unroll
                        for (int ks = 0; ks < kT5N / 16; ++ks)
                            t5_mma_ts(tm + 256 + x * kT5D, tm + x * kT5N + ks * 8, dv0 + ((2 * i * kT5TileBytes + ks * 2048) >> 4), idesc_pv,
                                      (j > 0 || ks > 0) ? 1u : 0u);
                        t5_commit(t5_s32(&bars.odone[x]));
                        if (last_user) t5_commit(t5_s32(&bars.kvempty[i]));
                    }
                    __syncwarp();
                    if (j + 1 < n_tiles[x]) {
                        if (!k_next_ready) {
                            ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.kfull[i ^ 1]), p2 ^ i, abort_flag));
                            if (!ok) break;
                            t5_fence_after();
                            k_next_ready = true;
                        }
                        issue_s(x, i ^ 1);
                    }
                }
            }
        }
    } else {
        // ================================ softmax: thread = query row ================================
        const int x = warp >> 2;  // query tile of this warp group
        const int row = m0 + x * kT5M + (threadIdx.x & 127);
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tm + lane_base + x * kT5N, tO = tm + lane_base + 256 + x * kT5D;
        const int nt = n_tiles[x];
        float m_used = -INFINITY, l = 0.0f;
        for (int j = 0; j < nt && ok; ++j) {
            ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.sfull[x]), j & 1, abort_flag));  // warp-uniform: the TMEM
            if (!ok) break;                                                                      // accesses below are warp-collective
            t5_fence_after();
#ifdef HS_T5_NOSOFTMAX
            t5_fence_before();
            t5_arrive(t5_s32(&bars.pready[x]));
            continue;
#endif
            const int n0 = j * kT5N;
            const bool masked = n0 + kT5N > min(kv_len, off + m0 + x * kT5M + 1);
            const int lim = min(kv_len - 1, off + row) - n0;  // last visible column of this row inside the tile
            // ---- pass 1: row maximum (all four loads in flight, one wait) ----
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            // (the score row stays in registers for the second pass: one trip to tensor memory per tile and row)
            uint32_t r[4][32];
            {
#pragma unroll
                for (int c = 0; c < 4; ++c) t5_ld32(tS + 32 * c, r[c]);
                t5_wait_ld();
                if (!masked) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            mx0 = t5_max3(mx0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                            mx1 = t5_max3(mx1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                            mx2 = t5_max3(mx2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                            mx3 = t5_max3(mx3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
                        }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float a0 = 32 * c + i > lim ? -INFINITY : __uint_as_float(r[c][i]);
                            const float a1 = 32 * c + i + 1 > lim ? -INFINITY : __uint_as_float(r[c][i + 1]);
                            mx0 = t5_max3(mx0, a0, a1);
                        }
                }
            }
            const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool need = m_new - m_used > kT5RescaleThreshold;  // false while both are -inf (NaN compares false)
                if (__any_sync(0xffffffffu, need)) {
                    ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.odone[x]), (j - 1) & 1, abort_flag));
                    if (!ok) break;
                    t5_fence_after();
                    const float f = need ? exp2f(m_used - m_new) : 1.0f;
#pragma unroll
                    for (int c0 = 0; c0 < kT5D; c0 += 8) {
                        uint32_t ro[8];
                        t5_ld8(tO + c0, ro);
                        t5_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
                        t5_st8(tO + c0, ro);
                    }
                    t5_wait_st();
                    l *= f;
                    if (need) m_used = m_new;
                }
                if (m_used == -INFINITY) m_used = m_new;
            }
            // ---- pass 2: P = exp2(s * scale - m) as bf16 pairs, written over the score buffer ----
            const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
            float ps0 = 0.0f, ps1 = 0.0f;
            {
                if (!masked) {
                    const uint64_t sc2 = t5_pack2(scale_log2, scale_log2), nm2 = t5_pack2(neg_m, neg_m);
                    uint64_t acc_a = t5_pack2(0.0f, 0.0f), acc_b = acc_a;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float x0, x1;
                            t5_unpack2(t5_fma2(t5_pack2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), sc2, nm2), x0, x1);
                            const float p0 = t5_ex2(x0), p1 = t5_ex2(x1);
                            if (i & 1) acc_b = t5_add2(acc_b, t5_pack2(p0, p1)); else acc_a = t5_add2(acc_a, t5_pack2(p0, p1));
                            w[i] = t5_pack_bf16x2(p0, p1);
                        }
                        t5_st16(tS + 16 * c, w);
                    }
                    float a0, a1;
                    t5_unpack2(t5_add2(acc_a, acc_b), a0, a1);
                    ps0 = a0; ps1 = a1;
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float p0 = 32 * c + 2 * i > lim ? 0.0f : t5_ex2(fmaf(__uint_as_float(r[c][2 * i]), scale_log2, neg_m));
                            const float p1 = 32 * c + 2 * i + 1 > lim ? 0.0f : t5_ex2(fmaf(__uint_as_float(r[c][2 * i + 1]), scale_log2, neg_m));
                            ps0 += p0; ps1 += p1;
                            w[i] = t5_pack_bf16x2(p0, p1);
                        }
                        t5_st16(tS + 16 * c, w);
                    }
                }
            }
            l += ps0 + ps1;
            t5_wait_st();
            t5_fence_before();
            t5_arrive(t5_s32(&bars.pready[x]));
        }
        // ---- epilogue ----
        if (ok && nt > 0) ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.odone[x]), (nt - 1) & 1, abort_flag));
        if (ok && nt > 0) {
            t5_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const int64_t base = ((static_cast<int64_t>(b) * q_len + row) * n_q_heads + h) * kT5D;
            const int64_t gbase = (static_cast<int64_t>(b) * q_len + row) * gate_ts + h * gate_hs;
#pragma unroll
            for (int c0 = 0; c0 < kT5D; c0 += 32) {
                uint32_t r[32];
                t5_ld32(tO + c0, r);
                t5_wait_ld();
                if (row < q_len) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float x0 = __uint_as_float(r[v4 * 8 + 2 * i]) * inv, x1 = __uint_as_float(r[v4 * 8 + 2 * i + 1]) * inv;
                            if (gate != nullptr) {
                                const uint32_t gw = *reinterpret_cast<const uint32_t *>(gate + gbase + c0 + v4 * 8 + 2 * i);
                                x0 = bf16_round(x0) * bf16_round(1.0f / (1.0f + __expf(-bf16lo(gw))));
                                x1 = bf16_round(x1) * bf16_round(1.0f / (1.0f + __expf(-bf16hi(gw))));
                            }
                            w[i] = pack_bf16(x0, x1);
                        }
                        *reinterpret_cast<uint4 *>(out + base + c0 + v4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    // ---- teardown: every thread arrives here, also after a timed-out wait ----
    if (*abort_flag) {
        if (threadIdx.x == 0) { atomicOr(err, HS_DEVERR_WAIT_TIMEOUT); atomicExch(reinterpret_cast<unsigned int *>(err + 1), launch_id); }
        const long long t0c = clock64();
        while (clock64() - t0c < 2000000LL) {}  // bounded grace period for copies and MMAs still in flight
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
}

// ================================================================================================================
// head_dim 256 (Qwen3.5 full attention, qwen3_5.rs:1012-1059): one 128-row query tile per CTA, key tiles of 64.
//   TMEM columns: four score/probability buffers of 64 columns ([0,256): tile j uses buffer j & 3, so q.k^T runs up to
//   three key tiles ahead of the softmax), the output accumulator 128 x 256 fp32 in [256,512).
//   Shared memory: Q 64 KB (four 64-column boxes of 128 rows), K ring 3 x 32 KB, V ring 2 x 32 KB (boxes of 64 rows).
//   Warps 0-3 and 4-7: softmax of the even and of the odd key tiles (thread = query row in both groups; the special-
//   function unit's 16 exp2 per clock bound a tile at 512 cycles, the same as its MMAs, so two groups alternate and one
//   group's loads, maximum and stores run under the other's exponentials); warp 8: loader, warp 9: MMA issuer.
//   The two groups share a row's reference maximum through shared memory: a group publishes it (and rescales O if it
//   grew by more than 2^8) right after its maximum pass, the other group's next tile starts from there; each group keeps
//   its own partial row sum with the reference it was last brought to, and the two are combined at the end.
//   S = Q.K^T is issued per pair of key tiles: 16 MMAs 128x128x16 on K ring stages of [128 keys][128 columns of d] (the Q
//   slice is read from shared memory once per 128 keys); O += P.V per key tile: 4 MMAs 128x256x16 (P from TMEM, V
//   MN-major: its four 64-column boxes are 8 KB apart).
constexpr int kW5D = 256, kW5M = 128, kW5N = 64;
constexpr int kW5KStages = 3, kW5VStages = 2, kW5SBufs = 4;
constexpr int kW5Threads = 320;  // warps 0-3 / 4-7: softmax of even / odd key tiles, warp 8: loader, warp 9: MMA issuer
constexpr int kW5QBytes = kW5M * kW5D * 2;    // 64 KB
constexpr int kW5QBox = kW5M * 128;           // one 64-column box of Q
constexpr int kW5KVBytes = kW5N * kW5D * 2;   // 32 KB
constexpr int kW5KVBox = kW5N * 128;          // one 64-column box of K or V
constexpr int kW5SmemBytes = kW5QBytes + (kW5KStages + kW5VStages) * kW5KVBytes + 1024;

struct W5Bars {
    uint64_t q, kfull[kW5KStages], kempty[kW5KStages], vfull[kW5VStages], vempty[kW5VStages], sfull[2], pready[kW5SBufs],
        pvdone[kW5SBufs];
};

__global__ void __launch_bounds__(kW5Threads, 1)
prefill_tc5_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, uint16_t *__restrict__ out, const uint16_t *__restrict__ gate, int64_t gate_ts,
                        int64_t gate_hs, int q_len, int kv_len, int n_q_heads, int n_kv_heads, float scale_log2, int *__restrict__ err, uint32_t launch_id) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) W5Bars bars;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ float s_mpub[kW5M];
    __shared__ int s_seq[kW5M];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t sQ = t5_s32(smem), sK = sQ + kW5QBytes, sV = sK + kW5KStages * kW5KVBytes;
    // the two softmax groups exchange their partial sums through the first K stage once every q.k^T has completed
    float(*s_lpart)[kW5M] = reinterpret_cast<float(*)[kW5M]>(smem + kW5QBytes);
    float(*s_mpart)[kW5M] = reinterpret_cast<float(*)[kW5M]>(smem + kW5QBytes + 2 * kW5M * sizeof(float));
    if (threadIdx.x < kW5M) {
        s_seq[threadIdx.x] = 0;
        s_mpub[threadIdx.x] = -INFINITY;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mb = gridDim.x - 1 - blockIdx.x;  // latest (heaviest) query blocks first
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (n_q_heads / n_kv_heads);
    const int m0 = mb * kW5M, off = kv_len - q_len;
    // 64-key tiles, rounded up to whole pairs: q.k^T is issued per pair of tiles; keys past the causal limit or past kv_len
    // (which the tensor maps fill with zeros) are masked in the softmax
    const int n_tiles = ((min(kv_len, off + min(m0 + kW5M, q_len)) + 2 * kW5N - 1) / (2 * kW5N)) * 2;
    const int n_pairs = n_tiles / 2;
    volatile int *abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        auto init = [](uint64_t *bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(t5_s32(bar)), "r"(count)); };
        init(&bars.q, 1);
        for (int s = 0; s < kW5KStages; ++s) { init(&bars.kfull[s], 1); init(&bars.kempty[s], 1); }
        for (int s = 0; s < kW5VStages; ++s) { init(&bars.vfull[s], 1); init(&bars.vempty[s], 1); }
        for (int i = 0; i < 2; ++i) init(&bars.sfull[i], 1);
        for (int i = 0; i < kW5SBufs; ++i) { init(&bars.pready[i], kW5M); init(&bars.pvdone[i], 1); }
        s_abort = *reinterpret_cast<volatile uint32_t *>(err + 1) == launch_id ? 1 : 0;  // a time-out recorded by this launch ends its later CTAs at once
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(t5_s32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const uint32_t tm = s_tmem;
    bool ok = true;

    if (warp == 8) {
        // ================================ loader ================================
        if (lane == 0) {
            t5_expect_tx(t5_s32(&bars.q), kW5QBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) t5_tma_load(sQ + c * kW5QBox, &map_q, 64 * c, h, m0, b, t5_s32(&bars.q));
            // Loads go out in the order the issuer consumes them: the K halves of pairs 0 and 1, then per pair t the V tiles 2t and
            // 2t+1 and the K halves of pair t+2.  A K half-stage holds [128 keys][128 columns of d] as two 64-column boxes.
            auto load_k = [&](int n) -> bool {  // half n: pair n >> 1, columns 128 (n & 1) ..
                const int s = n % kW5KStages;
                if (n >= kW5KStages && !t5_wait(t5_s32(&bars.kempty[s]), (n / kW5KStages - 1) & 1, abort_flag)) return false;
                t5_expect_tx(t5_s32(&bars.kfull[s]), kW5KVBytes);
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    t5_tma_load(sK + s * kW5KVBytes + c * kW5QBox, &map_k, 64 * (2 * (n & 1) + c), kvh, (n >> 1) * 2 * kW5N, b, t5_s32(&bars.kfull[s]));
                return true;
            };
            auto load_v = [&](int j) -> bool {
                const int s = j % kW5VStages;
                if (j >= kW5VStages && !t5_wait(t5_s32(&bars.vempty[s]), (j / kW5VStages - 1) & 1, abort_flag)) return false;
                t5_expect_tx(t5_s32(&bars.vfull[s]), kW5KVBytes);
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    t5_tma_load(sV + s * kW5KVBytes + c * kW5KVBox, &map_v, 64 * c, kvh, j * kW5N, b, t5_s32(&bars.vfull[s]));
                return true;
            };
            for (int n = 0; n < 4 && n < 2 * n_pairs && ok; ++n) ok = load_k(n);
            for (int t = 0; t < n_pairs && ok; ++t) {
                ok = load_v(2 * t) && load_v(2 * t + 1);
                if (ok && t + 2 < n_pairs) ok = load_k(2 * t + 4) && load_k(2 * t + 5);
            }
        }
    } else if (warp == 9) {
        // ================================ MMA issuer ================================
        // The whole warp walks a fixed schedule with blocking waits, and one elected lane issues:
        //     S(pair 0), S(pair 1), then per pair t of key tiles:  P.V_2t,  P.V_2t+1,  S(pair t+2).
        // S(pair) = Q K^T for 128 keys at once (16 MMAs 128x128x16: the Q slice is read from shared memory once per 128 keys, which
        // is what keeps this MMA at the tensor pipe's rate) into two adjacent 64-column score buffers; P.V stays per 64-key tile
        // (4 MMAs 128x256x16).  S(pair t+2) overwrites the buffers whose P tiles P.V_2t and P.V_2t+1 read: the MMAs of one thread
        // execute in issue order, so no wait lies between them and the tensor pipe never drains.
        // The loop is unrolled over 6 pairs (the common period of the 3 K half-stages and the 2 pairs of score buffers), so ring
        // indices, most barrier parities and every descriptor offset are compile-time constants.
        const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | (((2 * kW5N) >> 3) << 17) | ((kW5M >> 4) << 24);
        const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((kW5D >> 3) << 17) | ((kW5M >> 4) << 24);
        const uint64_t dq = t5_desc(sQ, 16, 1024), dk0 = t5_desc(sK, 16, 1024), dv0 = t5_desc(sV, kW5KVBox, 1024);
        // S(pair) into score buffers 2 pb, 2 pb + 1; its K halves are n0 and n0 + 1 (n0 = 2 * pair; ring stage n % 3, phase n / 3)
        auto issue_s = [&](int pb, int st0, uint32_t ph0, int st1, uint32_t ph1) -> bool {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int st = hf ? st1 : st0;
                if (!__all_sync(0xffffffffu, t5_wait(t5_s32(&bars.kfull[st]), hf ? ph1 : ph0, abort_flag))) return false;
                t5_fence_after();
                if (t5_elect()) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        t5_mma_ss(tm + pb * 2 * kW5N, dq + (((2 * hf + (ks >> 2)) * kW5QBox + (ks & 3) * 32) >> 4),
                                  dk0 + ((st * kW5KVBytes + (ks >> 2) * kW5QBox + (ks & 3) * 32) >> 4), idesc_qk, (hf > 0 || ks > 0) ? 1u : 0u);
                    t5_commit(t5_s32(&bars.kempty[st]));
                    if (hf) t5_commit(t5_s32(&bars.sfull[pb]));
                }
                __syncwarp();
            }
            return true;
        };
        ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.q), 0, abort_flag));
        if (ok) ok = issue_s(0, 0, 0, 1, 0);                 // halves 0, 1
        if (ok && n_pairs > 1) ok = issue_s(1, 2, 0, 0, 1);  // halves 2, 3
        for (int t0 = 0; t0 < n_pairs && ok; t0 += 6) {
            const uint32_t p6 = (t0 / 6) & 1;  // parity of the 6-pair period
#pragma unroll
            for (int i = 0; i < 6; ++i) {
                const int t = t0 + i;
                if (t >= n_pairs || !ok) break;
                // ---- P.V of tiles j = 2t + e = 12 q + 2i + e: buffer j & 3, barrier phase j >> 2 = 3q + ((2i + e) >> 2); V stage e,
                //      phase t = 6q + i ----
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int u = (2 * i + e) & 3;
                    ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.pready[u]), p6 ^ (((2 * i + e) >> 2) & 1), abort_flag) &&
                                                     t5_wait(t5_s32(&bars.vfull[e]), i & 1, abort_flag));
                    if (!ok) break;
                    t5_fence_after();
                    if (t5_elect()) {
#pragma unroll
                        for (int ks = 0; ks < kW5N / 16; ++ks)
                            t5_mma_ts(tm + 256, tm + u * kW5N + ks * 8, dv0 + ((e * kW5KVBytes + ks * 2048) >> 4), idesc_pv,
                                      (t > 0 || e > 0 || ks > 0) ? 1u : 0u);
                        t5_commit(t5_s32(&bars.pvdone[u]));  // one phase per four tiles: what the softmax warps wait on
                        t5_commit(t5_s32(&bars.vempty[e]));
                    }
                    __syncwarp();
                }
                if (!ok) break;
                // ---- S(pair t+2): halves n = 2(t+2) + hf = 12 q + 2i + 4 + hf, stage n % 3, phase n / 3 = 4q + (2i + 4 + hf) / 3 ----
                if (t + 2 < n_pairs) {
                    ok = issue_s(i & 1, (2 * i + 4) % 3, ((2 * i + 4) / 3) & 1, (2 * i + 5) % 3, ((2 * i + 5) / 3) & 1);
                }
            }
        }
    } else {
        // ================================ softmax: thread = query row, group = parity of the key tile ================================
        const int grp = warp >> 2, r_local = threadIdx.x & 127;
        const int row = m0 + r_local;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tO = tm + lane_base + 256;
        volatile float *m_pub = s_mpub + r_local;   // the row's reference maximum after the latest published tile
        volatile int *seq = s_seq + r_local;        // number of tiles whose reference has been published
        float l = 0.0f, m_ref = -INFINITY;          // this group's partial row sum, relative to m_ref
        for (int j = grp; j < n_tiles && ok; j += 2) {
            const uint32_t tS = tm + lane_base + (j & 3) * kW5N;
            ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.sfull[(j >> 1) & 1]), (j >> 2) & 1, abort_flag));
            if (!ok) break;
            t5_fence_after();
            const int n0 = j * kW5N;
            const bool masked = n0 + kW5N > min(kv_len, off + m0 + 1);
            const int lim = min(kv_len - 1, off + row) - n0;  // last visible column of this row inside the tile
            uint32_t r[2][32];
            t5_ld32(tS, r[0]);
            t5_ld32(tS + 32, r[1]);
            t5_wait_ld();
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (!masked) {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        mx0 = t5_max3(mx0, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
                        mx1 = t5_max3(mx1, __uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]));
                        mx2 = t5_max3(mx2, __uint_as_float(r[c][i + 4]), __uint_as_float(r[c][i + 5]));
                        mx3 = t5_max3(mx3, __uint_as_float(r[c][i + 6]), __uint_as_float(r[c][i + 7]));
                    }
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float a0 = 32 * c + i > lim ? -INFINITY : __uint_as_float(r[c][i]);
                        const float a1 = 32 * c + i + 1 > lim ? -INFINITY : __uint_as_float(r[c][i + 1]);
                        mx0 = t5_max3(mx0, a0, a1);
                    }
            }
            const float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
            // the reference the previous tile (other group) left behind
            float m_used = -INFINITY;
            if (j > 0) {
                bool seen = *seq >= j;
                if (!seen) {
                    const long long t0w = clock64();
                    while (!(seen = *seq >= j)) {
                        if (*abort_flag) break;
                        if (clock64() - t0w > kT5WaitCycles) { *abort_flag = 1; break; }
                    }
                }
                ok = __all_sync(0xffffffffu, seen);
                if (!ok) break;
                m_used = *m_pub;
            }
            const float m_new = fmaxf(m_used, tile_max);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool need = m_new - m_used > kT5RescaleThreshold;  // false while both are -inf (NaN compares false)
                if (__any_sync(0xffffffffu, need)) {
                    // O holds P.V of tiles 0 .. j-1: wait for tile j-1's on its score buffer's barrier (one phase per four
                    // tiles there, so the parity cannot be mistaken for an older phase; MMAs complete in order)
                    ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.pvdone[(j - 1) & 3]), ((j - 1) >> 2) & 1, abort_flag));
                    if (!ok) break;
                    t5_fence_after();
                    const float f = need ? exp2f(m_used - m_new) : 1.0f;
#pragma unroll 1
                    for (int c0 = 0; c0 < kW5D; c0 += 32) {
                        uint32_t o[32];
                        t5_ld32(tO + c0, o);
                        t5_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        t5_st32(tO + c0, o);
                    }
                    t5_wait_st();
                    if (need) m_used = m_new;
                }
                if (m_used == -INFINITY) m_used = m_new;
            }
            // publish: the other group's next tile may start its exponentials (and a rescale of O it needs is ordered after
            // this one by the same chain)
            *m_pub = m_used;
            __threadfence_block();
            *seq = j + 1;
            // bring this group's partial sum to the new reference
            if (m_ref != m_used) {
                l = m_ref == -INFINITY ? 0.0f : l * exp2f(m_ref - m_used);
                m_ref = m_used;
            }
            const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
            float ps0 = 0.0f, ps1 = 0.0f;
            if (!masked) {
                const uint64_t sc2 = t5_pack2(scale_log2, scale_log2), nm2 = t5_pack2(neg_m, neg_m);
                uint64_t acc_a = t5_pack2(0.0f, 0.0f), acc_b = acc_a;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t w[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float x0, x1;
                        t5_unpack2(t5_fma2(t5_pack2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1])), sc2, nm2), x0, x1);
                        const float p0 = t5_ex2(x0), p1 = t5_ex2(x1);
                        if (i & 1) acc_b = t5_add2(acc_b, t5_pack2(p0, p1)); else acc_a = t5_add2(acc_a, t5_pack2(p0, p1));
                        w[i] = t5_pack_bf16x2(p0, p1);
                    }
                    t5_st16(tS + 16 * c, w);
                }
                float a0, a1;
                t5_unpack2(t5_add2(acc_a, acc_b), a0, a1);
                ps0 = a0; ps1 = a1;
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t w[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float p0 = 32 * c + 2 * i > lim ? 0.0f : t5_ex2(fmaf(__uint_as_float(r[c][2 * i]), scale_log2, neg_m));
                        const float p1 = 32 * c + 2 * i + 1 > lim ? 0.0f : t5_ex2(fmaf(__uint_as_float(r[c][2 * i + 1]), scale_log2, neg_m));
                        ps0 += p0; ps1 += p1;
                        w[i] = t5_pack_bf16x2(p0, p1);
                    }
                    t5_st16(tS + 16 * c, w);
                }
            }
            l += ps0 + ps1;
            t5_wait_st();
            t5_fence_before();
            t5_arrive(t5_s32(&bars.pready[j & 3]));
        }
        // ---- every MMA has completed (the last P.V, hence all before it): the K ring is idle and carries the two groups'
        //      partial sums; every softmax warp reaches the barrier below, also after a timed-out wait ----
        if (ok && n_tiles > 0)
            ok = __all_sync(0xffffffffu, t5_wait(t5_s32(&bars.pvdone[(n_tiles - 1) & 3]), ((n_tiles - 1) >> 2) & 1, abort_flag));
        if (ok) {
            t5_fence_after();
            s_lpart[grp][r_local] = l;
            s_mpart[grp][r_local] = m_ref;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // ---- epilogue: group 0 writes output columns [0, 128), group 1 [128, 256) ----
        if (ok && n_tiles > 0 && !*abort_flag) {
            const float m_fin = *m_pub;  // the reference O is relative to
            float lsum = 0.0f;
#pragma unroll
            for (int gi = 0; gi < 2; ++gi) {
                const float lg = s_lpart[gi][r_local], mg = s_mpart[gi][r_local];
                if (mg != -INFINITY) lsum += lg * exp2f(mg - m_fin);
            }
            const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
            const int64_t base = ((static_cast<int64_t>(b) * q_len + row) * n_q_heads + h) * kW5D;
            const int64_t gbase = (static_cast<int64_t>(b) * q_len + row) * gate_ts + h * gate_hs;
#pragma unroll 1
            for (int c0 = grp * (kW5D / 2); c0 < (grp + 1) * (kW5D / 2); c0 += 32) {
                uint32_t o[32];
                t5_ld32(tO + c0, o);
                t5_wait_ld();
                if (row < q_len) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float x0 = __uint_as_float(o[v4 * 8 + 2 * i]) * inv, x1 = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
                            if (gate != nullptr) {
                                const uint32_t gw = *reinterpret_cast<const uint32_t *>(gate + gbase + c0 + v4 * 8 + 2 * i);
                                x0 = bf16_round(x0) * bf16_round(1.0f / (1.0f + __expf(-bf16lo(gw))));
                                x1 = bf16_round(x1) * bf16_round(1.0f / (1.0f + __expf(-bf16hi(gw))));
                            }
                            w[i] = pack_bf16(x0, x1);
                        }
                        *reinterpret_cast<uint4 *>(out + base + c0 + v4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    // ---- teardown: every thread arrives here, also after a timed-out wait ----
    if (*abort_flag) {
        if (threadIdx.x == 0) { atomicOr(err, HS_DEVERR_WAIT_TIMEOUT); atomicExch(reinterpret_cast<unsigned int *>(err + 1), launch_id); }
        const long long t0c = clock64();
        while (clock64() - t0c < 2000000LL) {}  // bounded grace period for copies and MMAs still in flight
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(512) : "memory");
}

// ---- host side --------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// [n_seqs, n_tokens, n_heads, head_dim] bf16 -> 4-D map (d, head, token, sequence), box 64 x 1 x box_rows x 1, 128-byte swizzle
static bool make_map(CUtensorMap *map, const void *base, int n_seqs, int n_tokens, int n_heads, int head_dim = kT5D, int box_rows = kT5N) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(n_heads), static_cast<cuuint64_t>(n_tokens),
                                static_cast<cuuint64_t>(n_seqs)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(n_heads) * head_dim * 2,
                                   static_cast<cuuint64_t>(n_tokens) * n_heads * head_dim * 2};
    const cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns HS_OK with *taken = 1 when this kernel took the launch, *taken = 0 when the caller should use the
// mma.sync kernel (head_dim != 128, or no tensor-map encoder in the driver).
int32_t prefill_tc5_try(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *out, const uint16_t *gate, int64_t gate_ts,
                        int64_t gate_hs, int n_seqs, int q_len, int kv_len, int n_q_heads, int n_kv_heads, int head_dim, float scale_log2,
                        cudaStream_t s, int *taken) {
    *taken = 0;
    if (q_len < 2) return HS_OK;
    if (head_dim == kW5D) {
        CUtensorMap mq, mk, mv;
        if (!make_map(&mq, q, n_seqs, q_len, n_q_heads, kW5D, kW5M) || !make_map(&mk, k, n_seqs, kv_len, n_kv_heads, kW5D, 2 * kW5N) ||
            !make_map(&mv, v, n_seqs, kv_len, n_kv_heads, kW5D, kW5N))
            return HS_OK;
        int *errw = device_error_word();
        if (!errw) return fail(HS_ERR_DEVICE, "hs_attn_prefill_causal: device error word unavailable");
        static PerDeviceState configured_w;
        const int dev = current_device();
        if (!configured_w.get(dev)) {
            cudaError_t e = cudaFuncSetAttribute(prefill_tc5_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kW5SmemBytes);
            if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_prefill_causal: %s", cudaGetErrorString(e));
            configured_w.set(dev, 1);
        }
        dim3 gridw((q_len + kW5M - 1) / kW5M, n_q_heads, n_seqs);
        prefill_tc5_wide_kernel<<<gridw, kW5Threads, kW5SmemBytes, s>>>(mq, mk, mv, out, gate, gate_ts, gate_hs, q_len, kv_len, n_q_heads, n_kv_heads, scale_log2, errw, next_launch_id());
        *taken = 1;
        return HS_OK;
    }
    if (head_dim != kT5D) return HS_OK;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, q, n_seqs, q_len, n_q_heads) || !make_map(&mk, k, n_seqs, kv_len, n_kv_heads) ||
        !make_map(&mv, v, n_seqs, kv_len, n_kv_heads))
        return HS_OK;
    int *err = device_error_word();
    if (!err) return fail(HS_ERR_DEVICE, "hs_attn_prefill_causal: device error word unavailable");
    static PerDeviceState configured;
    const int dev = current_device();
    if (!configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kT5SmemBytes);
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_prefill_causal: %s", cudaGetErrorString(e));
        configured.set(dev, 1);
    }
    dim3 grid((q_len + kT5BlockM - 1) / kT5BlockM, n_q_heads, n_seqs);
    prefill_tc5_kernel<<<grid, kT5Threads, kT5SmemBytes, s>>>(mq, mk, mv, out, gate, gate_ts, gate_hs, q_len, kv_len, n_q_heads, n_kv_heads, scale_log2, err, next_launch_id());
    *taken = 1;
    return HS_OK;
}

}  // namespace hs

