// Quantised-KV (int8, NF4, FP4) decode attention for head_dim 128, 8 kv heads, 4 query heads per kv head: a
// persistent, warp-specialised kernel.  (The int8 form is described; the 4-bit form differs only in how codes
// become fp16: one lookup per byte in a 256-entry fp16x2 table replicated per lane in shared memory.)
//
//   * two CTAs per SM (while one winds up a sequence or starts the next, the other keeps streaming); the
//     tokens of ALL sequences, cut into 16-token tiles, are divided evenly over the CTAs (flat split-KV),
//     so ragged batches balance without padding;
//   * each tile of the [tokens, kv_heads, 128] u8 cache is streamed into a 3-stage shared memory ring with
//     four bulk async copies (cp.async.bulk: K codes, V codes, K scales, V scales; each a single contiguous
//     run of 16 token rows, completion on an mbarrier).  Warp 0 works out the source addresses of 32 tiles at a
//     time; the warp that is last to finish a tile issues the copies of the tile three further on, so no warp
//     ever waits for a free stage;
//   * 8 warps: warp h owns kv head h and the 4 query heads that share it.
//     Codes are widened to fp16 with byte permutes only (the bytes become 1024 + code exactly); the
//     constant 1151 = 1024 + 127 is removed algebraically: q.(1024+c) - 1151*sum(q) and
//     p'.(1024+c) - 1151*sum(p').  q.K^T runs as mma.sync m16n8k16 with the query heads as rows, P.V with
//     the head_dim as rows (so P's accumulator registers are reused unchanged as the B operand and the
//     output accumulators are dense); fp32 accumulation; block scales applied to the fp32 scores (K) and
//     folded into P (V); online softmax in the exp2 domain with quad shuffles;
//   * each (CTA, sequence) pair writes one normalised partial + log-sum-exp; the merge kernel combines.
//
// Replaces, for the q_len == 1 path, cache.get() (full-history dequantise, kv_cache.rs:1499-1643) + GQA
// expansion (llama.rs:847-872) + compute_attention_masked (llama.rs:1023-1119) + the padding/mask of
// forward_batched (llama.rs:787-826,2540-2572).
//
// Every wait on an mbarrier is bounded; on expiry the CTA records HS_DEVERR_WAIT_TIMEOUT and winds down.
#include <cuda_fp16.h>

#include "hs_common.cuh"
#include "quant_dev.cuh"

namespace hs {

constexpr int kTcConsumers = 8;       // every warp consumes; whichever finishes a tile last refills its stage
constexpr int kTcThreads = kTcConsumers * 32;
constexpr int kTcPadUnits = 12;       // partition: cost of starting a sequence, in eighths of a tile (measured: 10-20 are alike)
#ifndef HS_TC_APPEND_UNITS
#define HS_TC_APPEND_UNITS 10
#endif
constexpr int kTcAppendUnits = HS_TC_APPEND_UNITS;  // ... and of writing a sequence's new token before its last tile is streamed
constexpr int kTcMaxSeqs = 512;       // tile-count prefix and lengths kept in shared memory (half as many for the head_dim 256 shape)
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
// counts an arrival in shared memory (release: this warp's reads of the stage are done; acquire: the warp that
// arrives last has seen everyone else's) and returns the count before it
__device__ __forceinline__ uint32_t smem_arrive_count(uint32_t addr) {
    uint32_t prev;
    asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(prev) : "r"(addr) : "memory");
    return prev;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// The cache is read once per step: its copies carry an evict-first L2 policy so that they do not push the partials
// (written early, read back by the merge) out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
// D += A.B, m16n8k16, fp16 operands, fp32 accumulate.  A rows 8..15 unused (a1 = a3 = 0).
__device__ __forceinline__ void mma_rows8(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two u8 codes (the bytes `selector` picks from w) -> fp16x2 of (1024 + code), exact
__device__ __forceinline__ uint32_t codes_biased_h2(uint32_t w, uint32_t selector) { return __byte_perm(w, 0x64646464u, selector); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float h2_sum(uint32_t w) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    return f.x + f.y;
}
__device__ __forceinline__ float clamp_h(float x) { return fminf(fmaxf(x, -65504.0f), 65504.0f); }
// 4-bit caches: the fp16x2 pair of code byte `k` (0..3) of word `w`, from the byte -> fp16x2 table replicated per lane in
// shared memory (`lut_lane` = shared address of this lane's column, entries 128 bytes apart): one byte permute, one
// multiply-add for the address, one shared load
__device__ __forceinline__ uint32_t lut_pair(uint32_t lut_lane, uint32_t w, uint32_t k) {
    const uint32_t byte = __byte_perm(w, 0u, 0x4440u | k);
    uint32_t v;
    asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(byte * 128u + lut_lane));
    return v;
}

// FOURBIT = false: u8 codes (128 B per head row).  FOURBIT = true: NF4 / FP4 codes (64 B per head row), widened through a
// 256-entry byte -> fp16x2 table replicated per lane (bank-conflict-free lookups).
//
// Two shapes share the kernel.  A token row of codes is cut into "lanes of 128": WIDE = false is 8 kv heads of
// head_dim 128 with 4 query heads each (one warp per kv head, 16-token tiles); WIDE = true is 2 kv heads of head_dim 256
// with 8 query heads each: a kv head is two 128-wide halves, a warp owns one half of one head for 16 of the tile's 32
// tokens, and the two warps of a head add their halves of q.k through shared memory before the softmax.  BPR counts the
// scale blocks of one 128-wide half.
template <bool FOURBIT, int BPR, bool SF16, bool WIDE>
struct TcLayout {
    static constexpr int kVH = WIDE ? 4 : 8;                     // 128-wide halves ("virtual heads") per token row
    static constexpr int kSplit = WIDE ? 2 : 1;                  // halves per kv head
    static constexpr int kG = WIDE ? 8 : 4;                      // query heads per kv head
    static constexpr int kTH = kTcConsumers / kVH;               // 16-token groups per tile, one warp each per half
    static constexpr int kTile = 16 * kTH;                       // tokens per stage
    static constexpr int kD = 128 * kSplit;                      // head_dim
    static constexpr int kHq = kVH / kSplit * kG;                // query heads
    static constexpr int kStages = FOURBIT ? 4 : 3;
    static constexpr int kHeadRow = FOURBIT ? 64 : 128;          // code bytes of one (token, half) row
    static constexpr int kRow = kVH * kHeadRow;                  // bytes of one token row of codes
    static constexpr int kSRow = kVH * BPR * (SF16 ? 2 : 4);     // scale bytes per token
    static constexpr int kKOff = 0;
    static constexpr int kVOff = kTile * kRow;
    static constexpr int kKsOff = 2 * kTile * kRow;
    static constexpr int kVsOff = kKsOff + kTile * kSRow;
    static constexpr int kStage = (kVsOff + kTile * kSRow + 127) / 128 * 128;
    static constexpr int kBarOff = kStages * kStage;
    static constexpr int kXBarOff = kBarOff + 2 * kStages * 8 + 16;    // 4 mbarriers: score exchange of a warp pair (WIDE)
    static constexpr int kMaxSeqs = WIDE ? kTcMaxSeqs / 2 : kTcMaxSeqs;  // (the head_dim 256 shape also holds the exchange buffers)
    static constexpr int kPrefOff = kXBarOff + 32;                     // int tile-count prefix [kMaxSeqs + 1]
    static constexpr int kLenOff = kPrefOff + (kMaxSeqs + 4) * 4;      // int clamped lengths [kMaxSeqs]
    static constexpr int kDescOff = kLenOff + kMaxSeqs * 4;            // uint64 [64 tiles][4 tables]: source addresses of the next tiles
    static constexpr int kXOff = (kDescOff + 64 * 4 * 8 + 127) / 128 * 128;  // float [4 pairs][2 parities][2 warps][32 lanes][4] (WIDE)
    static constexpr int kLutOff = kXOff + (WIDE ? 4 * 2 * 2 * 512 : 0);        // uint32 [256][32] (4-bit kinds only)
    static constexpr int kTotal = kLutOff + (FOURBIT ? 256 * 32 * 4 : 0);
    static constexpr uint32_t kTxBytes = 2u * kTile * kRow + 2u * kTile * kSRow;
    static_assert(kDescOff % 16 == 0, "tile addresses are stored 16 bytes at a time");
    // two CTAs per SM (228 KB, 1 KB reserved per CTA, 128 B of static shared memory) for every layout but the head_dim 256
    // shape with block 64 and f32 scales, which runs one CTA per SM
    static_assert((WIDE && BPR == 2 && !SF16) || 2 * (kTotal + 1024 + 128) <= 228 * 1024, "two CTAs per SM");
};

// Outputs of the merge that runs inside the kernel after a grid-wide barrier (cooperative launch only).
struct TcMergeArgs {
    uint16_t *out;        // bf16 [n_seqs, Hq, 128] or NULL
    const uint16_t *gate; // optional
    float *o_shard, *lse_shard;  // optional fp32 shard outputs
    int counter;          // which grid-barrier counter the launch uses: one per grid size (CTAs per SM - 1)
    int fine_items;       // merge work items of one query head instead of 512 / D (set when the batch gives the grid too few items)
    int after_write;      // launched as a programmatic dependent of the quantise-on-write kernel: wait for it before the first cache read
    AppendArgs append;    // k_new != NULL: the kernel writes the step's new token of every sequence itself (u8 caches)
    ShardArgs shard;      // world > 0: the merged result is a KV-length shard's; exchange it with the other GPUs and merge again
};

// ---- peer exchange primitives: {value, epoch} words on peer-mapped memory, ordinary 8- and 16-byte stores and loads ----
__device__ __forceinline__ void st_word(unsigned long long *p, float v, unsigned int epoch) {
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ void st_word2(unsigned long long *p, float v0, float v1, unsigned int epoch) {  // two adjacent words, 16-byte aligned
    asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(v0)), "r"(epoch), "r"(__float_as_uint(v1)), "r"(epoch)
                 : "memory");
}
__device__ __forceinline__ uint2 ld_word(const unsigned long long *p) {
    uint2 w;
    asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ uint4 ld_word2(const unsigned long long *p) {  // each 8-byte half is delivered whole; the two halves are checked separately
    uint4 w;
    asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(p) : "memory");
    return w;
}

// Arrivals of all launches so far (see the grid barrier in the kernel), one counter per grid size: a launch's CTAs
// find their target from their ticket and the grid size, so every launch that shares a counter must have the same one.
// INVARIANT: the tickets of two launches on one device must not interleave, i.e. two launches of this kernel must not be
// in flight on a device at the same time.  Launches on one stream are ordered by the stream.  Launches on different
// streams (or from different host threads) of one device must be serialised by the caller; include/hs_attn.h says so
// at hs_attn_decode.  Nothing in the library depends on "a full cooperative grid leaves no room for a second one".
// If the rule is broken, the bounded wait turns it into HS_DEVERR_WAIT_TIMEOUT and an undefined result, not into a hang.
__device__ unsigned long long g_tc_barrier[2];

template <bool FOURBIT, int BPR, bool SF16, bool WIDE>
__global__ void __launch_bounds__(kTcThreads, 2)
decode_int8_tc_kernel(ViewDev view, const uint16_t *__restrict__ q, const int32_t *__restrict__ seq_lens, int n_seqs,
                      int n_q_heads, float kmul, float *__restrict__ o_part, float *__restrict__ lse_part,
                      int *__restrict__ err, TcMergeArgs mg) {
    using LT = TcLayout<FOURBIT, BPR, SF16, WIDE>;
    constexpr int kTcStages = LT::kStages;
    constexpr int kTcTile = LT::kTile, kTcG = LT::kG, kD = LT::kD;
    extern __shared__ __align__(128) unsigned char smem[];
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + LT::kBarOff + 2 * kTcStages * 8);
    int *s_pref = reinterpret_cast<int *>(smem + LT::kPrefOff);
    int *s_len = reinterpret_cast<int *>(smem + LT::kLenOff);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + LT::kBarOff;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cap = view.page_tokens * view.pages_per_seq;

    // ---- tile counts of all sequences (one coalesced pass), exclusive prefix by warp 0 ----
    bool over = false;
    for (int i = threadIdx.x; i < n_seqs; i += kTcThreads) {
        const int L = seq_lens[i];
        over |= L > cap;
        s_len[i] = min(max(L, 0), cap);
        s_pref[i + 1] = (s_len[i] + kTcTile - 1) / kTcTile;
    }
    if (over && blockIdx.x == 0) atomicOr(err, HS_DEVERR_DECODE_RANGE);
    const uint32_t lut_lane = smem_u32(smem + LT::kLutOff) + 4u * lane;  // this lane's column of the table; entry of byte x at + 128 x
    if constexpr (FOURBIT) {
        // byte -> (table[high nibble], table[low nibble]) as fp16x2, low half = the even (first) element
        const float *tab = view.kind == HS_KV_NF4 ? c_nf4 : c_fp4;
        uint32_t *lut = reinterpret_cast<uint32_t *>(smem + LT::kLutOff);
        for (int i = threadIdx.x; i < 256 * 32; i += kTcThreads) lut[i] = pack_h2(tab[(i >> 5) >> 4], tab[(i >> 5) & 15]);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            *reinterpret_cast<unsigned long long *>(smem + LT::kBarOff + (kTcStages + s) * 8) = 0ULL;  // arrival count of the stage
        }
        mbar_init(bar_full + 2 * kTcStages * 8 + 8, 1);  // the merge's staging barrier
        if constexpr (WIDE)
            for (int i = 0; i < 4; ++i) mbar_init(smem_base + LT::kXBarOff + 8 * i, 2);  // one arrival per warp of the pair
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < n_seqs; base += 32) {
            const int i = base + lane;
            const int v = i < n_seqs ? s_pref[i + 1] : 0;
            int inc = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, off);
                if (lane >= off) inc += t;
            }
            if (i < n_seqs) s_pref[i + 1] = carry + inc;
            carry += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_pref[0] = 0;
    }
    __syncthreads();
    const int64_t total = s_pref[n_seqs];
    // ---- weighted flat partition ----
    // Tiles are laid out on a virtual axis, 8 units per tile, with kTcPadUnits empty units in front of every sequence:
    // a CTA whose range crosses into another sequence pays for a second partial, a second set of query fragments and a
    // cold restart, and the empty units give it that much less streaming to do.  The axis is cut evenly.  Never more
    // working CTAs than tiles, so that every CTA has at least 8 units and no CTA inside a sequence's span comes out empty.
    const int64_t cta = blockIdx.x;
    const int64_t n_ctas = total < static_cast<int64_t>(gridDim.x) ? (total > 0 ? total : 1) : static_cast<int64_t>(gridDim.x);
    // (when the kernel also writes the step's new tokens, the CTA that ends a sequence pays for that too: a wider gap)
    const int pad_units = kTcPadUnits + (mg.append.k_new != nullptr ? kTcAppendUnits : 0);
    const int64_t vtotal = 8 * total + static_cast<int64_t>(pad_units) * n_seqs;
    const bool small = vtotal * n_ctas < (1LL << 32);  // 32-bit divisions when they are exact
    auto vbegin = [&](int64_t c) -> int64_t {  // first virtual unit of CTA c
        return small ? static_cast<int64_t>(static_cast<uint32_t>(vtotal) * static_cast<uint32_t>(c) / static_cast<uint32_t>(n_ctas)) : vtotal * c / n_ctas;
    };
    auto tiles_before = [&](int64_t v) -> int {  // tiles whose first unit lies before virtual unit v
        if (v >= vtotal) return static_cast<int>(total);
        int lo = 0, hi = n_seqs;  // invariant: start(lo) <= v < start(hi), start(r) = 8 s_pref[r] + pad r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (8LL * s_pref[mid] + static_cast<int64_t>(pad_units) * mid <= v) lo = mid; else hi = mid;
        }
        const int64_t off = v - (8LL * s_pref[lo] + static_cast<int64_t>(pad_units) * lo) - pad_units;
        int64_t k = off <= 0 ? 0 : (off + 7) >> 3;
        const int64_t nt = s_pref[lo + 1] - s_pref[lo];
        if (k > nt) k = nt;
        return s_pref[lo] + static_cast<int>(k);
    };
    const int t_begin = cta < n_ctas ? tiles_before(vbegin(cta)) : 0, t_end = cta < n_ctas ? tiles_before(vbegin(cta + 1)) : 0;
    const bool has_work = t_begin < t_end;
    // first sequence of this CTA: the largest r with s_pref[r] <= t_begin
    int r_first = n_seqs;
    if (has_work) {
        int lo = 0, hi = n_seqs;  // invariant: s_pref[lo] <= t_begin < s_pref[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_pref[mid] <= t_begin) lo = mid; else hi = mid;
        }
        r_first = lo;
    }

    // ---- feeding the ring ----
    // Where a tile's rows lie (sequence, page, offset in the page -> four source addresses: K codes, V codes, K scales,
    // V scales) is worked out by warp 0 for 32 tiles at a time, one tile per lane, and parked in shared memory (64
    // slots: the batch being written never overlaps one still in use).  Nobody waits for a ring stage to become free:
    // every warp counts its arrival when it is done with a tile, and the warp that arrives last (all eight have then
    // read the stage) issues the copies of the tile three (four) further on into it - one 8-byte shared load and one
    // bulk copy per issuing lane.
    const int n_tiles_cta = has_work ? t_end - t_begin : 0;
    unsigned long long *s_desc = reinterpret_cast<unsigned long long *>(smem + LT::kDescOff);
    const uint32_t stage_count = smem_base + LT::kBarOff + kTcStages * 8;  // uint32 arrival counts, 8 bytes apart, never reset
    const uint64_t stream_policy = l2_evict_first_policy();
    auto fill_desc = [&](int p_base) {  // all lanes of warp 0: the addresses of tiles p_base .. p_base + 31 of this CTA
        const int p = p_base + lane;
        if (p < n_tiles_cta) {
            const int T = t_begin + p;
            int lo = r_first, hi = n_seqs;  // invariant: s_pref[lo] <= T < s_pref[hi]; ends at the sequence that owns tile T
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_pref[mid] <= T) lo = mid; else hi = mid;
            }
            const int t0 = (T - s_pref[lo]) * kTcTile;
            const int page = t0 / view.page_tokens;
            const int64_t in_page = t0 - page * view.page_tokens;
            const int64_t pidx = static_cast<int64_t>(lo) * view.pages_per_seq + page;
            const unsigned char *pk = reinterpret_cast<const unsigned char *>(view.k_pages[pidx]);
            const unsigned char *pv = reinterpret_cast<const unsigned char *>(view.v_pages[pidx]);
            const unsigned char *pks = reinterpret_cast<const unsigned char *>(view.k_scale_pages[pidx]);
            const unsigned char *pvs = reinterpret_cast<const unsigned char *>(view.v_scale_pages[pidx]);
            ulonglong2 *d = reinterpret_cast<ulonglong2 *>(s_desc + 4 * (p & 63));
            d[0] = make_ulonglong2(reinterpret_cast<unsigned long long>(pk + in_page * LT::kRow), reinterpret_cast<unsigned long long>(pv + in_page * LT::kRow));
            d[1] = make_ulonglong2(reinterpret_cast<unsigned long long>(pks + in_page * LT::kSRow), reinterpret_cast<unsigned long long>(pvs + in_page * LT::kSRow));
        }
        __threadfence_block();  // the warp that issues such a tile is ordered after this by warp 0's later arrival counts
        __syncwarp();
    };
    // the copies of this CTA's tile p into ring stage `stage` (all lanes of the calling warp)
    auto issue_tile = [&](int p, int stage) {
        if (lane < 4) {
            const unsigned char *src = reinterpret_cast<const unsigned char *>(s_desc[4 * (p & 63) + lane]);
            const uint32_t full = bar_full + 8 * stage;
            const uint32_t sbase = smem_base + stage * LT::kStage;
            if (lane == 0) mbar_expect_tx(full, LT::kTxBytes);
            __syncwarp(0xfu);
            if (lane < 2)
                bulk_g2s_hint(sbase + (lane ? LT::kVOff : LT::kKOff), src, kTcTile * LT::kRow, full, stream_policy);
            else
                bulk_g2s_hint(sbase + (lane == 2 ? LT::kKsOff : LT::kVsOff), src, kTcTile * LT::kSRow, full, stream_policy);
        }
        __syncwarp();
    };
    // Programmatic dependent launch: this grid may have started while the quantise-on-write kernel of the same step still
    // runs (its launch latency and everything above - lengths, prefix, partition - overlap with it); the cache itself must
    // not be read before that kernel has completed.  Every thread waits, because any warp may issue a tile's copies later.
    if (mg.after_write) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ---- the step's new tokens (LayerKVCache::update fused into the attention launch, kv_cache.rs:1275-1496) ----
    // The token of sequence r sits at position L_r - 1, in the sequence's last tile; the CTA that owns that tile quantises the
    // token's K and V rows into the cache - same arithmetic, same codes and scales as the write kernel - before the tile's
    // copies are issued: ordinary stores, a proxy fence, a block barrier, then the bulk copies may read them.  A thread takes
    // 8 consecutive elements (threads [0, Hkv*D/8) the K row, the next Hkv*D/8 the V row).  Where the CTA's first ring-full
    // of tiles does not contain such a tile, the write runs after those copies are issued, under their latency.
    bool append_pending = false, append_early = false;
    if constexpr (!FOURBIT) {
        if (mg.append.k_new != nullptr && has_work)
            for (int r = r_first; r < n_seqs && s_pref[r] < t_end; ++r) {
                const int last = s_pref[r + 1] - 1;
                if (s_pref[r + 1] == s_pref[r] || last < t_begin || last >= t_end) continue;
                append_pending = true;
                append_early |= last - t_begin < kTcStages;
            }
    }
    auto write_new_tokens = [&]() {  // all threads; CTA-uniform control flow
        if constexpr (!FOURBIT) {
            const int H = view.n_kv_heads, cpt = H * kD / 8;                   // 8-element chunks per K (or V) row of a token
            const bool is_v = static_cast<int>(threadIdx.x) >= cpt;
            const int chunk = static_cast<int>(threadIdx.x) - (is_v ? cpt : 0);
            const bool lane_live = chunk < cpt;
            const int hh = lane_live ? chunk / (kD / 8) : 0, d0 = lane_live ? (chunk % (kD / 8)) * 8 : 0;
            const int tpb = view.block / 8, bpr = kD / view.block;
            for (int r = r_first; r < n_seqs && s_pref[r] < t_end; ++r) {
                const int last = s_pref[r + 1] - 1;                               // the sequence's last tile
                if (s_pref[r + 1] == s_pref[r] || last < t_begin || last >= t_end) continue;
                const int pos = s_len[r] - 1;
                const int page = pos / view.page_tokens;
                const bool rope = !is_v && mg.append.sin != nullptr;
                bool okw = lane_live;
                if (rope && pos >= mg.append.n_positions) { okw = false; if (lane_live && chunk == 0) atomicOr(err, HS_DEVERR_KV_WRITE_RANGE); }
                float x[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                const uint16_t *src = (is_v ? mg.append.v_new : mg.append.k_new) + (static_cast<int64_t>(r) * H + hh) * kD;
                if (okw) load_row8_rope(src, d0, rope ? mg.append.sin : nullptr, mg.append.cos, pos, mg.append.rotary_dim, x);
                int c[8];
                const float a = quantize_n<HS_KV_INT8, 8>(x, tpb, view.scale_dtype, nullptr, c);  // (every lane takes part in the shuffles)
                if (!okw) continue;
                const int64_t pidx = static_cast<int64_t>(r) * view.pages_per_seq + page;
                const int64_t in_page = static_cast<int64_t>(pos - page * view.page_tokens) * H + hh;
                uint8_t *codes = reinterpret_cast<uint8_t *>((is_v ? view.v_pages : view.k_pages)[pidx]);
                void *scales = (is_v ? view.v_scale_pages : view.k_scale_pages)[pidx];
                if ((d0 & (view.block - 1)) == 0) store_scale(scales, in_page * bpr + d0 / view.block, view.scale_dtype, a);
                store_codes8<HS_KV_INT8>(codes, in_page * kD + d0, in_page * kD + d0 + 8, c, true);
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            __syncthreads();
        }
    };
    if (append_pending && append_early) write_new_tokens();
    bool ok = true;
    if (warp == 0 && has_work) {  // fill the ring before anything else touches global memory
        fill_desc(0);
        for (int p = 0; p < n_tiles_cta && p < kTcStages; ++p) issue_tile(p, p);
    }

    if (append_pending && !append_early) write_new_tokens();  // (under the latency of the copies just issued)

    // ================================ consumer warps ================================
    // warp -> (128-wide half `head` of the token row, 16-token group `th` of the tile); `kvh`, `half`: the kv head and
    // which half of its head_dim this warp owns
    const int head = warp % LT::kVH, th = warp / LT::kVH;
    const int kvh = head / LT::kSplit, half = head % LT::kSplit;
    const int g = lane >> 2, j = lane & 3;
    float *x_mine = nullptr;
    const float *x_peer = nullptr;
    uint32_t x_bar = 0;
    if constexpr (WIDE) {  // exchange buffers of the pair (this warp, the warp owning the other half of the head)
        const int pair = th * (LT::kVH / 2) + kvh;
        float *xb = reinterpret_cast<float *>(smem + LT::kXOff) + pair * 2 * 2 * 128;  // [parity][warp of pair][lane][4]
        x_mine = xb + half * 128 + lane * 4;
        x_peer = xb + (half ^ 1) * 128 + lane * 4;
        x_bar = smem_base + LT::kXBarOff + 8 * pair;
    }
    const float vmul = FOURBIT ? 1.0f : 1.0f / 127.0f;  // u8 codes are (code - 127): the 1/127 of the codebook goes here
    int it = 0, c_stage = 0;
    uint32_t c_par = 0;  // ring stage and barrier parity of tile `it`
    int pair_it = 0;  // tiles this warp pair has exchanged scores for (WIDE)
    (void)pair_it;
    for (int r = r_first; r < n_seqs && s_pref[r] < t_end && ok; ++r) {
        const int base = s_pref[r];
        const int lo = max(t_begin, base), hi = min(t_end, s_pref[r + 1]);
        if (lo >= hi) continue;
        const int L = s_len[r];

        // ---- query fragments: fp16, d permuted so that one 16-byte K load feeds 4 k-steps; per-block sums ----
        uint32_t qa[2][4][2];
        float qsum[2] = {0.0f, 0.0f};
        if (g < kTcG) {
            const uint16_t *qp = q + (static_cast<int64_t>(r) * n_q_heads + kvh * kTcG + g) * kD + half * 128;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const uint4 w0 = *reinterpret_cast<const uint4 *>(qp + 64 * b + 16 * j);
                const uint4 w1 = *reinterpret_cast<const uint4 *>(qp + 64 * b + 16 * j + 8);
                const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    qa[b][s][0] = pack_h2(clamp_h(bf16lo(ww[2 * s])), clamp_h(bf16hi(ww[2 * s])));
                    qa[b][s][1] = pack_h2(clamp_h(bf16lo(ww[2 * s + 1])), clamp_h(bf16hi(ww[2 * s + 1])));
                    if constexpr (!FOURBIT) qsum[b] += h2_sum(qa[b][s][0]) + h2_sum(qa[b][s][1]);  // (4-bit table values carry no bias)
                }
            }
        } else {
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int s = 0; s < 4; ++s) qa[b][s][0] = qa[b][s][1] = 0u;
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            qsum[b] += __shfl_xor_sync(0xffffffffu, qsum[b], 1);
            qsum[b] += __shfl_xor_sync(0xffffffffu, qsum[b], 2);
            qsum[b] *= FOURBIT ? 0.0f : 1151.0f;  // the 4-bit table values carry no bias
        }
        // pull the next sequence's query rows towards L1 now, so that the segment switch does not wait on L2
        if (g < kTcG) {
            for (int r2 = r + 1; r2 < n_seqs && s_pref[r2] < t_end; ++r2)
                if (s_pref[r2 + 1] > s_pref[r2]) {
                    const uint16_t *qn = q + (static_cast<int64_t>(r2) * n_q_heads + kvh * kTcG + g) * kD + half * 128 + 16 * j;
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(qn));
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(qn + 64));
                    break;
                }
        }
        // running softmax state of query head g (row layout of the q.K^T accumulators)
        float m = -INFINITY, l_part = 0.0f, ps_part[2] = {0.0f, 0.0f};
        // O^T accumulators: tile (b, mt): rows d = 64b + 8g + 4*(mt>>1) + 2*(mt&1) (+1 for regs 2,3), cols heads 2j, 2j+1
        float O[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.0f;

        for (int tile = lo - base; tile < hi - base; ++tile, ++it) {
            const int stage = c_stage;
            // the next batch of tile addresses, half a batch before its first tile is issued
            if (warp == 0 && it >= 16 && ((it - 16) & 31) == 0 && it + 16 < n_tiles_cta) fill_desc(it + 16);
            ok = mbar_wait(bar_full + 8 * stage, c_par, abort_flag);
            if (!ok) break;
            if (++c_stage == kTcStages) { c_stage = 0; c_par ^= 1u; }
            const unsigned char *sK = smem + stage * LT::kStage + LT::kKOff;
            const unsigned char *sV = smem + stage * LT::kStage + LT::kVOff;
            const unsigned char *sKs = smem + stage * LT::kStage + LT::kKsOff;
            const unsigned char *sVs = smem + stage * LT::kStage + LT::kVsOff;
            const int tl0 = 16 * th;
            {
                // ---- S = q.(1024 + K)^T for 16 tokens (two n-tiles of 8), one accumulator per 64-wide d block ----
                float sacc[2][2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int b = 0; b < 2; ++b) sacc[nt][b][0] = sacc[nt][b][1] = sacc[nt][b][2] = sacc[nt][b][3] = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    if constexpr (!FOURBIT) {
                        const unsigned char *krow = sK + (tl0 + nt * 8 + g) * LT::kRow + head * 128 + 16 * j;
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            const uint4 kv = *reinterpret_cast<const uint4 *>(krow + 64 * b);
                            const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                            for (int s = 0; s < 4; ++s)
                                mma_rows8(sacc[nt][b], qa[b][s][0], qa[b][s][1], codes_biased_h2(kw[s], 0x4140), codes_biased_h2(kw[s], 0x4342));
                        }
                    } else {
                        // 16 codes = 8 bytes per (block, lane); byte 2s holds d = 4s, 4s+1 and byte 2s+1 holds d = 4s+2, 4s+3
                        const unsigned char *krow = sK + (tl0 + nt * 8 + g) * LT::kRow + head * 64 + 8 * j;
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            const uint2 kv = *reinterpret_cast<const uint2 *>(krow + 32 * b);
#pragma unroll
                            for (int s = 0; s < 4; ++s) {
                                const uint32_t w = s < 2 ? kv.x : kv.y;
                                const uint32_t b0 = lut_pair(lut_lane, w, 2 * (s & 1)), b1 = lut_pair(lut_lane, w, 2 * (s & 1) + 1);
                                mma_rows8(sacc[nt][b], qa[b][s][0], qa[b][s][1], b0, b1);
                            }
                        }
                    }
                }
                // ---- scales of this thread's 4 tokens, scores in the exp2 domain, masking ----
                float p[2][2], pv[2][2][2];
                bool vld[2][2];
                float mx = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tl = tl0 + nt * 8 + 2 * j + e;
                        const bool valid = tile * kTcTile + tl < L;
                        vld[nt][e] = valid;
                        float ks[2], vs[2];
                        if (SF16) {
                            const __half *kp = reinterpret_cast<const __half *>(sKs) + (tl * LT::kVH + head) * BPR;
                            const __half *vp = reinterpret_cast<const __half *>(sVs) + (tl * LT::kVH + head) * BPR;
                            ks[0] = __half2float(kp[0]); vs[0] = __half2float(vp[0]);
                            ks[1] = BPR == 2 ? __half2float(kp[BPR - 1]) : ks[0];
                            vs[1] = BPR == 2 ? __half2float(vp[BPR - 1]) : vs[0];
                        } else {
                            const float *kp = reinterpret_cast<const float *>(sKs) + (tl * LT::kVH + head) * BPR;
                            const float *vp = reinterpret_cast<const float *>(sVs) + (tl * LT::kVH + head) * BPR;
                            ks[0] = kp[0]; vs[0] = vp[0];
                            ks[1] = BPR == 2 ? kp[BPR - 1] : ks[0];
                            vs[1] = BPR == 2 ? vp[BPR - 1] : vs[0];
                        }
                        const float s2 = ((sacc[nt][0][e] - qsum[0]) * ks[0] + (sacc[nt][1][e] - qsum[1]) * ks[1]) * kmul;
                        p[nt][e] = (valid || WIDE) ? s2 : -INFINITY;  // (WIDE: masked after the halves are added)
                        pv[nt][e][0] = valid ? vs[0] * vmul : 0.0f;
                        pv[nt][e][1] = valid ? vs[1] * vmul : 0.0f;
                        if constexpr (!WIDE) mx = fmaxf(mx, p[nt][e]);
                    }
                if constexpr (WIDE) {
                    // q.k over head_dim 256 = this warp's half + the peer's: swap through shared memory (two buffers by
                    // tile parity; the pair's mbarrier flips once per tile, one arrival per warp)
                    const int par = pair_it & 1;
                    *reinterpret_cast<float4 *>(x_mine + par * 256) = make_float4(p[0][0], p[0][1], p[1][0], p[1][1]);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_bar);
                    ok = mbar_wait(x_bar, par, abort_flag);
                    if (!ok) break;
                    const float4 o4 = *reinterpret_cast<const float4 *>(x_peer + par * 256);
                    ++pair_it;
                    p[0][0] = vld[0][0] ? p[0][0] + o4.x : -INFINITY;
                    p[0][1] = vld[0][1] ? p[0][1] + o4.y : -INFINITY;
                    p[1][0] = vld[1][0] ? p[1][0] + o4.z : -INFINITY;
                    p[1][1] = vld[1][1] ? p[1][1] + o4.w : -INFINITY;
                    mx = fmaxf(fmaxf(p[0][0], p[0][1]), fmaxf(p[1][0], p[1][1]));
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
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
                    // the O^T accumulators hold heads 2j, 2j+1: fetch their factors from the lanes whose row is that head
                    const float c0 = __shfl_sync(0xffffffffu, corr, 8 * j), c1 = __shfl_sync(0xffffffffu, corr, 8 * j + 4);
#pragma unroll
                    for (int i = 0; i < 8; ++i) { O[i][0] *= c0; O[i][1] *= c1; O[i][2] *= c0; O[i][3] *= c1; }
                    ps_part[0] *= corr; ps_part[1] *= corr;
                }
                // ---- O^T += (1024 + V)^T . P'^T, the V block scale folded into P' ----
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const uint32_t b0 = pack_h2(p[0][0] * pv[0][0][b], p[0][1] * pv[0][1][b]);
                    const uint32_t b1 = pack_h2(p[1][0] * pv[1][0][b], p[1][1] * pv[1][1][b]);
                    if constexpr (!FOURBIT) ps_part[b] += h2_sum(b0) + h2_sum(b1);
                    if constexpr (!FOURBIT) {
                        uint2 x[2][2];
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                x[nt][e] = *reinterpret_cast<const uint2 *>(sV + (tl0 + nt * 8 + 2 * j + e) * LT::kRow + head * 128 + 64 * b + 8 * g);
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const uint32_t A0 = k ? x[0][0].y : x[0][0].x, B0 = k ? x[0][1].y : x[0][1].x;
                            const uint32_t A1 = k ? x[1][0].y : x[1][0].x, B1 = k ? x[1][1].y : x[1][1].x;
                            const uint32_t t01 = __byte_perm(A0, B0, 0x5140), t23 = __byte_perm(A0, B0, 0x7362);
                            const uint32_t u01 = __byte_perm(A1, B1, 0x5140), u23 = __byte_perm(A1, B1, 0x7362);
                            mma_full(O[4 * b + 2 * k + 0], codes_biased_h2(t01, 0x4140), codes_biased_h2(t01, 0x4342),
                                     codes_biased_h2(u01, 0x4140), codes_biased_h2(u01, 0x4342), b0, b1);
                            mma_full(O[4 * b + 2 * k + 1], codes_biased_h2(t23, 0x4140), codes_biased_h2(t23, 0x4342),
                                     codes_biased_h2(u23, 0x4140), codes_biased_h2(u23, 0x4342), b0, b1);
                        }
                    } else {
                        // this lane's 8 values d = 64b + 8g .. +7 of a token are 4 bytes; byte k holds d = 8g + 2k (row g of
                        // m-tile k) and 8g + 2k + 1 (row g + 8)
                        uint32_t x[2][2];
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                x[nt][e] = *reinterpret_cast<const uint32_t *>(sV + (tl0 + nt * 8 + 2 * j + e) * LT::kRow + head * 64 + 32 * b + 4 * g);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t la = lut_pair(lut_lane, x[0][0], k), lb = lut_pair(lut_lane, x[0][1], k);
                            const uint32_t lc = lut_pair(lut_lane, x[1][0], k), ld = lut_pair(lut_lane, x[1][1], k);
                            mma_full(O[4 * b + k], __byte_perm(la, lb, 0x5410), __byte_perm(la, lb, 0x7632), __byte_perm(lc, ld, 0x5410),
                                     __byte_perm(lc, ld, 0x7632), b0, b1);
                        }
                    }
                }
            }
            __syncwarp();
            uint32_t before = 0;
            if (lane == 0) before = smem_arrive_count(stage_count + 8 * stage);
            before = __shfl_sync(0xffffffffu, before, 0);
            if ((before & (kTcConsumers - 1)) == kTcConsumers - 1 && it + kTcStages < n_tiles_cta) issue_tile(it + kTcStages, stage);
        }
        if (!ok) break;
        // ---- partial of this (CTA, sequence) pair ----
        float l = l_part;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            ps_part[b] += __shfl_xor_sync(0xffffffffu, ps_part[b], 1);
            ps_part[b] += __shfl_xor_sync(0xffffffffu, ps_part[b], 2);
            ps_part[b] *= FOURBIT ? 0.0f : 1151.0f;
        }
        // per-head values (row layout: lane 4*head') -> the lanes that hold heads 2j, 2j+1 in their accumulators
        const float l0 = __shfl_sync(0xffffffffu, l, 8 * j), l1 = __shfl_sync(0xffffffffu, l, 8 * j + 4);
        float c0[2], c1[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            c0[b] = __shfl_sync(0xffffffffu, ps_part[b], 8 * j);
            c1[b] = __shfl_sync(0xffffffffu, ps_part[b], 8 * j + 4);
        }
        const int64_t slot = (cta + r) * LT::kTH + th;
        if (2 * j < kTcG) {
            const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
            // this thread owns, for heads 2j and 2j+1 and each block b, the 8 consecutive outputs d = 64b + 8g .. +7:
            // two 16-byte stores each (whole 32-byte sectors)
            float *op0 = o_part + (slot * n_q_heads + kvh * kTcG + 2 * j) * kD + half * 128 + 8 * g;
            float *op1 = op0 + kD;
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const float *a = O[4 * b + 2 * hf], *c = O[4 * b + 2 * hf + 1];
                    *reinterpret_cast<float4 *>(op0 + 64 * b + 4 * hf) =
                        make_float4((a[0] - c0[b]) * inv0, (a[2] - c0[b]) * inv0, (c[0] - c0[b]) * inv0, (c[2] - c0[b]) * inv0);
                    *reinterpret_cast<float4 *>(op1 + 64 * b + 4 * hf) =
                        make_float4((a[1] - c1[b]) * inv1, (a[3] - c1[b]) * inv1, (c[1] - c1[b]) * inv1, (c[3] - c1[b]) * inv1);
                }
        }
        if (g < kTcG && j == 0 && half == 0)
            lse_part[slot * n_q_heads + kvh * kTcG + g] = l > 0.0f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
    if (!ok) {
        // a wait ran out: give the copies already in flight a bounded chance to land before the CTA's shared
        // memory is released, then report
        if (warp == 0) {
            const long long t0c = clock64();
            while (clock64() - t0c < 2000000LL) {}
        }
        if (lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
    }

    // ================================ grid barrier, then the log-sum-exp merge ================================
    // Work item = (sequence, group of `hpi` query heads).  The ring is idle after the barrier: the item's partials (hpi * D
    // floats of outputs and 16 bytes of log-sum-exps per contributing CTA) are brought into it with bulk copies that are all
    // in flight at once, up to `chunk` partials per round, so the merge costs one trip to L2 instead of one per batch of
    // loads.  hpi = 512 / D heads (2 KB per partial, 32 partials per round, a thread per output pair) when that gives the
    // grid enough items; for a batch of few, long sequences - many partials per sequence, few items - hpi = 1: four (two)
    // times as many items, every partial of an item in one round (120 / 60 per round), and the CTA's thread groups share
    // an item's partials and add their sums through shared memory.
    // Everything that does not depend on other CTAs (which partials the first item needs) is worked out before the wait.
    constexpr int kHpiCoarse = 512 / kD;
    const int hpi = mg.fine_items ? 1 : kHpiCoarse;
    const int row_floats = hpi * kD;                               // staged outputs per partial
    const uint32_t part_bytes = static_cast<uint32_t>(row_floats) * 4u + 16u;
    const int chunk = mg.fine_items ? (kD == 128 ? 120 : 60) : 32;
    static_assert(32 * 2064 <= LT::kBarOff && 120 * 528 <= LT::kBarOff && 60 * 1040 <= LT::kBarOff, "merge staging must fit in the ring");
    float *m_val = reinterpret_cast<float *>(smem);                                            // [chunk][hpi][D]
    float *m_lse = reinterpret_cast<float *>(smem + static_cast<size_t>(chunk) * row_floats * 4);  // [chunk][4]
    const uint32_t bar_merge = bar_full + 2 * kTcStages * 8 + 8;
    uint32_t mphase = 0;
    const int groups = n_q_heads / hpi;
    const int item_threads = row_floats / 2;                       // a thread per output pair of the item
    const int tgroups = kTcThreads / item_threads;                 // thread groups that share an item's partials (1, 2 or 4)
    const int tg = threadIdx.x / item_threads, within = threadIdx.x - tg * item_threads;
    auto owner = [&](int64_t t, int r) -> int64_t {  // the CTA whose range holds tile t of sequence r
        const int64_t v = 8 * t + static_cast<int64_t>(pad_units) * (r + 1);  // the tile's first virtual unit
        int64_t c = small ? static_cast<int64_t>(static_cast<uint32_t>(v) * static_cast<uint32_t>(n_ctas) / static_cast<uint32_t>(vtotal)) : v * n_ctas / vtotal;
        if (c > n_ctas - 1) c = n_ctas - 1;
        while (c > 0 && vbegin(c) > v) --c;
        while (c < n_ctas - 1 && vbegin(c + 1) <= v) ++c;
        return c;
    };
    auto item_parts = [&](int item, int &r, int &h0, int64_t &c_lo, int &np) {
        r = item / groups;
        h0 = (item - r * groups) * hpi;
        const int64_t before = s_pref[r], nt = s_pref[r + 1] - s_pref[r];
        c_lo = 0;
        np = 0;
        if (nt > 0) {
            c_lo = owner(before, r);
            np = static_cast<int>(owner(before + nt - 1, r) - c_lo + 1) * LT::kTH;
        }
    };
    int r = 0, h0 = 0, np = 0;
    int64_t c_lo = 0;
    const bool has_item = static_cast<int>(blockIdx.x) < n_seqs * groups;
    if (has_item) item_parts(blockIdx.x, r, h0, c_lo, np);

    // All CTAs are co-resident (cooperative launch).  The counter only ever counts up: a CTA's ticket tells it which
    // multiple of the grid size completes its launch (every launch that uses this counter has the same grid size - one
    // counter for one CTA per SM, one for two - and every CTA, even one whose waits ran out, takes exactly one ticket).
    // The wait is bounded.
    __shared__ int s_bar_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (has_item && np > 0) mbar_expect_tx(bar_merge, static_cast<uint32_t>(min(chunk, np)) * part_bytes);
        const unsigned long long n = gridDim.x;
        unsigned long long ticket;
        // release: this CTA's partials are visible device-wide before it is counted; acquire: the CTA that arrives last sees
        // everyone else's
        asm volatile("atom.add.acq_rel.gpu.global.u64 %0, [%1], 1;" : "=l"(ticket) : "l"(&g_tc_barrier[mg.counter]) : "memory");
        const unsigned long long target = (ticket / n + 1ULL) * n;
        int good = 1;
        if (ticket + 1ULL != target) {
            const long long t0b = clock64();
            while (true) {
                unsigned long long seen;
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(&g_tc_barrier[mg.counter]) : "memory");
                if (seen >= target) break;
                if (clock64() - t0b > kTcWaitCycles) { good = 0; break; }
                __nanosleep(32);
            }
        }
        s_bar_ok = good;
    }
    __syncthreads();
    if (!s_bar_ok) {
        if (threadIdx.x == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
        return;
    }
    asm volatile("fence.proxy.async;" ::: "memory");  // partials were written with ordinary stores, the copies read them through the async proxy
    for (int item = blockIdx.x; item < n_seqs * groups; item += gridDim.x) {
        const bool first_item = item == static_cast<int>(blockIdx.x);
        if (!first_item) item_parts(item, r, h0, c_lo, np);
        const int hh = within / (kD / 2), d = (within % (kD / 2)) * 2;  // thread = (head of the item, column pair)
        const int h0a = h0 & ~3, hl = h0 - h0a + hh;                    // log-sum-exps travel in aligned groups of 4 heads
        float M = -INFINITY, den = 0.0f;
        float2 num = make_float2(0.0f, 0.0f);
        for (int p0 = 0; p0 < np; p0 += chunk) {
            const int n = min(chunk, np - p0);
            if (!(first_item && p0 == 0)) {  // (the first round's byte count was posted before the grid barrier)
                __syncthreads();  // the previous round's readers are done with the staging area
                if (threadIdx.x == 0) mbar_expect_tx(bar_merge, static_cast<uint32_t>(n) * part_bytes);
                __syncthreads();
            }
            if (threadIdx.x < n) {
                const int64_t slot = (c_lo + r) * LT::kTH + p0 + threadIdx.x;
                bulk_g2s(smem_u32(m_val + threadIdx.x * row_floats), o_part + (slot * n_q_heads + h0) * kD, static_cast<uint32_t>(row_floats) * 4u, bar_merge);
                bulk_g2s(smem_u32(m_lse + threadIdx.x * 4), lse_part + slot * n_q_heads + h0a, 16u, bar_merge);
            }
            if (!mbar_wait(bar_merge, mphase, abort_flag)) {
                if (lane == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
                return;
            }
            mphase ^= 1u;
            float Mc = M;
            for (int pi = 0; pi < n; ++pi) Mc = fmaxf(Mc, m_lse[pi * 4 + hl]);  // every thread group sees every partial's log-sum-exp
            if (Mc != -INFINITY) {
                const float resc = M == -INFINITY ? 0.0f : __expf(M - Mc);
                num.x *= resc; num.y *= resc; den *= resc;
                M = Mc;
#pragma unroll 4
                for (int pi = tg; pi < n; pi += tgroups) {  // this thread group's share of the partials
                    const float ls = m_lse[pi * 4 + hl];
                    const float w = ls == -INFINITY ? 0.0f : __expf(ls - M);
                    const float2 v = *reinterpret_cast<const float2 *>(m_val + pi * row_floats + hh * kD + d);
                    den += w;
                    num.x = fmaf(w, v.x, num.x);
                    num.y = fmaf(w, v.y, num.y);
                }
            }
        }
        if (tgroups > 1) {  // add the thread groups' sums (same M in all of them) in group 0, through the staging area
            __syncthreads();
            float *red = reinterpret_cast<float *>(smem);  // [tgroups - 1][item_threads][3]
            if (tg > 0) {
                float *p = red + (static_cast<size_t>(tg - 1) * item_threads + within) * 3;
                p[0] = num.x; p[1] = num.y; p[2] = den;
            }
            __syncthreads();
            if (tg == 0)
                for (int g2 = 1; g2 < tgroups; ++g2) {
                    const float *p = red + (static_cast<size_t>(g2 - 1) * item_threads + within) * 3;
                    num.x += p[0]; num.y += p[1]; den += p[2];
                }
        }
        const bool active = tg == 0;  // the threads that own an output pair of the item
        const int64_t row = static_cast<int64_t>(r) * n_q_heads + h0 + hh;
        float o0 = den > 0.0f ? num.x / den : 0.0f, o1 = den > 0.0f ? num.y / den : 0.0f;
        if (mg.shard.world > 0) {
            // ---- KV-length shards on several GPUs: deliver this shard's (o, lse) of the item to every rank's inbox as
            // {value, epoch} words (ordinary stores over NVLink), then wait - bounded - until the other ranks' words of the
            // same rows carry this step's epoch in the own inbox, and merge them.  A CTA's deliveries precede its waits.
            const ShardArgs &sh = mg.shard;
            const int W = sh.world;
            const long long half = sh.epoch & 1u, stride = kD + 2;
            const float lse_mine = den > 0.0f ? M + __logf(den) : -INFINITY;
            const long long w_mine = ((half * W + sh.rank) * sh.rows_cap + row) * stride;
            if (active)
                for (int s2 = 0; s2 < W; ++s2) {
                    st_word2(sh.inbox[s2] + w_mine + d, o0, o1, sh.epoch);
                    if (d == 0) st_word(sh.inbox[s2] + w_mine + kD, lse_mine, sh.epoch);
                }
            if (sh.push_only) continue;
            const unsigned long long *box = sh.inbox[sh.rank];
            int arrived = 1;
            float Mx = -INFINITY;
            const long long t0s = clock64();
            for (int s2 = 0; s2 < W && arrived && active; ++s2) {  // every word this thread will read, from every source
                const unsigned long long *rp = box + ((half * W + s2) * sh.rows_cap + row) * stride;
                while (true) {
                    const uint2 wl = ld_word(rp + kD);
                    const uint4 wo = ld_word2(rp + d);
                    if (wl.y == sh.epoch && wo.y == sh.epoch && wo.w == sh.epoch) {
                        Mx = fmaxf(Mx, __uint_as_float(wl.x));
                        break;
                    }
                    if (clock64() - t0s > sh.wait_cycles) { arrived = 0; break; }
                    __nanosleep(40);
                }
            }
            if (!__syncthreads_and(arrived)) {  // a rank did not deliver in time: recorded, this item gets no output, the launch goes on
                if (threadIdx.x == 0) atomicOr(err, HS_DEVERR_WAIT_TIMEOUT);
                continue;
            }
            float nx = 0.0f, ny = 0.0f, dn = 0.0f;
            for (int s2 = 0; s2 < W; ++s2) {
                const unsigned long long *rp = box + ((half * W + s2) * sh.rows_cap + row) * stride;
                const float ls = __uint_as_float(ld_word(rp + kD).x);
                const uint4 wo = ld_word2(rp + d);
                const float w = ls == -INFINITY ? 0.0f : __expf(ls - Mx);
                nx = fmaf(w, __uint_as_float(wo.x), nx); ny = fmaf(w, __uint_as_float(wo.z), ny); dn += w;
            }
            o0 = dn > 0.0f ? nx / dn : 0.0f;
            o1 = dn > 0.0f ? ny / dn : 0.0f;
        }
        if (!active) continue;
        if (mg.o_shard != nullptr) {
            *reinterpret_cast<float2 *>(mg.o_shard + row * kD + d) = make_float2(o0, o1);
            if (d == 0) mg.lse_shard[row] = den > 0.0f ? M + __logf(den) : -INFINITY;
        } else {
            float r0 = o0, r1 = o1;
            if (mg.gate != nullptr) {  // ctx * sigmoid(gate) in bf16 (qwen3_5.rs:1056-1059)
                const uint32_t gw = *reinterpret_cast<const uint32_t *>(mg.gate + row * kD + d);
                r0 = bf16_round(o0) * bf16_round(1.0f / (1.0f + __expf(-bf16lo(gw))));
                r1 = bf16_round(o1) * bf16_round(1.0f / (1.0f + __expf(-bf16hi(gw))));
            }
            *reinterpret_cast<uint32_t *>(mg.out + row * kD + d) = pack_bf16(r0, r1);
        }
    }
}

template <bool FOURBIT, int BPR, bool SF16, bool WIDE>
static int32_t launch_tc(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads, float kmul,
                         float *o_part, float *lse_part, int *err, int *n_ctas_io, TcMergeArgs mg, cudaStream_t s, int *fused_out) {
    using LT = TcLayout<FOURBIT, BPR, SF16, WIDE>;
    auto kern = decode_int8_tc_kernel<FOURBIT, BPR, SF16, WIDE>;
    // per instantiation and device: 0 = not configured, 1 / 2 = CTAs per SM of the cooperative grid, -1 = the device does not
    // take this kernel as a cooperative launch (the generic kernel serves it)
    static PerDeviceState config;
    const int dev = current_device();
    int ctas_per_sm = config.get(dev);
    if (ctas_per_sm == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LT::kTotal);
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_decode: %s", cudaGetErrorString(e));
        int coop = 0, per_sm = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kTcThreads, LT::kTotal);
        ctas_per_sm = (coop != 0 && per_sm >= 1) ? (per_sm >= 2 ? 2 : 1) : -1;
        config.set(dev, ctas_per_sm);
    }
    *fused_out = 0;
    if (ctas_per_sm < 0) return HS_OK;
    const int n_ctas = ctas_per_sm * sm_count();  // never more than the caller sized the partial slots for (two per SM)
    if (n_ctas > *n_ctas_io) return HS_OK;
    *n_ctas_io = n_ctas;
    mg.counter = ctas_per_sm - 1;
    ViewDev vv = v;
    void *args[] = {&vv, &q, &seq_lens, &n_seqs, &n_q_heads, &kmul, &o_part, &lse_part, &err, &mg};
    cudaError_t e = cudaErrorUnknown;
    if (mg.after_write) {
        // cooperative + programmatic stream serialisation; a driver that refuses the combination gets the plain launch for good
        static PerDeviceState pdl;  // 0 = untried, 1 = accepted, -1 = refused
        if (pdl.get(dev) >= 0) {
            cudaLaunchAttribute attrs[2];
            attrs[0].id = cudaLaunchAttributeCooperative;
            attrs[0].val.cooperative = 1;
            attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[1].val.programmaticStreamSerializationAllowed = 1;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(n_ctas);
            cfg.blockDim = dim3(kTcThreads);
            cfg.dynamicSmemBytes = LT::kTotal;
            cfg.stream = s;
            cfg.attrs = attrs;
            cfg.numAttrs = 2;
            e = cudaLaunchKernelExC(&cfg, reinterpret_cast<const void *>(kern), args);
            if (e == cudaSuccess) {
                pdl.set(dev, 1);
                *fused_out = 1;
                return HS_OK;
            }
            cudaGetLastError();
            pdl.set(dev, -1);
        }
        mg.after_write = 0;  // ordinary stream order: the write kernel has completed when this grid starts
    }
    e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kern), dim3(n_ctas), dim3(kTcThreads), args, LT::kTotal, s);
    if (e == cudaSuccess) {
        *fused_out = 1;
        return HS_OK;
    }
    cudaGetLastError();  // refused (e.g. the device is shared and cannot hold the whole grid): the generic kernel takes over for good
    config.set(dev, -1);
    return HS_OK;
}

// Returns HS_OK and sets *n_ctas_out (> 0) and *merged_out = 1 when the tensor-core kernel took the launch (it
// merges its own partials, which needs a cooperative launch); *n_ctas_out = 0 when the shape is not covered or
// the device refuses cooperative launches, and the caller should use the generic kernel.
int32_t decode_int8_tc_try(const ViewDev &v, const uint16_t *q, const int32_t *seq_lens, int n_seqs, int n_q_heads,
                           float softmax_scale, float *o_part, float *lse_part, int *err, cudaStream_t s, int *n_ctas_out,
                           uint16_t *out, const uint16_t *gate, float *o_shard, float *lse_shard, int *merged_out,
                           const ShardArgs *shard, int after_write, const AppendArgs *append) {
    *n_ctas_out = 0;
    *merged_out = 0;
    // covered shapes: 8 kv heads x 128 with 4 query heads each, and 2 kv heads x 256 with 8 query heads each
    const bool wide = v.head_dim == 256 && v.n_kv_heads == 2 && n_q_heads == 16;
    if (v.kind == HS_KV_BF16 || !(wide || (v.head_dim == 128 && v.n_kv_heads == 8 && n_q_heads == 32))) return HS_OK;
    if (v.page_tokens % 32 != 0 || n_seqs > (wide ? kTcMaxSeqs / 2 : kTcMaxSeqs)) return HS_OK;
    // the merge writes 4-byte pairs
    if ((out && !aligned(out, 4)) || (gate && !aligned(gate, 4)) || (o_shard && !aligned(o_shard, 8))) return HS_OK;
    const bool four = v.kind != HS_KV_INT8;
    const int bpr = 128 / v.block;  // scale blocks per 128-wide half of a head row
    if (bpr != 1 && bpr != 2) return HS_OK;
    if (four && (bpr != 2 || wide)) return HS_OK;  // 4-bit caches: the reference's block of 64, Llama shape
    const bool sf16 = v.scale_dtype == HS_SCALE_F16;
    int n_ctas = 2 * sm_count();  // upper bound; the launch settles on one or two CTAs per SM
    const float kmul = softmax_scale * 1.4426950408889634f / (four ? 1.0f : 127.0f);
    TcMergeArgs mg{out, gate, o_shard, lse_shard, 0, 0, after_write, AppendArgs{}, ShardArgs{}};
    mg.append.k_new = nullptr;
    if (append) {
        if (four) return HS_OK;  // only u8 caches are written inside the kernel: the caller launches the write kernel
        mg.append = *append;
    }
    // few, long sequences: with 512 / D heads per merge item less than half of the SMs would merge, each in several rounds
    mg.fine_items = static_cast<int64_t>(n_seqs) * n_q_heads / (512 / v.head_dim) * 2 <= sm_count() ? 1 : 0;
    mg.shard.world = 0;
    if (shard) mg.shard = *shard;
    int32_t st;
#define HS_TC_LAUNCH(F, B, S, W) launch_tc<F, B, S, W>(v, q, seq_lens, n_seqs, n_q_heads, kmul, o_part, lse_part, err, &n_ctas, mg, s, merged_out)
    if (wide) {
        if (bpr == 2 && !sf16) st = HS_TC_LAUNCH(false, 2, false, true);
        else if (bpr == 2) st = HS_TC_LAUNCH(false, 2, true, true);
        else if (!sf16) st = HS_TC_LAUNCH(false, 1, false, true);
        else st = HS_TC_LAUNCH(false, 1, true, true);
    } else if (four && !sf16) st = HS_TC_LAUNCH(true, 2, false, false);
    else if (four) st = HS_TC_LAUNCH(true, 2, true, false);
    else if (bpr == 2 && !sf16) st = HS_TC_LAUNCH(false, 2, false, false);
    else if (bpr == 2 && sf16) st = HS_TC_LAUNCH(false, 2, true, false);
    else if (bpr == 1 && !sf16) st = HS_TC_LAUNCH(false, 1, false, false);
    else st = HS_TC_LAUNCH(false, 1, true, false);
#undef HS_TC_LAUNCH
    if (st == HS_OK && *merged_out) *n_ctas_out = n_ctas;
    return st;
}

}  // namespace hs
