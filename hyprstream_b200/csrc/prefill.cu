// Causal GQA prefill attention (q_len >= 1 query tokens per sequence against kv_len >= q_len keys).
//
// Replaces compute_attention_masked's multi-token branch, single shot and 1024-row chunked
// (architectures/llama.rs:1023-1119), including GQA expansion (llama.rs:847-872) and the cached-prefix mask
// offset tril(k_len - q_len) (llama.rs:1074-1084), and Qwen3_5FullAttention's prefill branch with its
// output gate (qwen3_5.rs:1012-1059).  Scores and the softmax are fp32; P is rounded to bf16 for P.V
// (as the Qwen3.5 reference does, qwen3_5.rs:1031-1032; the Llama reference keeps fp32 — the difference is
// inside the 2e-2 / 2e-3 acceptance band against an fp32 recomputation).  Masked positions get -inf
// (the reference's -10000 fill is numerically the same for any row with one unmasked key).
//
// This file holds the mma.sync (m16n8k16, bf16) flash-attention form: one CTA = 4 warps = 64 query rows of
// one head; K/V tiles of 64 keys stream through a double-buffered, XOR-swizzled shared-memory ring with
// cp.async; the score matrix never leaves registers.
#include "hs_common.cuh"

namespace hs {

constexpr int kPfM = 64;       // query rows per CTA
constexpr int kPfWarps = 4;
constexpr int kPfThreads = kPfWarps * 32;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool pred) {
    const int sz = pred ? 16 : 0;  // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold D bf16 (D*2 bytes), XOR-swizzled
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// rows [row0, row0 + ROWS) of a [n_rows, stride_elems] bf16 matrix -> swizzled shared tile; rows >= n_rows are zero
template <int D, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t smem_tile, const uint16_t *base, int64_t stride_elems, int row0, int n_rows) {
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    for (int i = threadIdx.x; i < ROWS * CPR; i += kPfThreads) {
        const int r = i / CPR, c = i - r * CPR;
        const bool ok = row0 + r < n_rows;
        const uint16_t *src = base + static_cast<int64_t>(ok ? row0 + r : 0) * stride_elems + c * 8;
        cp_async16(smem_tile + swz<D>(r, c), src, ok);
    }
}

template <int D, int BN>
__global__ void __launch_bounds__(kPfThreads)
prefill_mma_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                   uint16_t *__restrict__ out, const uint16_t *__restrict__ gate, int64_t gate_ts, int64_t gate_hs, int q_len, int kv_len,
                   int n_q_heads, int n_kv_heads, float scale_log2) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kQBytes = kPfM * D * 2, kTile = BN * D * 2;
    const uint32_t sQ = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const uint32_t sK = sQ + kQBytes, sV = sK + 2 * kTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
    const int mb = gridDim.x - 1 - blockIdx.x;  // heaviest (latest) query blocks first
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (n_q_heads / n_kv_heads);
    const int m0 = mb * kPfM;
    const int off = kv_len - q_len;  // query row i may see keys j <= off + i
    const int64_t q_stride = static_cast<int64_t>(n_q_heads) * D, kv_stride = static_cast<int64_t>(n_kv_heads) * D;
    const uint16_t *qb = q + (static_cast<int64_t>(b) * q_len * n_q_heads + h) * D;
    const uint16_t *kb = k + (static_cast<int64_t>(b) * kv_len * n_kv_heads + kvh) * D;
    const uint16_t *vb = v + (static_cast<int64_t>(b) * kv_len * n_kv_heads + kvh) * D;
    // keys this query block can see: [0, n_end)
    const int n_end = min(kv_len, off + min(m0 + kPfM, q_len));
    const int n_blocks = (n_end + BN - 1) / BN;

    load_tile<D, kPfM>(sQ, qb, q_stride, m0, q_len);
    load_tile<D, BN>(sK, kb, kv_stride, 0, kv_len);
    load_tile<D, BN>(sV, vb, kv_stride, 0, kv_len);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // Q fragments of this warp's 16 rows stay in registers
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldsm4(qf[kk], sQ + swz<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.0f, 0.0f};
    const int row_lo = m0 + warp * 16 + g, row_hi = row_lo + 8;  // this thread's two query rows

    for (int nb = 0; nb < n_blocks; ++nb) {
        const int buf = nb & 1;
        if (nb + 1 < n_blocks) {  // prefetch the next K/V tile into the other buffer
            load_tile<D, BN>(sK + (buf ^ 1) * kTile, kb, kv_stride, (nb + 1) * BN, kv_len);
            load_tile<D, BN>(sV + (buf ^ 1) * kTile, vb, kv_stride, (nb + 1) * BN, kv_len);
        }
        cp_async_commit();
        const uint32_t tK = sK + buf * kTile, tV = sV + buf * kTile;
        // ---- S = Q K^T ----
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t kf[4];
                ldsm4(kf, tK + swz<D>(np * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[kk], kf[0], kf[1]);
                mma_bf16(s[2 * np + 1], qf[kk], kf[2], kf[3]);
            }
        }
        // ---- mask + online softmax (exp2 domain) ----
        const int n0 = nb * BN;
        const bool need_mask = n0 + BN > min(kv_len, off + m0 + warp * 16 + 1);  // tile reaches past the first row's limit
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < BN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = s[i][e] * scale_log2;
                if (need_mask) {
                    const int col = n0 + i * 8 + 2 * j + (e & 1);
                    const int row = (e & 2) ? row_hi : row_lo;
                    if (col > off + row || col >= kv_len) x = -INFINITY;
                }
                s[i][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(mrow[r], mx[r]);
            corr[r] = mn == -INFINITY ? 1.0f : exp2f(mrow[r] - mn);
            mrow[r] = mn;
        }
        float ps[2] = {0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < BN / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = mrow[e >> 1] == -INFINITY ? 0.0f : exp2f(s[i][e] - mrow[e >> 1]);
                s[i][e] = p;
                ps[e >> 1] += p;
            }
        lrow[0] = lrow[0] * corr[0] + ps[0];
        lrow[1] = lrow[1] * corr[1] + ps[1];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t vf[4];
                ldsm4_t(vf, tV + swz<D>(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), dp * 2 + (lane >> 4)));
                mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
                mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
            }
        }
        cp_async_wait<0>();
        __syncthreads();  // next tile landed; everyone is done with this one
    }
    // ---- epilogue: normalise, optional sigmoid gate in bf16 (qwen3_5.rs:1056-1059), store bf16 ----
    float l[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] = lrow[r];
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        l[r] = l[r] > 0.0f ? 1.0f / l[r] : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r ? row_hi : row_lo;
        if (row >= q_len) continue;
        const int64_t base = (static_cast<int64_t>(b) * q_len + row) * q_stride + static_cast<int64_t>(h) * D;
        const int64_t gbase = (static_cast<int64_t>(b) * q_len + row) * gate_ts + static_cast<int64_t>(h) * gate_hs;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            float x0 = o[i][2 * r] * l[r], x1 = o[i][2 * r + 1] * l[r];
            const int col = i * 8 + 2 * j;
            if (gate != nullptr) {
                const uint32_t gw = *reinterpret_cast<const uint32_t *>(gate + gbase + col);
                x0 = bf16_round(x0) * bf16_round(1.0f / (1.0f + __expf(-bf16lo(gw))));
                x1 = bf16_round(x1) * bf16_round(1.0f / (1.0f + __expf(-bf16hi(gw))));
            }
            *reinterpret_cast<uint32_t *>(out + base + col) = pack_bf16(x0, x1);
        }
    }
}

template <int D, int BN>
static int32_t launch_prefill(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *out, const uint16_t *gate,
                              int64_t gate_ts, int64_t gate_hs, int n_seqs, int q_len, int kv_len, int hq, int hkv, float scale_log2, cudaStream_t s) {
    constexpr int smem = kPfM * D * 2 + 4 * BN * D * 2;
    auto kern = prefill_mma_kernel<D, BN>;
    static PerDeviceState configured;  // per instantiation and device
    const int dev = current_device();
    if (smem > 48 * 1024 && !configured.get(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "hs_attn_prefill_causal: %s", cudaGetErrorString(e));
        configured.set(dev, 1);
    }
    dim3 grid((q_len + kPfM - 1) / kPfM, hq, n_seqs);
    kern<<<grid, kPfThreads, smem, s>>>(q, k, v, out, gate, gate_ts, gate_hs, q_len, kv_len, hq, hkv, scale_log2);
    return HS_OK;
}

// prefill_tc5.cu: tcgen05 / TMEM / TMA kernel for head_dim 128
int32_t prefill_tc5_try(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *out, const uint16_t *gate, int64_t gate_ts,
                        int64_t gate_hs, int n_seqs, int q_len, int kv_len, int n_q_heads, int n_kv_heads, int head_dim, float scale_log2,
                        cudaStream_t s, int *taken);

// The body of hs_attn_prefill_causal with the gate's strides spelled out (elements between tokens and between heads): the Qwen3.5
// layer entry reads the gate halves where the projection left them.
int32_t prefill_causal_impl(const void *q, const void *k, const void *v, void *out, const void *gate, int64_t gate_ts, int64_t gate_hs,
                            int32_t n_seqs, int32_t q_len, int32_t kv_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                            float softmax_scale, hs_stream_t stream) {
    if (int32_t st = check_device()) return st;
    if (n_seqs < 0 || q_len < 0 || kv_len < 0 || n_q_heads <= 0 || n_kv_heads <= 0) return fail(HS_ERR_ARG, "hs_attn_prefill_causal: bad sizes");
    if (n_q_heads % n_kv_heads != 0) return fail(HS_ERR_ARG, "hs_attn_prefill_causal: n_q_heads %d not a multiple of n_kv_heads %d", n_q_heads, n_kv_heads);
    if (kv_len < q_len) return fail(HS_ERR_ARG, "hs_attn_prefill_causal: kv_len %d < q_len %d", kv_len, q_len);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return fail(HS_ERR_UNSUPPORTED, "hs_attn_prefill_causal: head_dim %d (supported: 64, 128, 256)", head_dim);
    if (n_seqs == 0 || q_len == 0) return HS_OK;
    if (!q || !k || !v || !out) return fail(HS_ERR_ARG, "hs_attn_prefill_causal: NULL pointer");
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(out, 4) || (gate && !aligned(gate, 4)))
        return fail(HS_ERR_ARG, "hs_attn_prefill_causal: q, k, v must be 16-byte aligned");
    if (gate && (gate_ts % 2 != 0 || gate_hs % 2 != 0)) return fail(HS_ERR_ARG, "hs_attn_prefill_causal: gate strides must be even");
    if (n_seqs > 65535 || n_q_heads > 65535) return fail(HS_ERR_UNSUPPORTED, "hs_attn_prefill_causal: grid too large");
    const float sl2 = softmax_scale * 1.4426950408889634f;
    cudaStream_t s = as_stream(stream);
    const uint16_t *qp = reinterpret_cast<const uint16_t *>(q), *kp = reinterpret_cast<const uint16_t *>(k), *vp = reinterpret_cast<const uint16_t *>(v);
    uint16_t *op = reinterpret_cast<uint16_t *>(out);
    const uint16_t *gp = reinterpret_cast<const uint16_t *>(gate);
    int32_t st;
    int taken = 0;
    prof_begin(s);
    st = prefill_tc5_try(qp, kp, vp, op, gp, gate_ts, gate_hs, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads, head_dim, sl2, s, &taken);
    if (st != HS_OK || taken) {
    } else if (head_dim == 64) st = launch_prefill<64, 64>(qp, kp, vp, op, gp, gate_ts, gate_hs, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads, sl2, s);
    else if (head_dim == 128) st = launch_prefill<128, 64>(qp, kp, vp, op, gp, gate_ts, gate_hs, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads, sl2, s);
    else st = launch_prefill<256, 32>(qp, kp, vp, op, gp, gate_ts, gate_hs, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads, sl2, s);
    prof_end(s);
    if (st != HS_OK) return st;
    return check_launch("hs_attn_prefill_causal");
}

}  // namespace hs

using namespace hs;

extern "C" {

int32_t hs_attn_prefill_causal(const void *q, const void *k, const void *v, void *out, const void *gate, int32_t n_seqs,
                               int32_t q_len, int32_t kv_len, int32_t n_q_heads, int32_t n_kv_heads, int32_t head_dim,
                               float softmax_scale, hs_stream_t stream) {
    return prefill_causal_impl(q, k, v, out, gate, static_cast<int64_t>(n_q_heads) * head_dim, head_dim, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads,
                               head_dim, softmax_scale, stream);
}

}  // extern "C"
