// Diagnostic harness for the tensor-core decode kernel: times it without Python on a synthetic ragged batch of the
// BASELINE.json configs[1] geometry (32 q / 8 kv heads, head_dim 128, int8 codes, block 128, f16 scales) and, when
// built with -DHS_TC_TIMING, prints where the CTAs spend their time (globaltimer stamps taken inside the kernel).
// Not part of the library: it includes the kernel's translation unit directly so that the diagnostic switches
// (HS_TC_TIMING, HS_TC_DRAIN_ONLY) reach it.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -I include -DHS_TC_TIMING \
//        hyprstream_b200/csrc/diag/decode_timeline.cu hyprstream_b200/csrc/runtime.cu -o decode_timeline
//   ./decode_timeline [batch]        (default 32 sequences of 512..8192 tokens)
//
// Contents of the cache are constant bytes: the kernel's time does not depend on the values.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "../decode_tc.cu"

using namespace hs;

#define CK(x)                                                                 \
    do {                                                                      \
        cudaError_t e_ = (x);                                                 \
        if (e_ != cudaSuccess) {                                              \
            printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

int main(int argc, char **argv) {
    const int B = argc > 1 ? atoi(argv[1]) : 32;
    if (B <= 0 || B > 256) { printf("batch must be in 1..256\n"); return 1; }
    std::mt19937 rng(1);
    std::vector<int> lens(B);
    long total_tokens = 0;
    for (int i = 0; i < B; ++i) { lens[i] = 512 + static_cast<int>(rng() % 7681); total_tokens += lens[i]; }
    const int cap = 9216, hq = 32;
    const size_t row_bytes = 8 * 128, scale_row_bytes = 8 * 2;  // per token: codes of 8 kv heads, one f16 scale each
    unsigned char *kd, *vd, *ksd, *vsd;
    CK(cudaMalloc(&kd, B * cap * row_bytes)); CK(cudaMalloc(&vd, B * cap * row_bytes));
    CK(cudaMalloc(&ksd, B * cap * scale_row_bytes)); CK(cudaMalloc(&vsd, B * cap * scale_row_bytes));
    CK(cudaMemset(kd, 0x55, B * cap * row_bytes)); CK(cudaMemset(vd, 0x66, B * cap * row_bytes));
    CK(cudaMemset(ksd, 0x3c, B * cap * scale_row_bytes)); CK(cudaMemset(vsd, 0x3c, B * cap * scale_row_bytes));
    std::vector<void *> tables(4 * B);
    for (int i = 0; i < B; ++i) {
        tables[i] = kd + i * cap * row_bytes; tables[B + i] = vd + i * cap * row_bytes;
        tables[2 * B + i] = ksd + i * cap * scale_row_bytes; tables[3 * B + i] = vsd + i * cap * scale_row_bytes;
    }
    void **tab;
    CK(cudaMalloc(&tab, tables.size() * sizeof(void *)));
    CK(cudaMemcpy(tab, tables.data(), tables.size() * sizeof(void *), cudaMemcpyHostToDevice));
    ViewDev v;
    v.k_pages = tab; v.v_pages = tab + B; v.k_scale_pages = tab + 2 * B; v.v_scale_pages = tab + 3 * B;
    v.kind = HS_KV_INT8; v.scale_dtype = HS_SCALE_F16; v.block = 128; v.n_kv_heads = 8; v.head_dim = 128;
    v.page_tokens = cap; v.pages_per_seq = 1;
    int *seq_lens;
    CK(cudaMalloc(&seq_lens, B * sizeof(int)));
    CK(cudaMemcpy(seq_lens, lens.data(), B * sizeof(int), cudaMemcpyHostToDevice));
    uint16_t *q, *out;
    CK(cudaMalloc(&q, B * hq * 128 * 2)); CK(cudaMemset(q, 0x3c, B * hq * 128 * 2));
    CK(cudaMalloc(&out, B * hq * 128 * 2));
    const int max_ctas = 2 * sm_count();
    float *o_part, *lse_part;
    CK(cudaMalloc(&o_part, static_cast<size_t>(max_ctas + B) * hq * 128 * sizeof(float)));
    CK(cudaMalloc(&lse_part, static_cast<size_t>(max_ctas + B) * hq * sizeof(float)));
    int *err = device_error_word();
    if (!err) { printf("no device error word\n"); return 1; }
    int n_ctas = 0, merged = 0;
    auto launch = [&]() { return decode_int8_tc_try(v, q, seq_lens, B, hq, 0.088f, o_part, lse_part, err, 0, &n_ctas, out, nullptr, nullptr, nullptr, &merged); };

    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    const double bytes = static_cast<double>(total_tokens) * 2 * (row_bytes + scale_row_bytes);
    for (int rep = 0; rep < 3; ++rep) {
        for (int i = 0; i < 5; ++i) launch();
        CK(cudaDeviceSynchronize());
        const int n = 50;
        CK(cudaEventRecord(e0));
        for (int i = 0; i < n; ++i) launch();
        CK(cudaEventRecord(e1));
        CK(cudaDeviceSynchronize());
        float ms;
        CK(cudaEventElapsedTime(&ms, e0, e1));
        printf("ctas %d (merged in the kernel: %d)  tokens %ld  %.2f us per launch  %.1f GB/s\n", n_ctas, merged, total_tokens, 1000.0 * ms / n,
               bytes / (ms / n) / 1e6);
    }
#ifdef HS_TC_TIMING
    if (n_ctas > 0) {
        // the kernel writes 16 stamps (ns) per warp: [cta][20 warps][16 slots]; warp 1's row is read (an ordinary consumer)
        unsigned long long *stamps;
        const size_t n = static_cast<size_t>(n_ctas) * 20 * 16;
        CK(cudaMalloc(&stamps, n * 8)); CK(cudaMemset(stamps, 0, n * 8));
        CK(cudaMemcpyToSymbol(g_tc_timing, &stamps, sizeof(stamps)));
        launch();
        CK(cudaDeviceSynchronize());
        std::vector<unsigned long long> h(n);
        CK(cudaMemcpy(h.data(), stamps, n * 8, cudaMemcpyDeviceToHost));
        unsigned long long t0 = ~0ull;
        for (size_t i = 0; i < n; ++i) if (h[i] && h[i] < t0) t0 = h[i];
        const char *names[16] = {"CTA starts", "streaming done", "sequence 1: starts", "  query fragments loaded", "  tiles done", "  partial written",
                                 "sequence 2: starts", "  query fragments loaded", "  tiles done", "  partial written", "at the grid barrier",
                                 "past the grid barrier", "merge item starts", "merge copies landed", "merge item stored", "CTA ends"};
        printf("%-28s %5s %8s %8s %8s %8s %8s   (us after the first CTA starts)\n", "stamp", "CTAs", "min", "10%", "median", "90%", "max");
        for (int s = 0; s < 16; ++s) {
            // (the stamp right after the barrier is left out: it reads earlier than the last arrival although no merge item
            // starts before that arrival - the merge stamps below are the ones to go by)
            if (s == 11) continue;
            std::vector<double> t;
            for (int c = 0; c < n_ctas; ++c) {
                const unsigned long long x = h[(static_cast<size_t>(c) * 20 + 1) * 16 + s];
                if (x) t.push_back((x - t0) / 1000.0);
            }
            if (t.empty()) continue;
            std::sort(t.begin(), t.end());
            printf("%-28s %5zu %8.2f %8.2f %8.2f %8.2f %8.2f\n", names[s], t.size(), t.front(), t[t.size() / 10], t[t.size() / 2], t[9 * t.size() / 10], t.back());
        }
    }
#endif
    int flags = 0;
    CK(cudaMemcpy(&flags, err, sizeof(int), cudaMemcpyDeviceToHost));
    printf("device error flags %d\n", flags);
    return flags == 0 ? 0 : 1;
}
