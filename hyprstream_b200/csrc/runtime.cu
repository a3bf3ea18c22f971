// Status plumbing shared by every entry point: thread-local error text, device check, view validation.
#include <cstring>

#include <atomic>

#include "hs_common.cuh"

namespace hs {

static thread_local char g_err[512] = "";
// word 0: HS_DEVERR_* flags; word 1: id of the latest launch that recorded a wait time-out (see hs_common.cuh)
static __device__ int g_device_error[4];
static std::atomic<int *> g_device_error_ptr[kMaxDevices];

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return dev;
}

int *device_error_word() {
    const int dev = current_device();
    if (dev < 0) return nullptr;
    if (dev < kMaxDevices) {
        if (int *p = g_device_error_ptr[dev].load(std::memory_order_acquire)) return p;
    }
    int *p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_device_error) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (dev < kMaxDevices) g_device_error_ptr[dev].store(p, std::memory_order_release);
    return p;
}

uint32_t next_launch_id() {
    static std::atomic<uint32_t> g_id{0};
    uint32_t id = g_id.fetch_add(1, std::memory_order_relaxed) + 1;
    if (id == 0) id = g_id.fetch_add(1, std::memory_order_relaxed) + 1;
    return id;
}

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int32_t fail(int32_t code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

static int32_t device_status(int dev) {
    int major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(HS_ERR_DEVICE, "no usable CUDA device: %s", cudaGetErrorString(e));
    }
    if (major != 10) return fail(HS_ERR_DEVICE, "device %d is compute capability %d.x; this library is sm_100a only", dev, major);
    return HS_OK;
}

int32_t check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(HS_ERR_DEVICE, "no usable CUDA device: %s", cudaGetErrorString(e));
    }
    static thread_local int ok_dev = -1;
    if (ok_dev == dev) return HS_OK;
    int32_t st = device_status(dev);
    if (st == HS_OK) ok_dev = dev;
    return st;
}

int sm_count() {
    static PerDeviceState cache;
    const int dev = current_device();
    if (int n = cache.get(dev)) return n;
    int n = 148;
    if (dev >= 0) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cache.set(dev, n);
    return n;
}

static std::atomic<long long> g_launches{0};

int32_t check_launch(const char *what) {  // called once after every kernel launch of the library
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(static_cast<int32_t>(e), "%s: %s", what, cudaGetErrorString(e));
    return HS_OK;
}

// ---- optional per-kernel timing (off by default) -------------------------------------------------
static bool g_prof_on = false;
static bool g_prof_valid = false;
static cudaEvent_t g_prof_ev[2] = {nullptr, nullptr};

void prof_begin(cudaStream_t s) {
    if (g_prof_on) cudaEventRecord(g_prof_ev[0], s);
}
void prof_end(cudaStream_t s) {
    if (g_prof_on) {
        cudaEventRecord(g_prof_ev[1], s);
        g_prof_valid = true;
    }
}

int32_t validate_view(const hs_kv_view *v) {
    if (!v) return fail(HS_ERR_ARG, "kv view is NULL");
    if (v->kind < HS_KV_BF16 || v->kind > HS_KV_FP4) return fail(HS_ERR_ARG, "kv view: unknown kind %d", v->kind);
    if (v->n_kv_heads <= 0 || v->page_tokens <= 0 || v->pages_per_seq <= 0)
        return fail(HS_ERR_ARG, "kv view: n_kv_heads, page_tokens and pages_per_seq must be positive");
    if (v->head_dim != 64 && v->head_dim != 128 && v->head_dim != 256)
        return fail(HS_ERR_UNSUPPORTED, "kv view: head_dim %d (supported: 64, 128, 256)", v->head_dim);
    if (!v->k_pages || !v->v_pages) return fail(HS_ERR_ARG, "kv view: page tables are NULL");
    if (v->kind != HS_KV_BF16) {
        if (v->block != 64 && v->block != 128 && v->block != 256)
            return fail(HS_ERR_UNSUPPORTED, "kv view: block %d (supported: 64, 128, 256)", v->block);
        if (v->head_dim % v->block != 0)
            return fail(HS_ERR_UNSUPPORTED, "kv view: block %d must divide head_dim %d", v->block, v->head_dim);
        if (v->scale_dtype != HS_SCALE_F32 && v->scale_dtype != HS_SCALE_F16)
            return fail(HS_ERR_ARG, "kv view: unknown scale dtype %d", v->scale_dtype);
        if (!v->k_scale_pages || !v->v_scale_pages) return fail(HS_ERR_ARG, "kv view: scale page tables are NULL");
    }
    return HS_OK;
}

}  // namespace hs

extern "C" {

int32_t hs_attn_version(void) { return 100; }

int32_t hs_attn_device_check(int32_t device) {
    if (device < 0) return hs::check_device();
    return hs::device_status(device);
}

const char *hs_attn_last_error(void) { return hs::g_err; }

int64_t hs_attn_launch_count(void) { return hs::g_launches.load(std::memory_order_relaxed); }

int32_t hs_attn_set_profiling(int32_t on) {
    if (int32_t st = hs::check_device()) return st;
    if (on && !hs::g_prof_ev[0]) {
        for (int i = 0; i < 2; ++i) {
            cudaError_t e = cudaEventCreate(&hs::g_prof_ev[i]);
            if (e != cudaSuccess) return hs::fail(static_cast<int32_t>(e), "hs_attn_set_profiling: %s", cudaGetErrorString(e));
        }
    }
    hs::g_prof_on = on != 0;
    hs::g_prof_valid = false;
    return HS_OK;
}

int32_t hs_attn_last_kernel_ms(float *ms) {
    if (!ms) return hs::fail(HS_ERR_ARG, "hs_attn_last_kernel_ms: NULL output");
    if (!hs::g_prof_valid) return hs::fail(HS_ERR_ARG, "hs_attn_last_kernel_ms: no profiled launch since profiling was switched on");
    cudaError_t e = cudaEventSynchronize(hs::g_prof_ev[1]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, hs::g_prof_ev[0], hs::g_prof_ev[1]);
    if (e != cudaSuccess) return hs::fail(static_cast<int32_t>(e), "hs_attn_last_kernel_ms: %s", cudaGetErrorString(e));
    return HS_OK;
}

int32_t hs_attn_take_device_error(int32_t *flags) {
    if (!flags) return hs::fail(HS_ERR_ARG, "hs_attn_take_device_error: NULL output");
    if (int32_t st = hs::check_device()) return st;
    int v = 0, zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, hs::g_device_error, sizeof v);
    if (e == cudaSuccess && v != 0) e = cudaMemcpyToSymbol(hs::g_device_error, &zero, sizeof zero);  // clear the flags
    if (e != cudaSuccess) return hs::fail(static_cast<int32_t>(e), "hs_attn_take_device_error: %s", cudaGetErrorString(e));
    *flags = v;
    return HS_OK;
}

// Test hook: ORs `flags` into the current device's error word from the host (a plain copy; no kernel, no fault), so
// that the behaviour of the entry points with flags pending can be tested without making a wait run out.
int32_t hs_attn_inject_device_error(int32_t flags) {
    if (int32_t st = hs::check_device()) return st;
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, hs::g_device_error, sizeof v);
    v |= flags;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(hs::g_device_error, &v, sizeof v);
    if (e != cudaSuccess) return hs::fail(static_cast<int32_t>(e), "hs_attn_inject_device_error: %s", cudaGetErrorString(e));
    return HS_OK;
}

}  // extern "C"
