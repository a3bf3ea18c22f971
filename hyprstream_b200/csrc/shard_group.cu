// KV-length-sharded decode in one launch per GPU: the host object that owns a rank's inbox and knows its peers'.
//
// The reference has no collective on this path (its multi-GPU support is replicas and a layer split).  A context too
// long for one GPU is cut into contiguous KV-length shards, one per GPU; a decode step needs every shard's normalised
// output and log-sum-exp on every GPU.  Here the decode kernel itself delivers them: after its own split-KV merge each
// rank stores its (o, lse) into every rank's inbox with ordinary stores over NVLink (peer-mapped memory) as 8-byte
// {value, epoch} words, waits - bounded - until the other ranks' words in its own inbox carry the step's epoch and merges
// them.  No collective library call, no second launch, no fence, nothing allocated per step.
//
// An inbox is one cudaMalloc allocation (so that it can be exported as a CUDA IPC handle to the other ranks' processes)
// laid out as hs_common.cuh describes at ShardArgs.  Groups that live in one process (one host thread driving several
// GPUs, or several "ranks" on one GPU in a test) are connected directly by pointer.
#include <cstring>
#include <vector>

#include "hs_common.cuh"

namespace hs {
int32_t decode_impl(const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs, int32_t n_q_heads, float softmax_scale,
                    void *out, const void *gate, void *workspace, int64_t workspace_bytes, float *o_shard, float *lse_shard,
                    const ShardArgs *shard, hs_stream_t stream, int after_write = 0, const AppendArgs *append = nullptr, int *appended = nullptr);
}

struct hs_shard_group {
    int rank = 0, world = 0, device = 0;
    int n_q_heads = 0, head_dim = 0;
    long long rows_cap = 0;
    size_t bytes = 0;
    unsigned char *base = nullptr;                      // this rank's inbox
    unsigned char *peer_base[hs::kShardMaxWorld] = {};  // every rank's inbox as addressable from this device
    bool peer_opened[hs::kShardMaxWorld] = {};          // mapped with cudaIpcOpenMemHandle (to be closed)
    bool connected = false;
    unsigned int epoch = 0;
    int wait_ms = 2000;
    int clock_khz = 1965000;  // SM clock of the device, read once (the attribute query is slow)
};

using namespace hs;

extern "C" {

int32_t hs_shard_group_create(int32_t rank, int32_t world, int32_t max_seqs, int32_t n_q_heads, int32_t head_dim, hs_shard_group **out) {
    if (!out) return fail(HS_ERR_ARG, "hs_shard_group_create: NULL output");
    *out = nullptr;
    if (int32_t st = check_device()) return st;
    if (world < 1 || world > kShardMaxWorld || rank < 0 || rank >= world)
        return fail(HS_ERR_ARG, "hs_shard_group_create: rank %d of world %d (1..%d ranks)", rank, world, kShardMaxWorld);
    if (max_seqs <= 0 || n_q_heads <= 0 || (head_dim != 128 && head_dim != 256))
        return fail(HS_ERR_ARG, "hs_shard_group_create: max_seqs and n_q_heads must be positive, head_dim 128 or 256");
    hs_shard_group *g = new hs_shard_group();
    g->rank = rank; g->world = world; g->device = current_device();
    g->n_q_heads = n_q_heads; g->head_dim = head_dim;
    g->rows_cap = static_cast<long long>(max_seqs) * n_q_heads;
    g->bytes = static_cast<size_t>(2) * world * g->rows_cap * (head_dim + 2) * sizeof(unsigned long long);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, g->bytes);  // never the replaceable allocator: the handle must name a whole allocation
    if (e == cudaSuccess) e = cudaMemset(p, 0, g->bytes);  // every word starts with epoch 0, which no step carries
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (p) cudaFree(p);
        delete g;
        return fail(static_cast<int32_t>(e), "hs_shard_group_create: %s", cudaGetErrorString(e));
    }
    g->base = static_cast<unsigned char *>(p);
    g->peer_base[rank] = g->base;
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, g->device) == cudaSuccess && khz > 0) g->clock_khz = khz;
    cudaGetLastError();
    if (world == 1) g->connected = true;
    *out = g;
    return HS_OK;
}

int32_t hs_shard_group_handle_bytes(void) { return static_cast<int32_t>(sizeof(cudaIpcMemHandle_t)); }

int32_t hs_shard_group_export(hs_shard_group *group, void *handle_out) {
    if (!group || !handle_out) return fail(HS_ERR_ARG, "hs_shard_group_export: NULL argument");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, group->base);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(static_cast<int32_t>(e), "hs_shard_group_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    }
    std::memcpy(handle_out, &h, sizeof h);
    return HS_OK;
}

int32_t hs_shard_group_connect(hs_shard_group *group, const void *handles) {
    if (!group || !handles) return fail(HS_ERR_ARG, "hs_shard_group_connect: NULL argument");
    if (group->connected) return fail(HS_ERR_ARG, "hs_shard_group_connect: the group is connected already");
    if (current_device() != group->device) return fail(HS_ERR_ARG, "hs_shard_group_connect: make the group's device (%d) current", group->device);
    const unsigned char *hb = static_cast<const unsigned char *>(handles);
    for (int s = 0; s < group->world; ++s) {
        if (s == group->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, hb + static_cast<size_t>(s) * sizeof h, sizeof h);
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(static_cast<int32_t>(e), "hs_shard_group_connect: cudaIpcOpenMemHandle for rank %d: %s", s, cudaGetErrorString(e));
        }
        group->peer_base[s] = static_cast<unsigned char *>(p);
        group->peer_opened[s] = true;
    }
    group->connected = true;
    return HS_OK;
}

int32_t hs_shard_group_connect_local(hs_shard_group *const *groups, int32_t world) {
    if (!groups || world < 1 || world > kShardMaxWorld) return fail(HS_ERR_ARG, "hs_shard_group_connect_local: bad arguments");
    for (int r = 0; r < world; ++r) {
        if (!groups[r] || groups[r]->world != world || groups[r]->rank != r)
            return fail(HS_ERR_ARG, "hs_shard_group_connect_local: groups[%d] must be rank %d of a world of %d", r, r, world);
        if (groups[r]->rows_cap != groups[0]->rows_cap || groups[r]->head_dim != groups[0]->head_dim)
            return fail(HS_ERR_ARG, "hs_shard_group_connect_local: the groups were created for different shapes");
    }
    const int before = current_device();
    for (int r = 0; r < world; ++r) {
        hs_shard_group *g = groups[r];
        for (int s = 0; s < world; ++s) {
            if (groups[s]->device != g->device) {
                int can = 0;
                cudaDeviceCanAccessPeer(&can, g->device, groups[s]->device);
                if (!can) {
                    cudaSetDevice(before);
                    return fail(HS_ERR_DEVICE, "hs_shard_group_connect_local: device %d cannot address device %d", g->device, groups[s]->device);
                }
                cudaSetDevice(g->device);
                cudaError_t e = cudaDeviceEnablePeerAccess(groups[s]->device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                    cudaGetLastError();
                    cudaSetDevice(before);
                    return fail(static_cast<int32_t>(e), "hs_shard_group_connect_local: cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
                }
                cudaGetLastError();
            }
            g->peer_base[s] = groups[s]->base;
        }
        g->connected = true;
    }
    if (before >= 0) cudaSetDevice(before);
    return HS_OK;
}

int32_t hs_shard_group_set_wait_ms(hs_shard_group *group, int32_t wait_ms) {
    if (!group || wait_ms <= 0 || wait_ms > 10000) return fail(HS_ERR_ARG, "hs_shard_group_set_wait_ms: 1..10000 ms");
    group->wait_ms = wait_ms;
    return HS_OK;
}

int32_t hs_shard_group_epoch(const hs_shard_group *group) { return group ? static_cast<int32_t>(group->epoch & 0x7fffffffu) : 0; }

void hs_shard_group_destroy(hs_shard_group *group) {
    if (!group) return;
    for (int s = 0; s < group->world; ++s)
        if (group->peer_opened[s] && group->peer_base[s]) cudaIpcCloseMemHandle(group->peer_base[s]);
    if (group->base) cudaFree(group->base);
    cudaGetLastError();
    delete group;
}

int32_t hs_attn_decode_sharded(hs_shard_group *group, const void *q, const hs_kv_view *view, const int32_t *seq_lens, int32_t n_seqs,
                               int32_t n_q_heads, float softmax_scale, void *out, const void *gate, void *workspace,
                               int64_t workspace_bytes, int32_t flags, hs_stream_t stream) {
    if (!group) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: NULL group");
    if (!group->connected) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: the group is not connected to its peers yet");
    if (int32_t st = check_device()) return st;
    if (current_device() != group->device) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: make the group's device (%d) current", group->device);
    if (!view) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: NULL view");
    if (n_seqs <= 0) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: n_seqs must be positive (an empty shard passes seq_lens of 0)");
    if (n_q_heads != group->n_q_heads || view->head_dim != group->head_dim || static_cast<long long>(n_seqs) * n_q_heads > group->rows_cap)
        return fail(HS_ERR_ARG, "hs_attn_decode_sharded: shape (%d sequences x %d heads x %d) does not fit the group (%lld rows of %d heads x %d)",
                    n_seqs, n_q_heads, view->head_dim, group->rows_cap, group->n_q_heads, group->head_dim);
    const bool push_only = (flags & HS_SHARD_PUSH_ONLY) != 0;
    if (!push_only && !out) return fail(HS_ERR_ARG, "hs_attn_decode_sharded: no output");
    ShardArgs sh;
    std::memset(&sh, 0, sizeof sh);
    for (int s = 0; s < group->world; ++s) sh.inbox[s] = reinterpret_cast<unsigned long long *>(group->peer_base[s]);
    sh.rank = group->rank;
    sh.world = group->world;
    unsigned int epoch = group->epoch + 1;
    if (epoch == 0) epoch = 2;  // never 0 (the cleared flags), and the halves keep alternating
    sh.epoch = epoch;
    sh.push_only = push_only ? 1 : 0;
    sh.wait_cycles = static_cast<long long>(group->wait_ms) * group->clock_khz;
    sh.rows_cap = group->rows_cap;
    int32_t st = decode_impl(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, push_only ? nullptr : out, gate, workspace, workspace_bytes,
                             nullptr, nullptr, &sh, stream);
    if (st == HS_OK) group->epoch = epoch;  // a refused call delivered nothing: the step number stands
    return st;
}

}  // extern "C"
