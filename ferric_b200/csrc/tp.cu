// Tensor-parallel exchange group: the all-reduce of the row-parallel products' f32 partial sums,
// done by this library's own kernels over peer-mapped memory (NVLink), one process per GPU.
//
// The reference has no collective at all (its multi-device story is host-buffer hops,
// crates/ferric-tensor/src/sched.rs:209-265); the exchange exists because the layer matrices are
// sharded across GPUs.  Shape of one exchange, for kind k (0: after o, 1: after down):
//   1. the row-parallel GEMV writes its [m, hidden] partial straight into this rank's exchange
//      buffer k (plain device memory, exported to the peers with CUDA IPC);
//   2. a one-CTA signal kernel bumps this rank's count for k and stores it, release / system
//      scope, into every peer's flag slot for this rank;
//   3. the consumer (the fused add + rmsnorm + prepare kernel) waits, bounded, until all flag
//      slots have reached its own count, then reads every rank's partial with plain peer loads
//      and sums them in rank order -- bit-identical on every rank.
// One buffer per kind suffices only because consecutive exchanges alternate between the two kinds (after o, after
// down, after o, ...): a rank overwrites its kind-k buffer for exchange n+1 after its own consumer of the kind-(1-k)
// exchange in between ran, which needed every peer's signal for that exchange, which each peer gave only after its
// consumer of the kind-k exchange n had finished reading.  The same kind twice in a row would let a rank overwrite a
// buffer a slower peer is still reading, so ferric_cuda_tp_signal refuses it.  No multicast, no multimem: peer
// loads/stores only.
//
// The pushed form of the same exchange (tp_matmul_push + tp_add_rmsnorm_prepare_pushed) takes the
// signal kernel and the round trip of the peer loads off the critical path: the product's epilogue
// stores (value, exchange number) pairs into every rank's receive region [kind][parity][source rank],
// and the consumer polls the pairs in its own memory.  Parity double-buffers the regions: a rank
// can write exchange n+2 of a kind only after it consumed n+1, which needed every peer's n+1, which
// each peer produced after its own consumer of n had finished reading.
#include <string.h>

#include <new>

#include "../../include/ferric_cuda.h"
#include "common.cuh"
#include "handles.h"
#include "kernels.h"

using namespace ferric;

struct ferric_tp_group {
    int device = 0, rank = 0, world = 1;
    size_t elems = 0;                 // floats per exchange buffer
    // one local allocation: [2 buffers of elems floats][flags 2 x kMaxRanks][epoch 2][status 1][slot tables]
    void* local = nullptr;
    size_t local_bytes = 0;
    float* part[2] = {};
    unsigned* flags[2] = {};          // [kind][world] written by peers
    unsigned* epoch = nullptr;        // [2]
    int* status = nullptr;
    unsigned** slot_table[2] = {};    // device arrays [world] of peers' flag-slot addresses for this rank
    unsigned* push_epoch = nullptr;   // [2] pushed exchanges of each kind completed on this rank
    unsigned* push_ticket = nullptr;  // [2] CTA counters of the consumers
    uint2* recv = nullptr;            // [kind][parity][world][elems] (value, exchange number) pairs
    unsigned* wide_epoch = nullptr;   // [2] two-step all-reduces of each kind completed on this rank
    unsigned* wide_ticket = nullptr;  // [2]
    void* peer_base[kMaxRanks] = {};  // IPC mappings of the peers' `local`
    bool connected = false;
    bool local_peers = false;         // peers are groups of this process (no IPC mappings to close)
    int last_signal_kind = -1;        // the signalled (pull) form keeps one buffer per kind: kinds must alternate
};

namespace {
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
size_t off_flags(size_t elems) { return align_up(2 * elems * sizeof(float), 256); }
size_t off_epoch(size_t elems) { return off_flags(elems) + 2 * kMaxRanks * sizeof(unsigned); }
size_t off_status(size_t elems) { return off_epoch(elems) + 2 * sizeof(unsigned); }
size_t off_slots(size_t elems) { return align_up(off_status(elems) + sizeof(int), 256); }
size_t off_push_meta(size_t elems) { return align_up(off_slots(elems) + 2 * kMaxRanks * sizeof(void*), 256); }
size_t off_recv(size_t elems) { return off_push_meta(elems) + 256; }
size_t recv_pairs(size_t elems, int world) { return (size_t)world * elems; }   // one parity of one kind
size_t off_wide_meta(size_t elems, int world) { return off_recv(elems) + 4 * recv_pairs(elems, world) * sizeof(uint2); }
// the two-step all-reduce of whole matrices: slices of `wide_slice` floats per rank; per kind and parity, stage 1 holds
// every source's copy of this rank's slice and stage 2 the summed vector
size_t wide_slice(size_t elems, int world) { return ((elems + world - 1) / world + 3) / 4 * 4; }
size_t wide_pairs(size_t elems, int world) { return (size_t)world * wide_slice(elems, world); }   // one parity of one kind, either stage
size_t off_wide1(size_t elems, int world) { return off_wide_meta(elems, world) + 256; }
size_t off_wide2(size_t elems, int world) { return off_wide1(elems, world) + 4 * wide_pairs(elems, world) * sizeof(uint2); }
size_t total_bytes(size_t elems, int world) { return off_wide2(elems, world) + 4 * wide_pairs(elems, world) * sizeof(uint2); }
}  // namespace

static void fill_push_dst(const ferric_tp_group* g, int kind, PushDst& p)
{
    p.world = g->world;
    p.epoch = g->push_epoch + kind;
    p.parity_stride = recv_pairs(g->elems, g->world);
    for (int r = 0; r < g->world; r++)
        p.dst[r] = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(g->peer_base[r]) + off_recv(g->elems)) +
                   (size_t)kind * 2 * p.parity_stride + (size_t)g->rank * g->elems;
}
static void fill_push_src(const ferric_cuda_ctx* ctx, const ferric_tp_group* g, int kind, PushSrc& p)
{
    p.world = g->world;
    p.elems = g->elems;
    p.recv = g->recv + (size_t)kind * 2 * recv_pairs(g->elems, g->world);
    p.epoch = g->push_epoch + kind;
    p.ticket = g->push_ticket + kind;
    p.status = g->status;
    if (ctx->tune.wait_spins > 0) p.wait_spins = ctx->tune.wait_spins;
}

extern "C" {

int32_t ferric_cuda_tp_create(ferric_cuda_ctx* ctx, int32_t rank, int32_t world, size_t elems, ferric_tp_group** out)
{
    if (!ctx || !out || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || elems == 0 || (elems & 3)) {
        set_last_error("tp_create: bad arguments (world 1..%d, 0 <= rank < world, elems a positive multiple of 4)", kMaxRanks);
        return kErrInvalidArg;
    }
    *out = nullptr;
    DeviceGuard guard(ctx->device);
    ferric_tp_group* g = new (std::nothrow) ferric_tp_group;
    if (!g) return kErrOom;
    g->device = ctx->device;
    g->rank = rank;
    g->world = world;
    g->elems = elems;
    g->local_bytes = total_bytes(elems, world);
    cudaError_t e = cudaMalloc(&g->local, g->local_bytes);
    if (e != cudaSuccess) {
        delete g;
        return cuda_fail(e, "cudaMalloc(exchange buffers)");
    }
    e = cudaMemset(g->local, 0, g->local_bytes);
    if (e != cudaSuccess) {
        cudaFree(g->local);
        delete g;
        return cuda_fail(e, "cudaMemset(exchange buffers)");
    }
    uint8_t* base = reinterpret_cast<uint8_t*>(g->local);
    g->part[0] = reinterpret_cast<float*>(base);
    g->part[1] = g->part[0] + elems;
    g->flags[0] = reinterpret_cast<unsigned*>(base + off_flags(elems));
    g->flags[1] = g->flags[0] + kMaxRanks;
    g->epoch = reinterpret_cast<unsigned*>(base + off_epoch(elems));
    g->status = reinterpret_cast<int*>(base + off_status(elems));
    g->slot_table[0] = reinterpret_cast<unsigned**>(base + off_slots(elems));
    g->slot_table[1] = g->slot_table[0] + kMaxRanks;
    g->push_epoch = reinterpret_cast<unsigned*>(base + off_push_meta(elems));
    g->push_ticket = g->push_epoch + 2;
    g->recv = reinterpret_cast<uint2*>(base + off_recv(elems));
    g->wide_epoch = reinterpret_cast<unsigned*>(base + off_wide_meta(elems, world));
    g->wide_ticket = g->wide_epoch + 2;
    g->peer_base[rank] = g->local;
    *out = g;
    return kOk;
}

int32_t ferric_cuda_tp_export(ferric_tp_group* g, uint8_t* handle64)
{
    if (!g || !handle64) {
        set_last_error("NULL group or handle buffer");
        return kErrInvalidArg;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    DeviceGuard guard(g->device);
    cudaIpcMemHandle_t h;
    FERRIC_CUDA_TRY(cudaIpcGetMemHandle(&h, g->local));
    memcpy(handle64, &h, 64);
    return kOk;
}

int32_t ferric_cuda_tp_connect(ferric_tp_group* g, const uint8_t* handles)
{
    if (!g || !handles) {
        set_last_error("NULL group or handles");
        return kErrInvalidArg;
    }
    if (g->connected) return kOk;
    DeviceGuard guard(g->device);
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * r, 64);
        FERRIC_CUDA_TRY(cudaIpcOpenMemHandle(&g->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    // where this rank announces itself: slot [kind][rank] of every rank's flag array
    unsigned* slots[2][kMaxRanks] = {};
    for (int k = 0; k < 2; k++)
        for (int r = 0; r < g->world; r++)
            slots[k][r] = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(g->peer_base[r]) + off_flags(g->elems)) +
                          k * kMaxRanks + g->rank;
    FERRIC_CUDA_TRY(cudaMemcpy(g->slot_table[0], slots, sizeof(slots), cudaMemcpyHostToDevice));
    g->connected = true;
    return kOk;
}

int32_t ferric_cuda_tp_connect_local(ferric_tp_group* g, ferric_tp_group* const* groups)
{
    if (!g || !groups) {
        set_last_error("NULL group or group table");
        return kErrInvalidArg;
    }
    if (g->connected) return kOk;
    for (int r = 0; r < g->world; r++) {
        const ferric_tp_group* o = groups[r];
        if (!o || o->world != g->world || o->rank != r || o->elems != g->elems || (r == g->rank && o != g)) {
            set_last_error("tp_connect_local: entry %d is not rank %d of a group of the same shape", r, r);
            return kErrInvalidArg;
        }
    }
    DeviceGuard guard(g->device);
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank) continue;
        if (groups[r]->device != g->device) {
            int can = 0;
            FERRIC_CUDA_TRY(cudaDeviceCanAccessPeer(&can, g->device, groups[r]->device));
            if (!can) {
                set_last_error("device %d cannot address device %d", g->device, groups[r]->device);
                return kErrCuda;
            }
            cudaError_t e = cudaDeviceEnablePeerAccess(groups[r]->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
            cudaGetLastError();
        }
        g->peer_base[r] = groups[r]->local;
    }
    g->local_peers = true;
    unsigned* slots[2][kMaxRanks] = {};
    for (int k = 0; k < 2; k++)
        for (int r = 0; r < g->world; r++)
            slots[k][r] = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(g->peer_base[r]) + off_flags(g->elems)) +
                          k * kMaxRanks + g->rank;
    FERRIC_CUDA_TRY(cudaMemcpy(g->slot_table[0], slots, sizeof(slots), cudaMemcpyHostToDevice));
    g->connected = true;
    return kOk;
}

void* ferric_cuda_tp_partial(ferric_tp_group* g, int32_t kind) { return (g && kind >= 0 && kind < 2) ? g->part[kind] : nullptr; }

int32_t ferric_cuda_tp_signal(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind)
{
    if (!ctx || !g || kind < 0 || kind > 1 || !g->connected) {
        set_last_error("tp_signal: NULL / unconnected group or bad kind");
        return kErrInvalidArg;
    }
    if (g->world > 1 && kind == g->last_signal_kind) {
        set_last_error("tp_signal: exchange kind %d signalled twice in a row; the signalled form has one buffer per kind and must alternate kinds", kind);
        return kErrInvalidArg;
    }
    g->last_signal_kind = kind;
    DeviceGuard guard(ctx->device);
    ctx->launches++;
    return launch_tp_signal(ctx->stream, g->epoch + kind, g->slot_table[kind], g->world, ctx->tune);
}

int32_t ferric_cuda_tp_add_rmsnorm_prepare(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind,
                                           const ferric_qmatrix* qm, const float* a_dev, const float* weight_dev,
                                           float eps, size_t m, float* sum_dev, float* norm_dev)
{
    if (!ctx || !g || !qm || kind < 0 || kind > 1 || !g->connected || (m > 0 && !a_dev)) {
        set_last_error("tp_add_rmsnorm_prepare: NULL / unconnected argument or bad kind");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) return kUnsupported;
    if (m * qm->w.cols > g->elems) {
        set_last_error("exchange buffers hold %zu floats, %zu x %zu requested", g->elems, m, qm->w.cols);
        return kErrShape;
    }
    if (m == 0 || qm->w.nblk == 0) return kOk;
    DeviceGuard guard(ctx->device);
    int32_t rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, m));
    if (rc != kOk) return rc;
    PeerSum p;
    p.world = g->world;
    for (int r = 0; r < g->world; r++)
        p.part[r] = reinterpret_cast<const float*>(g->peer_base[r]) + (size_t)kind * g->elems;
    p.flags = g->flags[kind];
    p.epoch = g->epoch + kind;
    p.status = g->status;
    if (ctx->tune.wait_spins > 0) p.wait_spins = ctx->tune.wait_spins;
    ctx->launches++;
    return launch_norm_prep(ctx->stream, qm->ty, qm->w, a_dev, nullptr, weight_dev, eps, m, sum_dev, norm_dev, ctx->scratch,
                            ctx->tune, p);
}

int32_t ferric_cuda_tp_matmul_push(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind, const ferric_qmatrix* qm,
                                   const float* x_dev, size_t m, size_t ldx)
{
    if (!ctx || !g || !qm || kind < 0 || kind > 1 || !g->connected || (m > 0 && !x_dev)) {
        set_last_error("tp_matmul_push: NULL / unconnected argument or bad kind");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) return kUnsupported;
    if (ldx == 0) ldx = qm->w.cols;
    if (ldx < qm->w.cols || (ldx & 3)) {
        set_last_error("row stride ldx %zu must cover the row and be a multiple of 4", ldx);
        return kErrShape;
    }
    if (m * qm->w.rows > g->elems) {
        set_last_error("exchange buffers hold %zu floats, %zu x %zu requested", g->elems, m, qm->w.rows);
        return kErrShape;
    }
    if (m == 0 || qm->w.rows == 0) return kOk;
    if (qm->w.nblk == 0) {
        set_last_error("tp_matmul_push: empty K range");
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    int32_t rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, m));
    if (rc != kOk) return rc;
    rc = launch_prep(ctx->stream, qm->ty, qm->w, x_dev, m, ldx, ctx->scratch, ctx->tune);
    if (rc != kOk) return rc;
    PushDst p;
    fill_push_dst(g, kind, p);
    ctx->launches += 2;
    return launch_gemv(ctx->stream, qm->ty, qm->w, ctx->scratch, m, nullptr, qm->w.rows, kEpiPush, ctx->tune, p);
}

int32_t ferric_cuda_tp_add_rmsnorm_prepare_pushed(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind,
                                                  const ferric_qmatrix* qm, const float* a_dev, const float* weight_dev,
                                                  float eps, size_t m, float* sum_dev, float* norm_dev)
{
    if (!ctx || !g || !qm || kind < 0 || kind > 1 || !g->connected || (m > 0 && (!a_dev || !sum_dev))) {
        set_last_error("tp_add_rmsnorm_prepare_pushed: NULL / unconnected argument (sum_dev is required) or bad kind");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) return kUnsupported;
    if (m * qm->w.cols > g->elems) {
        set_last_error("exchange buffers hold %zu floats, %zu x %zu requested", g->elems, m, qm->w.cols);
        return kErrShape;
    }
    if (m == 0 || qm->w.nblk == 0) return kOk;
    DeviceGuard guard(ctx->device);
    int32_t rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, m));
    if (rc != kOk) return rc;
    PushSrc p;
    fill_push_src(ctx, g, kind, p);
    ctx->launches++;
    return launch_norm_prep(ctx->stream, qm->ty, qm->w, a_dev, nullptr, weight_dev, eps, m, sum_dev, norm_dev, ctx->scratch,
                            ctx->tune, PeerSum(), p);
}

// The addresses of exchange `kind` of the two-step pushed all-reduce, as this rank sees them.
static void fill_wide_dst(const ferric_cuda_ctx* ctx, const ferric_tp_group* g, int kind, WideDst& w)
{
    const size_t pairs = wide_pairs(g->elems, g->world);
    w.world = g->world;
    w.rank = g->rank;
    w.slice = wide_slice(g->elems, g->world);
    w.parity_stride1 = w.parity_stride2 = pairs;
    w.epoch = g->wide_epoch + kind;
    w.ticket = g->wide_ticket + kind;
    w.status = g->status;
    if (ctx->tune.wait_spins > 0) w.wait_spins = ctx->tune.wait_spins;
    uint8_t* local = reinterpret_cast<uint8_t*>(g->local);
    w.recv1 = reinterpret_cast<const uint2*>(local + off_wide1(g->elems, g->world)) + (size_t)kind * 2 * pairs;
    w.recv2 = reinterpret_cast<const uint2*>(local + off_wide2(g->elems, g->world)) + (size_t)kind * 2 * pairs;
    for (int r = 0; r < g->world; r++) {
        uint8_t* peer = reinterpret_cast<uint8_t*>(g->peer_base[r]);
        w.stage1[r] = reinterpret_cast<uint2*>(peer + off_wide1(g->elems, g->world)) + (size_t)kind * 2 * pairs + (size_t)g->rank * w.slice;
        w.stage2[r] = reinterpret_cast<uint2*>(peer + off_wide2(g->elems, g->world)) + (size_t)kind * 2 * pairs;
    }
}

int32_t ferric_cuda_tp_allreduce_add_rmsnorm(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind, const float* partial_dev,
                                             const float* a_dev, const float* weight_dev, float eps, size_t rows, size_t d,
                                             float* sum_dev, float* norm_dev)
{
    return ferric_cuda_tp_allreduce_add_rmsnorm_steps(ctx, g, kind, partial_dev, a_dev, weight_dev, eps, rows, d, sum_dev, norm_dev, 7);
}

int32_t ferric_cuda_tp_allreduce_add_rmsnorm_steps(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind, const float* partial_dev,
                                                   const float* a_dev, const float* weight_dev, float eps, size_t rows, size_t d,
                                                   float* sum_dev, float* norm_dev, int32_t steps)
{
    if (steps < 1 || steps > 7) {
        set_last_error("tp_allreduce_add_rmsnorm_steps: steps is a mask of 1 (scatter), 2 (reduce), 4 (consume)");
        return kErrInvalidArg;
    }
    if (!ctx || !g || kind < 0 || kind > 1 || !g->connected || (rows * d > 0 && (!partial_dev || !a_dev || !sum_dev))) {
        set_last_error("tp_allreduce_add_rmsnorm: NULL / unconnected argument (sum_dev is required) or bad kind");
        return kErrInvalidArg;
    }
    if (rows * d > g->elems || (d & 3) || (reinterpret_cast<uintptr_t>(partial_dev) & 15) || (reinterpret_cast<uintptr_t>(a_dev) & 15) ||
        (reinterpret_cast<uintptr_t>(sum_dev) & 15) || (reinterpret_cast<uintptr_t>(norm_dev) & 15) ||
        (reinterpret_cast<uintptr_t>(weight_dev) & 15)) {
        set_last_error("tp_allreduce_add_rmsnorm: %zu x %zu floats must fit the group's %zu, d be a multiple of 4 and the buffers 16-byte aligned",
                       rows, d, g->elems);
        return kErrShape;
    }
    if (rows * d == 0) return kOk;
    DeviceGuard guard(ctx->device);
    WideDst w;
    fill_wide_dst(ctx, g, kind, w);
    ctx->launches += (steps & 1) + ((steps >> 1) & 1) + ((steps >> 2) & 1);
    return launch_wide_allreduce_add_rmsnorm(ctx->stream, partial_dev, a_dev, weight_dev, eps, rows, d, sum_dev, norm_dev, w, ctx->tune,
                                             steps);
}

int32_t ferric_cuda_tp_matmul_scatter(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind, const ferric_qmatrix* qm,
                                      const float* x_dev, size_t m, size_t ldx, int32_t* fused_out)
{
    if (fused_out) *fused_out = 0;
    if (!ctx || !g || !qm || kind < 0 || kind > 1 || !g->connected || (m > 0 && !x_dev)) {
        set_last_error("tp_matmul_scatter: NULL / unconnected argument or bad kind");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) return kUnsupported;
    if (ldx == 0) ldx = qm->w.cols;
    if (ldx < qm->w.cols || (ldx & 3) || (reinterpret_cast<uintptr_t>(x_dev) & 15)) {
        set_last_error("row stride ldx %zu must cover the row and be a multiple of 4, x 16-byte aligned", ldx);
        return kErrShape;
    }
    if (m * qm->w.rows > g->elems || (qm->w.rows & 3)) {
        set_last_error("exchange buffers hold %zu floats, %zu x %zu requested (rows must be a multiple of 4)", g->elems, m, qm->w.rows);
        return kErrShape;
    }
    if (m == 0 || qm->w.rows == 0) return kOk;
    if (qm->w.nblk == 0) {
        set_last_error("tp_matmul_scatter: empty K range");
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    WideDst w;
    fill_wide_dst(ctx, g, kind, w);
    float* part = g->part[kind];
    int32_t rc;
    bool fused = false;
    if (gemv_tc_eligible(qm->ty, qm->w, m)) {
        if ((rc = ensure_scratch(ctx, gemv_tc_scratch_bytes(qm->ty, qm->w, m, kEpiStore, ctx->tune.sm_count))) != kOk) return rc;
        int launched = 0;
        rc = launch_gemv_tc(ctx->stream, qm->ty, qm->w, x_dev, m, ldx, part, qm->w.rows, kEpiStore, ctx->scratch, ctx->tune, &launched, &w,
                            &fused);
        ctx->launches += launched;
    } else {
        if ((rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, m))) != kOk) return rc;
        if ((rc = launch_prep(ctx->stream, qm->ty, qm->w, x_dev, m, ldx, ctx->scratch, ctx->tune)) != kOk) return rc;
        ctx->launches += 2;
        rc = launch_gemv(ctx->stream, qm->ty, qm->w, ctx->scratch, m, part, qm->w.rows, kEpiStore, ctx->tune);
    }
    if (rc != kOk) return rc;
    if (fused_out) *fused_out = fused ? 1 : 0;
    if (fused) return kOk;
    ctx->launches++;
    return launch_wide_allreduce_add_rmsnorm(ctx->stream, part, nullptr, nullptr, 0.0f, m, qm->w.rows, nullptr, nullptr, w, ctx->tune, 1);
}

int32_t ferric_cuda_tp_status(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t* timed_out)
{
    if (!ctx || !g || !timed_out) {
        set_last_error("NULL argument");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    FERRIC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    int s = 0;
    FERRIC_CUDA_TRY(cudaMemcpy(&s, g->status, sizeof(int), cudaMemcpyDeviceToHost));
    *timed_out = s;
    if (s) {
        set_last_error("a peer did not announce its partial within the wait bound");
        return kErrTimeout;
    }
    return kOk;
}

int32_t ferric_cuda_tp_chain_matmul(ferric_cuda_ctx* ctx, ferric_tp_group* g, int32_t kind, const ferric_chain_link* link, size_t m)
{
    if (!g || kind < 0 || kind > 1 || !g->connected) {
        set_last_error("tp_chain_matmul: NULL / unconnected group or bad kind");
        return kErrInvalidArg;
    }
    Chain chain;
    const void* frag = nullptr;
    Epilogue epi = kEpiStore;
    size_t ldy = 0;
    int32_t rc = chain_setup(ctx, link, m, true, &chain, &frag, &epi, &ldy);
    if (rc != kOk) return rc;
    const ferric_qmatrix* qm = link->qm;
    if (m * qm->w.rows > g->elems) {
        set_last_error("exchange buffers hold %zu floats, %zu x %zu requested", g->elems, m, qm->w.rows);
        return kErrShape;
    }
    if (m == 0 || qm->w.rows == 0) return kOk;
    if (qm->w.nblk == 0) {
        set_last_error("tp_chain_matmul: empty K range");
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    PushDst p;
    fill_push_dst(g, kind, p);
    fill_push_src(ctx, g, kind, chain.job.pushed);
    ctx->launches++;
    // ldy of a pushed product is the row length in the receive regions
    return launch_gemv(ctx->stream, qm->ty, qm->w, frag, m, nullptr, qm->w.rows, kEpiPush, ctx->tune, p, &chain);
}

int32_t ferric_cuda_tp_reset(ferric_cuda_ctx* ctx, ferric_tp_group* g)
{
    if (!ctx || !g) {
        set_last_error("NULL argument");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    FERRIC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    // everything but the peers' slot tables: partial buffers, flags, counters, status, receive regions
    uint8_t* base = reinterpret_cast<uint8_t*>(g->local);
    FERRIC_CUDA_TRY(cudaMemset(base, 0, off_slots(g->elems)));
    FERRIC_CUDA_TRY(cudaMemset(base + off_push_meta(g->elems), 0, g->local_bytes - off_push_meta(g->elems)));
    g->last_signal_kind = -1;
    return kOk;
}

void ferric_cuda_tp_free(ferric_tp_group* g)
{
    if (!g) return;
    DeviceGuard guard(g->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < g->world; r++)
        if (r != g->rank && g->peer_base[r] && !g->local_peers) cudaIpcCloseMemHandle(g->peer_base[r]);
    cudaFree(g->local);
    delete g;
}

}  // extern "C"
