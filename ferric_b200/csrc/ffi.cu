// The C ABI (include/ferric_cuda.h): argument checking, ownership, stream plumbing.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <time.h>

#include <algorithm>
#include <new>
#include <string>
#include <vector>

#include "../../include/ferric_cuda.h"
#include "common.cuh"
#include "kernels.h"
#include "handles.h"

namespace ferric {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
    va_end(ap);
}

int32_t cuda_fail(cudaError_t e, const char* what)
{
    set_last_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? kErrOom : kErrCuda;
}

}  // namespace ferric

using namespace ferric;

namespace ferric {
int32_t ensure_scratch(ferric_cuda_ctx* ctx, size_t bytes)
{
    if (bytes <= ctx->scratch_bytes) return kOk;
    // Stream-ordered, so a buffer still read by queued kernels is released only after them.
    if (ctx->scratch) FERRIC_CUDA_TRY(cudaFreeAsync(ctx->scratch, ctx->stream));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes + bytes / 4 + 4096;
    FERRIC_CUDA_TRY(cudaMallocAsync(&ctx->scratch, want, ctx->stream));
    ctx->scratch_bytes = want;
    return kOk;
}

}  // namespace ferric

namespace {

bool block_info(uint32_t ty, size_t* vals, size_t* bytes)
{
    switch (ty) {
    case kGgmlQ8_0: *vals = 32; *bytes = 34; return true;
    case kGgmlQ4K: *vals = 256; *bytes = 144; return true;
    case kGgmlQ5K: *vals = 256; *bytes = 176; return true;
    case kGgmlQ6K: *vals = 256; *bytes = 210; return true;
    default: return false;
    }
}

int32_t check_matmul_args(const ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const void* x, size_t m,
                          size_t x_cols, const void* y)
{
    if (!ctx || !qm) {
        set_last_error("NULL context or matrix handle");
        return kErrInvalidArg;
    }
    if (qm->device != ctx->device) {
        set_last_error("matrix lives on device %d, context on device %d", qm->device, ctx->device);
        return kErrInvalidArg;
    }
    if (x_cols != qm->w.cols) {
        set_last_error("inner dim mismatch: x[..,%zu] vs W[..,%zu]", x_cols, qm->w.cols);
        return kErrShape;
    }
    if (m > 0 && ((!x && qm->w.cols > 0) || (!y && qm->w.rows > 0))) {
        set_last_error("NULL activation or result buffer");
        return kErrInvalidArg;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 3)) {
        set_last_error("activation buffer must be 16-byte aligned (result 4-byte)");
        return kErrInvalidArg;
    }
    return kOk;
}

int32_t build_matrix(ferric_cuda_ctx* ctx, const uint8_t* bytes, bool on_device, size_t len, uint32_t ty,
                     size_t rows, size_t cols, size_t row0, size_t nrows, size_t col0, size_t ncols,
                     ferric_qmatrix** out)
{
    if (!ctx || !out) {
        set_last_error("NULL context or output pointer");
        return kErrInvalidArg;
    }
    *out = nullptr;
    size_t vals, bbytes;
    if (!block_info(ty, &vals, &bbytes)) {
        set_last_error("QMatrix: no native matmul for ggml type %u", ty);
        return kErrUnsupportedType;
    }
    if (cols % vals != 0) {
        set_last_error("cols (%zu) must be a multiple of %zu for ggml type %u", cols, vals, ty);
        return kErrShape;
    }
    // the kernels index rows and columns with 32-bit integers, and the size arithmetic below must not wrap
    if (rows > (size_t)INT32_MAX || cols > (size_t)INT32_MAX) {
        set_last_error("matrix [%zu, %zu] is larger than this backend indexes (2^31 - 1 rows / columns)", rows, cols);
        return kErrShape;
    }
    size_t want_len = 0;
    if (__builtin_mul_overflow(rows, cols / vals, &want_len) || __builtin_mul_overflow(want_len, bbytes, &want_len)) {
        set_last_error("byte size of [%zu, %zu] of ggml type %u overflows", rows, cols, ty);
        return kErrShape;
    }
    if (len != want_len) {
        set_last_error("unexpected byte length %zu for [%zu, %zu] of ggml type %u (want %zu)", len, rows, cols, ty, want_len);
        return kErrShape;
    }
    if (row0 + nrows > rows || col0 + ncols > cols || col0 % vals != 0 || ncols % vals != 0) {
        set_last_error("sub-matrix [%zu+%zu, %zu+%zu] outside [%zu, %zu] or not block aligned", row0, nrows, col0,
                       ncols, rows, cols);
        return kErrShape;
    }
    if (len > 0 && !bytes) {
        set_last_error("NULL weight bytes");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");

    ferric_qmatrix* qm = new (std::nothrow) ferric_qmatrix;
    if (!qm) return kErrOom;
    qm->ty = ty;
    qm->device = ctx->device;
    qm->w.rows = nrows;
    qm->w.cols = ncols;
    qm->w.nblk = ncols / vals;
    size_t src_nblk = cols / vals, blk0 = col0 / vals;

    size_t bytes_needed, d_off = 0;
    if (ty == kGgmlQ8_0) {
        d_off = (nrows * ncols + 255) / 256 * 256;
        bytes_needed = d_off + nrows * qm->w.nblk * 2;
    } else {
        bytes_needed = qm->w.row_tiles() * qm->w.nblk * 16 * bbytes;
    }
    if (bytes_needed == 0) bytes_needed = 16;
    cudaError_t e = cudaMalloc(&qm->storage, bytes_needed);
    if (e != cudaSuccess) {
        delete qm;
        return cuda_fail(e, "cudaMalloc(weights)");
    }
    qm->storage_bytes = bytes_needed;
    if (ty == kGgmlQ8_0) {
        qm->w.q8_qs = reinterpret_cast<int8_t*>(qm->storage);
        qm->w.q8_d = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(qm->storage) + d_off);
    } else {
        qm->w.units = reinterpret_cast<uint8_t*>(qm->storage);
    }

    int32_t rc = kOk;
    void* staging = nullptr;
    do {
        // rows past `nrows` in the last 16-row tile stay zero (d = 0 -> they contribute nothing)
        if ((e = cudaMemsetAsync(qm->storage, 0, bytes_needed, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemsetAsync"); break; }
        const uint8_t* src = bytes;
        if (!on_device && len > 0) {
            // stage only the row range that is needed
            size_t row_bytes = src_nblk * bbytes, off = row0 * row_bytes, n = nrows * row_bytes;
            if (n > 0) {
                if ((e = cudaMalloc(&staging, n)) != cudaSuccess) { rc = cuda_fail(e, "cudaMalloc(staging)"); break; }
                if ((e = cudaMemcpyAsync(staging, bytes + off, n, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(weights)"); break; }
            }
            src = reinterpret_cast<const uint8_t*>(staging);
            row0 = 0;
        }
        if (nrows > 0 && qm->w.nblk > 0) {
            rc = launch_repack(ctx->stream, ty, src, qm->w, src_nblk, row0, blk0);
            ctx->launches++;
        }
        if (rc != kOk) break;
        // the host bytes / staging buffer must not be needed after return
        if ((e = cudaStreamSynchronize(ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaStreamSynchronize"); break; }
    } while (0);
    if (staging) cudaFree(staging);
    if (rc != kOk) {
        cudaFree(qm->storage);
        delete qm;
        return rc;
    }
    *out = qm;
    return kOk;
}

// phases: 1 = prepare activation fragments, 2 = product from prepared fragments, 3 = both
int32_t run_matmul(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x, size_t m, size_t ldx, float* y,
                   size_t ldy, Epilogue epi, int phases = 3)
{
    if (m == 0 || qm->w.rows == 0) return kOk;
    const size_t out_cols = epi == kEpiSwiglu ? qm->w.rows / 2 : qm->w.rows;
    if (ldx == 0) ldx = qm->w.cols;
    if (ldy == 0) ldy = out_cols;
    if (ldx < qm->w.cols || ldy < out_cols || (ldx & 3)) {
        set_last_error("row strides (ldx %zu, ldy %zu) must cover the rows and ldx be a multiple of 4", ldx, ldy);
        return kErrShape;
    }
    if (!has_prepared_form(qm->ty)) {
        if (!(phases & 2)) return kOk;
        if (!x) {
            set_last_error("this format has no prepared form: pass the activations");
            return kErrInvalidArg;
        }
        if (epi != kEpiStore) return kUnsupported;
        ctx->launches++;
        if (qm->ty == kGgmlF32) return launch_gemv_f32(ctx->stream, qm->w, x, m, ldx, y, ldy, ctx->tune);
        return launch_gemv_q8_0(ctx->stream, qm->w, x, m, ldx, y, ldy, ctx->tune);
    }
    if (qm->w.nblk == 0) {  // cols == 0: an empty sum
        if (phases & 2) FERRIC_CUDA_TRY(cudaMemset2DAsync(y, ldy * sizeof(float), 0, out_cols * sizeof(float), m, ctx->stream));
        return kOk;
    }
    int32_t rc = kOk;
    if (phases == 3 && gemv_tc_eligible(qm->ty, qm->w, m)) {
        // more than a few activation rows: the exact-integer tensor-core kernel (its own activation form)
        if ((rc = ensure_scratch(ctx, gemv_tc_scratch_bytes(qm->ty, qm->w, m, epi, ctx->tune.sm_count))) != kOk) return rc;
        int launched = 0;
        rc = launch_gemv_tc(ctx->stream, qm->ty, qm->w, x, m, ldx, y, ldy, epi, ctx->scratch, ctx->tune, &launched);
        ctx->launches += launched;
        return rc;
    }
    const size_t need = frag_bytes(qm->ty, qm->w, m);
    if (phases & 1) {
        if ((rc = ensure_scratch(ctx, need)) != kOk) return rc;
        if ((rc = launch_prep(ctx->stream, qm->ty, qm->w, x, m, ldx, ctx->scratch, ctx->tune)) != kOk) return rc;
        ctx->launches++;
    }
    if (phases & 2) {
        if (ctx->scratch_bytes < need) {
            set_last_error("no prepared activations on this context for m = %zu", m);
            return kErrInvalidArg;
        }
        rc = launch_gemv(ctx->stream, qm->ty, qm->w, ctx->scratch, m, y, ldy, epi, ctx->tune);
        ctx->launches++;
    }
    return rc;
}

}  // namespace

extern "C" {

const char* ferric_cuda_last_error(void) { return g_last_error; }

int32_t ferric_gguf_type_size(uint32_t ty, size_t n, size_t* out_bytes)
{
    if (!out_bytes) {
        set_last_error("NULL output pointer");
        return kErrInvalidArg;
    }
    if ((ty == FERRIC_GGML_F32 && n > SIZE_MAX / 4) || ((ty == FERRIC_GGML_F16 || ty == FERRIC_GGML_BF16) && n > SIZE_MAX / 2)) {
        set_last_error("byte size of %zu elements of ggml type %u overflows", n, ty);
        return kErrShape;
    }
    switch (ty) {
    case FERRIC_GGML_F32: *out_bytes = n * 4; return kOk;
    case FERRIC_GGML_F16: *out_bytes = n * 2; return kOk;
    case FERRIC_GGML_BF16: *out_bytes = n * 2; return kOk;
    case FERRIC_GGML_Q8_0: *out_bytes = n / 32 * 34; return kOk;
    case FERRIC_GGML_Q4_K: *out_bytes = n / 256 * 144; return kOk;
    case FERRIC_GGML_Q5_K: *out_bytes = n / 256 * 176; return kOk;
    case FERRIC_GGML_Q6_K: *out_bytes = n / 256 * 210; return kOk;
    default:
        set_last_error("unsupported ggml type %u", ty);
        return kErrUnsupportedType;
    }
}

int32_t ferric_cuda_qmatrix_block_bytes(uint32_t ty, size_t* vals, size_t* bytes)
{
    if (!vals || !bytes) {
        set_last_error("NULL output pointer");
        return kErrInvalidArg;
    }
    if (!block_info(ty, vals, bytes)) return kUnsupported;
    return kOk;
}

int32_t ferric_cuda_ctx_create_on_stream(int device, void* cuda_stream, ferric_cuda_ctx** out)
{
    if (!out) {
        set_last_error("NULL output pointer");
        return kErrInvalidArg;
    }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        set_last_error("no CUDA device available (%s); this backend has no CPU fallback",
                       e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        return kErrCuda;
    }
    if (device < 0 || device >= count) {
        set_last_error("device %d out of range [0, %d)", device, count);
        return kErrInvalidArg;
    }
    DeviceGuard guard(device);
    if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
    ferric_cuda_ctx* ctx = new (std::nothrow) ferric_cuda_ctx;
    if (!ctx) return kErrOom;
    ctx->device = device;
    ctx->stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    if ((e = cudaGetDeviceProperties(&ctx->prop, device)) != cudaSuccess) {
        delete ctx;
        return cuda_fail(e, "cudaGetDeviceProperties");
    }
    if (ctx->prop.major < 10) {
        set_last_error("device %d is sm_%d%d; this library holds sm_100a code only", device, ctx->prop.major,
                       ctx->prop.minor);
        delete ctx;
        return kErrCuda;
    }
    ctx->tune.sm_count = ctx->prop.multiProcessorCount;
    if (const char* s = getenv("FERRIC_CUDA_GEMV_WK")) ctx->tune.wk = atoi(s);
    if (const char* s = getenv("FERRIC_CUDA_PDL")) ctx->tune.pdl = atoi(s) != 0;
    if (const char* s = getenv("FERRIC_CUDA_PUSH_CLUSTER")) ctx->tune.push_cluster = atoi(s);
    if (const char* s = getenv("FERRIC_CUDA_GEMV_STREAM")) ctx->tune.stream = atoi(s) != 0;
    if (const char* s = getenv("FERRIC_CUDA_GEMV_STREAM_CTAS")) ctx->tune.stream_ctas = atoi(s);
    if (const char* s = getenv("FERRIC_CUDA_PEER_WAIT_SPINS")) ctx->tune.wait_spins = atoi(s) > 0 ? atoi(s) : 0;
    {
        const size_t chain_words = kChainMaxRows * kChainMaxBlocks + kChainMaxBlocks + 64;
        const size_t bytes = kSplitWsFloats * sizeof(float) + kSplitTickets * sizeof(unsigned) + chain_words * 4;
        void* ws = nullptr;
        cudaError_t e2 = cudaMalloc(&ws, bytes);
        if (e2 == cudaSuccess) e2 = cudaMemset(ws, 0, bytes);
        if (e2 != cudaSuccess) {
            if (ws) cudaFree(ws);
            if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
            delete ctx;
            return cuda_fail(e2, "cudaMalloc(split workspace)");
        }
        ctx->tune.split_ws.partial = reinterpret_cast<float*>(ws);
        ctx->tune.split_ws.tickets = reinterpret_cast<unsigned*>(ctx->tune.split_ws.partial + kSplitWsFloats);
        ctx->chain_ssq = reinterpret_cast<float*>(ctx->tune.split_ws.tickets + kSplitTickets);
        ctx->chain_tickets = reinterpret_cast<unsigned*>(ctx->chain_ssq + kChainMaxRows * kChainMaxBlocks);
        ctx->chain_done = ctx->chain_tickets + kChainMaxBlocks;
    }
    *out = ctx;
    return kOk;
}

int32_t ferric_cuda_ctx_create(int device, ferric_cuda_ctx** out)
{
    int32_t rc = ferric_cuda_ctx_create_on_stream(device, nullptr, out);
    if (rc != kOk) return rc;
    DeviceGuard guard(device);
    cudaError_t e = cudaStreamCreateWithFlags(&(*out)->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete *out;
        *out = nullptr;
        return cuda_fail(e, "cudaStreamCreateWithFlags");
    }
    (*out)->owns_stream = true;
    return kOk;
}

int32_t ferric_cuda_ctx_set_stream(ferric_cuda_ctx* ctx, void* cuda_stream)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    if (ctx->owns_stream) {
        DeviceGuard guard(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
        ctx->owns_stream = false;
    }
    ctx->stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    return kOk;
}

void* ferric_cuda_ctx_stream(const ferric_cuda_ctx* ctx) { return ctx ? ctx->stream : nullptr; }

int32_t ferric_cuda_ctx_sync(ferric_cuda_ctx* ctx)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    FERRIC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return kOk;
}

void ferric_cuda_ctx_free(ferric_cuda_ctx* ctx)
{
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->tune.split_ws.partial) cudaFree(ctx->tune.split_ws.partial);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int32_t ferric_cuda_ctx_caps(const ferric_cuda_ctx* ctx, ferric_cuda_caps* out)
{
    if (!ctx || !out) {
        set_last_error("NULL context or output pointer");
        return kErrInvalidArg;
    }
    out->device = ctx->device;
    out->sm_count = ctx->prop.multiProcessorCount;
    out->cc_major = ctx->prop.major;
    out->cc_minor = ctx->prop.minor;
    out->l2_bytes = (uint64_t)ctx->prop.l2CacheSize;
    out->total_mem_bytes = (uint64_t)ctx->prop.totalGlobalMem;
    out->max_smem_per_block = (uint64_t)ctx->prop.sharedMemPerBlockOptin;
    return kOk;
}

int32_t ferric_cuda_ctx_reserve_scratch(ferric_cuda_ctx* ctx, size_t bytes)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    return ensure_scratch(ctx, bytes);
}

uint64_t ferric_cuda_ctx_launches(const ferric_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

// prof / prof_report (crates/ferric-tensor/src/lib.rs:3017-3046): synchronise, then charge the time since the previous
// mark to a named bucket.  It serialises the stream, so it shows where the time goes, not the fastest achievable.
static double host_ms()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

int32_t ferric_cuda_prof_enable(ferric_cuda_ctx* ctx, int32_t on)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    ctx->prof_on = on != 0;
    ctx->prof_marked = false;
    return kOk;
}

int32_t ferric_cuda_prof(ferric_cuda_ctx* ctx, const char* label)
{
    if (!ctx || !label) {
        set_last_error("NULL context or label");
        return kErrInvalidArg;
    }
    if (!ctx->prof_on) return kOk;
    DeviceGuard guard(ctx->device);
    FERRIC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    const double now = host_ms();
    if (ctx->prof_marked) ctx->prof[label] += now - ctx->prof_prev_ms;
    ctx->prof_prev_ms = now;
    ctx->prof_marked = true;
    return kOk;
}

int32_t ferric_cuda_prof_report(ferric_cuda_ctx* ctx, char* buf, size_t cap, size_t* len)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    std::vector<std::pair<std::string, double>> v(ctx->prof.begin(), ctx->prof.end());
    std::sort(v.begin(), v.end(), [](const auto& a, const auto& b) { return a.second > b.second; });
    double total = 0.0;
    for (const auto& e : v) total += e.second;
    char line[256];
    std::string out;
    snprintf(line, sizeof line, "profile (ms, %.3f total)\n", total);
    out += line;
    for (const auto& e : v) {
        snprintf(line, sizeof line, "  %-24s %10.3f  %5.1f%%\n", e.first.c_str(), e.second, total > 0 ? 100.0 * e.second / total : 0.0);
        out += line;
    }
    if (len) *len = out.size();
    if (buf && cap > 0) {
        const size_t n = std::min(cap - 1, out.size());
        memcpy(buf, out.data(), n);
        buf[n] = 0;
        if (cap > out.size()) {   // the whole report was delivered: reset, as the reference does after printing
            ctx->prof.clear();
            ctx->prof_marked = false;
        }
    }
    return kOk;
}

int32_t ferric_cuda_qmatrix_from_bytes(ferric_cuda_ctx* ctx, const uint8_t* bytes, size_t len, uint32_t ty,
                                       size_t rows, size_t cols, ferric_qmatrix** out)
{
    return build_matrix(ctx, bytes, false, len, ty, rows, cols, 0, rows, 0, cols, out);
}

int32_t ferric_cuda_qmatrix_from_bytes_view(ferric_cuda_ctx* ctx, const uint8_t* bytes, size_t len, uint32_t ty,
                                            size_t rows, size_t cols, size_t row0, size_t nrows, size_t col0,
                                            size_t ncols, ferric_qmatrix** out)
{
    return build_matrix(ctx, bytes, false, len, ty, rows, cols, row0, nrows, col0, ncols, out);
}

int32_t ferric_cuda_qmatrix_from_device_bytes(ferric_cuda_ctx* ctx, const uint8_t* bytes_dev, size_t len, uint32_t ty,
                                              size_t rows, size_t cols, ferric_qmatrix** out)
{
    return build_matrix(ctx, bytes_dev, true, len, ty, rows, cols, 0, rows, 0, cols, out);
}

int32_t ferric_cuda_qmatrix_from_dense(ferric_cuda_ctx* ctx, const float* w_host, size_t rows, size_t cols, ferric_qmatrix** out)
{
    if (!ctx || !out || (rows * cols > 0 && !w_host)) {
        set_last_error("NULL context, weights or output pointer");
        return kErrInvalidArg;
    }
    *out = nullptr;
    size_t bytes = 0;
    if (rows > (size_t)INT32_MAX || cols > (size_t)INT32_MAX || __builtin_mul_overflow(rows, cols, &bytes) ||
        __builtin_mul_overflow(bytes, sizeof(float), &bytes)) {
        set_last_error("matrix [%zu, %zu] is larger than this backend indexes", rows, cols);
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    if (!guard.ok) return cuda_fail(cudaGetLastError(), "cudaSetDevice");
    ferric_qmatrix* qm = new (std::nothrow) ferric_qmatrix;
    if (!qm) return kErrOom;
    qm->ty = kGgmlF32;
    qm->device = ctx->device;
    qm->w.rows = rows;
    qm->w.cols = cols;
    qm->storage_bytes = bytes ? bytes : 16;
    cudaError_t e = cudaMalloc(&qm->storage, qm->storage_bytes);
    if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(qm->storage, w_host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // the host pointer is not kept
    if (e != cudaSuccess) {
        if (qm->storage) cudaFree(qm->storage);
        delete qm;
        return cuda_fail(e, "qmatrix_from_dense");
    }
    qm->w.dense = reinterpret_cast<float*>(qm->storage);
    *out = qm;
    return kOk;
}

size_t ferric_cuda_qmatrix_rows(const ferric_qmatrix* qm) { return qm ? qm->w.rows : 0; }
size_t ferric_cuda_qmatrix_cols(const ferric_qmatrix* qm) { return qm ? qm->w.cols : 0; }
size_t ferric_cuda_qmatrix_nbytes(const ferric_qmatrix* qm)
{
    if (!qm) return 0;
    if (qm->ty == kGgmlF32) return qm->w.rows * qm->w.cols * sizeof(float);   // DenseWeight::nbytes, dtype.rs:826
    size_t vals, bytes;
    block_info(qm->ty, &vals, &bytes);
    return qm->w.rows * (qm->w.cols / vals) * bytes;
}
size_t ferric_cuda_qmatrix_n_shards(const ferric_qmatrix* qm) { return qm ? 1 : 0; }
uint32_t ferric_cuda_qmatrix_ggml_type(const ferric_qmatrix* qm) { return qm ? qm->ty : 0; }

void ferric_cuda_qmatrix_free(ferric_qmatrix* qm)
{
    if (!qm) return;
    DeviceGuard guard(qm->device);
    cudaFree(qm->storage);
    delete qm;
}

size_t ferric_cuda_qmatrix_scratch_bytes(const ferric_qmatrix* qm, size_t m)
{
    if (!qm) return 0;
    size_t need = frag_bytes(qm->ty, qm->w, m);
    if (gemv_tc_eligible(qm->ty, qm->w, m)) {
        // the tensor-core decode path keeps limbs, sums and K-split partials there; the SwiGLU form needs the most
        const size_t tc = gemv_tc_scratch_bytes(qm->ty, qm->w, m, kEpiSwiglu, 148);
        if (tc > need) need = tc;
    }
    // the bf16 prefill product cuts the tiles of a partly filled last wave along K and meets their pieces there
    const size_t ws = gemm_workspace_bytes(qm->w, m, 148);
    if (ws > need) need = ws;
    return need;
}

int32_t ferric_cuda_matmul_q(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t m,
                             size_t x_cols, float* y_dev)
{
    int32_t rc = check_matmul_args(ctx, qm, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    DeviceGuard guard(ctx->device);
    return run_matmul(ctx, qm, x_dev, m, 0, y_dev, 0, kEpiStore);
}

int32_t ferric_cuda_matmul_q_bf16(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const uint16_t* x_bf16_dev, size_t m,
                                  size_t x_cols, float* y_dev)
{
    int32_t rc = check_matmul_args(ctx, qm, x_bf16_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    if (m > (size_t)INT32_MAX || qm->w.rows > (size_t)INT32_MAX) {
        set_last_error("matrix or batch too large");
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    // tiles of a partly filled last wave are cut along K; their pieces meet in the context's scratch
    const size_t ws = gemm_workspace_bytes(qm->w, m, ctx->tune.sm_count);
    if (ws > 0 && (rc = ensure_scratch(ctx, ws)) != kOk) return rc;
    ctx->launches += ws > 0 ? 2 : 1;
    return launch_gemm_bf16(ctx->stream, qm->ty, qm->w, x_bf16_dev, m, qm->w.cols, y_dev, qm->w.rows, ws > 0 ? ctx->scratch : nullptr,
                            ctx->tune.sm_count);
}

int32_t ferric_cuda_gemm_status(ferric_cuda_ctx* ctx, int32_t* code)
{
    if (!ctx || !code) {
        set_last_error("NULL argument");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    int v = 0;
    int32_t rc = gemm_status(ctx->stream, &v);
    if (rc != kOk) return rc;
    *code = v;
    if (v) {
        set_last_error("a tensor-core GEMM block gave up waiting (role code %d)", v);
        return kErrTimeout;
    }
    return kOk;
}

int32_t ferric_cuda_matmul_q_swiglu(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t m,
                                    size_t x_cols, float* y_dev)
{
    int32_t rc = check_matmul_args(ctx, qm, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    if (!has_prepared_form(qm->ty) || qm->w.rows % 32 != 0) return kUnsupported;
    DeviceGuard guard(ctx->device);
    return run_matmul(ctx, qm, x_dev, m, 0, y_dev, 0, kEpiSwiglu);
}

int32_t ferric_cuda_matmul_q_ld(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t m,
                                size_t x_cols, size_t ldx, float* y_dev, size_t ldy)
{
    int32_t rc = check_matmul_args(ctx, qm, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    DeviceGuard guard(ctx->device);
    return run_matmul(ctx, qm, x_dev, m, ldx, y_dev, ldy, kEpiStore);
}

int32_t ferric_cuda_prepare_x(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t m,
                              size_t x_cols, size_t ldx)
{
    float dummy;
    int32_t rc = check_matmul_args(ctx, qm, x_dev, m, x_cols, &dummy);
    if (rc != kOk) return rc;
    if (!has_prepared_form(qm->ty)) {
        set_last_error("Q8_0 and dense matrices have no prepared form");
        return kUnsupported;
    }
    DeviceGuard guard(ctx->device);
    return run_matmul(ctx, qm, x_dev, m, ldx, nullptr, 0, kEpiStore, 1);
}

int32_t ferric_cuda_matmul_q_prepared(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, size_t m, float* y_dev,
                                      size_t ldy, int32_t swiglu)
{
    if (!ctx || !qm || (m > 0 && !y_dev && qm->w.rows > 0)) {
        set_last_error("NULL context, matrix or result buffer");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) {
        set_last_error("Q8_0 and dense matrices have no prepared form");
        return kUnsupported;
    }
    if (swiglu && qm->w.rows % 32 != 0) return kUnsupported;
    DeviceGuard guard(ctx->device);
    return run_matmul(ctx, qm, nullptr, m, 0, y_dev, ldy, swiglu ? kEpiSwiglu : kEpiStore, 2);
}

int32_t ferric_cuda_add_rmsnorm(ferric_cuda_ctx* ctx, const float* a_dev, const float* b_dev, const float* weight_dev,
                                float eps, size_t rows, size_t d, float* sum_dev, float* norm_dev)
{
    if (!ctx || (rows * d > 0 && (!a_dev || !norm_dev))) {
        set_last_error("NULL context or buffer");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    ctx->launches++;
    return launch_add_rmsnorm(ctx->stream, a_dev, b_dev, weight_dev, eps, rows, d, sum_dev, norm_dev, ctx->tune);
}

int32_t ferric_cuda_add_rmsnorm_prepare(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* a_dev,
                                        const float* b_dev, const float* weight_dev, float eps, size_t m, float* sum_dev,
                                        float* norm_dev)
{
    if (!ctx || !qm || (m > 0 && !a_dev)) {
        set_last_error("NULL context, matrix or buffer");
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) {
        set_last_error("Q8_0 and dense matrices have no prepared form");
        return kUnsupported;
    }
    if ((reinterpret_cast<uintptr_t>(a_dev) | reinterpret_cast<uintptr_t>(b_dev) | reinterpret_cast<uintptr_t>(sum_dev) |
         reinterpret_cast<uintptr_t>(norm_dev) | reinterpret_cast<uintptr_t>(weight_dev)) & 15) {
        set_last_error("buffers must be 16-byte aligned");
        return kErrInvalidArg;
    }
    if (m == 0 || qm->w.nblk == 0) return kOk;
    DeviceGuard guard(ctx->device);
    int32_t rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, m));
    if (rc != kOk) return rc;
    ctx->launches++;
    return launch_norm_prep(ctx->stream, qm->ty, qm->w, a_dev, b_dev, weight_dev, eps, m, sum_dev, norm_dev, ctx->scratch,
                            ctx->tune);
}

int32_t ferric_cuda_matmul_q_host(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_host, size_t m,
                                  size_t x_cols, float* y_host)
{
    if (!ctx || !qm) {
        set_last_error("NULL context or matrix handle");
        return kErrInvalidArg;
    }
    if (x_cols != qm->w.cols) {
        set_last_error("inner dim mismatch: x[..,%zu] vs W[..,%zu]", x_cols, qm->w.cols);
        return kErrShape;
    }
    if (m == 0) return kOk;
    if (!x_host || !y_host) {
        set_last_error("NULL activation or result buffer");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    size_t xb = m * x_cols * sizeof(float), yb = m * qm->w.rows * sizeof(float);
    size_t xoff = (xb + 255) / 256 * 256;
    void* buf = nullptr;
    FERRIC_CUDA_TRY(cudaMallocAsync(&buf, xoff + yb + 16, ctx->stream));
    float* xd = reinterpret_cast<float*>(buf);
    float* yd = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(buf) + xoff);
    int32_t rc = kOk;
    cudaError_t e;
    do {
        if (xb && (e = cudaMemcpyAsync(xd, x_host, xb, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(x)"); break; }
        if ((rc = run_matmul(ctx, qm, xd, m, 0, yd, 0, kEpiStore)) != kOk) break;
        if (yb && (e = cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(y)"); break; }
    } while (0);
    cudaFreeAsync(buf, ctx->stream);
    e = cudaStreamSynchronize(ctx->stream);
    if (rc == kOk && e != cudaSuccess) rc = cuda_fail(e, "cudaStreamSynchronize");
    return rc;
}

int32_t ferric_cuda_swiglu(ferric_cuda_ctx* ctx, const float* gu_dev, size_t t, size_t d, float* out_dev)
{
    if (!ctx || (t * d > 0 && (!gu_dev || !out_dev))) {
        set_last_error("NULL context or buffer");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    ctx->launches++;
    return launch_swiglu(ctx->stream, gu_dev, t, d, out_dev, ctx->tune);
}

int32_t ferric_cuda_dequant_f32(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, float* out_dev)
{
    if (!ctx || !qm || (!out_dev && qm->w.rows * qm->w.cols > 0)) {
        set_last_error("NULL context, matrix or output");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    if (qm->ty == kGgmlF32) {
        FERRIC_CUDA_TRY(cudaMemcpyAsync(out_dev, qm->w.dense, qm->w.rows * qm->w.cols * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        return kOk;
    }
    ctx->launches++;
    return launch_dequant_weights(ctx->stream, qm->ty, qm->w, out_dev, false);
}

int32_t ferric_cuda_dequant_bf16(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, uint16_t* out_dev)
{
    if (!ctx || !qm || (!out_dev && qm->w.rows * qm->w.cols > 0)) {
        set_last_error("NULL context, matrix or output");
        return kErrInvalidArg;
    }
    if (qm->ty == kGgmlF32) {
        set_last_error("a dense matrix has no bf16 decode");
        return kUnsupported;
    }
    DeviceGuard guard(ctx->device);
    ctx->launches++;
    return launch_dequant_weights(ctx->stream, qm->ty, qm->w, out_dev, true);
}

int32_t ferric_gguf_deq_raw(ferric_cuda_ctx* ctx, const uint8_t* raw, size_t raw_len, size_t n, uint32_t ty,
                            float* out)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    size_t vals, bbytes;
    if (!block_info(ty, &vals, &bbytes)) {
        set_last_error("unsupported ggml type %u", ty);
        return kErrUnsupportedType;
    }
    size_t need = n / vals * bbytes;
    if (raw_len < need) {
        set_last_error("raw buffer too short: %zu bytes for %zu elements of type %u (need %zu)", raw_len, n, ty, need);
        return kErrShape;
    }
    if (n == 0) return kOk;
    if (!raw || !out) {
        set_last_error("NULL buffer");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    size_t roff = (need + 255) / 256 * 256 + 256;
    void* buf = nullptr;
    FERRIC_CUDA_TRY(cudaMallocAsync(&buf, roff + n * sizeof(float), ctx->stream));
    uint8_t* rd = reinterpret_cast<uint8_t*>(buf);
    float* od = reinterpret_cast<float*>(rd + roff);
    int32_t rc = kOk;
    cudaError_t e;
    do {
        // elements past the last whole block stay zero, as in the reference (vec![0.0; n])
        if ((e = cudaMemsetAsync(od, 0, n * sizeof(float), ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemsetAsync"); break; }
        if (need && (e = cudaMemcpyAsync(rd, raw, need, cudaMemcpyHostToDevice, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(raw)"); break; }
        if ((rc = launch_dequant_raw(ctx->stream, ty, rd, n, od, false)) != kOk) break;
        ctx->launches++;
        if ((e = cudaMemcpyAsync(out, od, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream)) != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(out)"); break; }
    } while (0);
    cudaFreeAsync(buf, ctx->stream);
    e = cudaStreamSynchronize(ctx->stream);
    if (rc == kOk && e != cudaSuccess) rc = cuda_fail(e, "cudaStreamSynchronize");
    return rc;
}

// ---------------------------------------------------------------------------------------------
// Proj (crates/ferric-llama/src/qwen3.rs:192-228): a projection with several stacked outputs that is one matrix when
// the parts share a quant format and one matrix per part when they do not.
// ---------------------------------------------------------------------------------------------
int32_t ferric_cuda_proj_from_parts(ferric_qmatrix* const* parts, size_t n_parts, ferric_proj** out)
{
    if (!parts || n_parts == 0 || n_parts > 8 || !out) {
        set_last_error("proj_from_parts: NULL argument, or not 1..8 parts");
        return kErrInvalidArg;
    }
    *out = nullptr;
    for (size_t k = 0; k < n_parts; k++) {
        if (!parts[k] || parts[k]->device != parts[0]->device || parts[k]->w.cols != parts[0]->w.cols) {
            set_last_error("proj_from_parts: part %zu is NULL, on another device or has another input dim", k);
            return parts[k] && parts[k]->w.cols != parts[0]->w.cols ? kErrShape : kErrInvalidArg;
        }
    }
    ferric_proj* p = new (std::nothrow) ferric_proj;
    if (!p) return kErrOom;
    p->n_parts = n_parts;
    p->cols = parts[0]->w.cols;
    for (size_t k = 0; k < n_parts; k++) {
        p->parts[k] = parts[k];
        p->rows += parts[k]->w.rows;
    }
    *out = p;
    return kOk;
}

size_t ferric_cuda_proj_n_parts(const ferric_proj* p) { return p ? p->n_parts : 0; }
size_t ferric_cuda_proj_rows(const ferric_proj* p) { return p ? p->rows : 0; }
size_t ferric_cuda_proj_cols(const ferric_proj* p) { return p ? p->cols : 0; }
const ferric_qmatrix* ferric_cuda_proj_part(const ferric_proj* p, size_t i) { return (p && i < p->n_parts) ? p->parts[i] : nullptr; }

void ferric_cuda_proj_free(ferric_proj* p)
{
    if (!p) return;
    for (size_t k = 0; k < p->n_parts; k++) ferric_cuda_qmatrix_free(p->parts[k]);
    delete p;
}

// Proj::matmul: every part's product lands at its column offset of y[m, rows] -- the reference's matmul + cat.
// Parts that share an activation format (Q4_K and Q5_K; Q6_K) share one preparation of x.
static int32_t proj_matmul_ld(ferric_cuda_ctx* ctx, const ferric_proj* p, const float* x, size_t m, float* y, size_t ldy)
{
    int32_t rc = kOk;
    const ferric_qmatrix* prepared_for = nullptr;
    auto family = [](uint32_t ty) { return ty == kGgmlQ5K ? kGgmlQ4K : ty; };
    size_t col = 0;
    for (size_t k = 0; k < p->n_parts && rc == kOk; k++) {
        const ferric_qmatrix* qm = p->parts[k];
        float* yk = y + col;
        col += qm->w.rows;
        if (!has_prepared_form(qm->ty) || gemv_tc_eligible(qm->ty, qm->w, m) || qm->w.nblk == 0) {
            rc = run_matmul(ctx, qm, x, m, 0, yk, ldy, kEpiStore);
            prepared_for = nullptr;   // the tensor-core path uses the scratch for its own activation form
            continue;
        }
        if (!prepared_for || family(prepared_for->ty) != family(qm->ty)) {
            if ((rc = run_matmul(ctx, qm, x, m, 0, nullptr, 0, kEpiStore, 1)) != kOk) break;
            prepared_for = qm;
        }
        rc = run_matmul(ctx, qm, nullptr, m, 0, yk, ldy, kEpiStore, 2);
    }
    return rc;
}

static int32_t check_proj_args(const ferric_cuda_ctx* ctx, const ferric_proj* p, const void* x, size_t m, size_t x_cols, const void* y)
{
    if (!ctx || !p || p->n_parts == 0) {
        set_last_error("NULL context or projection");
        return kErrInvalidArg;
    }
    return check_matmul_args(ctx, p->parts[0], x, m, x_cols, y);
}

int32_t ferric_cuda_proj_matmul(ferric_cuda_ctx* ctx, const ferric_proj* p, const float* x_dev, size_t m, size_t x_cols, float* y_dev)
{
    int32_t rc = check_proj_args(ctx, p, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    DeviceGuard guard(ctx->device);
    if (p->n_parts == 1) return run_matmul(ctx, p->parts[0], x_dev, m, 0, y_dev, 0, kEpiStore);
    return proj_matmul_ld(ctx, p, x_dev, m, y_dev, p->rows);
}

// Proj::gate_up_swiglu: the fused kernel when gate|up is one fusable matrix, otherwise matmul + cat, then swiglu.
int32_t ferric_cuda_proj_gate_up_swiglu(ferric_cuda_ctx* ctx, const ferric_proj* p, const float* x_dev, size_t m, size_t x_cols,
                                        size_t n_ff, float* y_dev)
{
    int32_t rc = check_proj_args(ctx, p, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    if (p->rows != 2 * n_ff) {
        set_last_error("gate_up_swiglu: the projection has %zu rows, not 2 x n_ff = %zu", p->rows, 2 * n_ff);
        return kErrShape;
    }
    if (m == 0 || n_ff == 0) return kOk;
    DeviceGuard guard(ctx->device);
    if (p->n_parts == 1 && has_prepared_form(p->parts[0]->ty) && p->parts[0]->w.rows % 32 == 0)
        return run_matmul(ctx, p->parts[0], x_dev, m, 0, y_dev, 0, kEpiSwiglu);
    float* gu = nullptr;
    FERRIC_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&gu), m * p->rows * sizeof(float), ctx->stream));
    rc = p->n_parts == 1 ? run_matmul(ctx, p->parts[0], x_dev, m, 0, gu, 0, kEpiStore) : proj_matmul_ld(ctx, p, x_dev, m, gu, p->rows);
    if (rc == kOk) {
        ctx->launches++;
        rc = launch_swiglu(ctx->stream, gu, m, n_ff, y_dev, ctx->tune);
    }
    cudaFreeAsync(gu, ctx->stream);
    return rc;
}

// ---------------------------------------------------------------------------------------------
// Indexed (mixture-of-experts) products, crates/ferric-tensor/src/dtype.rs:1620-1677: the matrix stacks all experts,
// expert-major; the router's [T, 2k] output (weights | indices as f32) picks k experts per token on the device.
// ---------------------------------------------------------------------------------------------
static int32_t check_id_args(const ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const void* x, const void* selw, const void* y,
                             size_t t, size_t k, size_t x_cols, size_t rows_per_expert)
{
    if (!ctx || !qm) {
        set_last_error("NULL context or matrix handle");
        return kErrInvalidArg;
    }
    if (qm->device != ctx->device) {
        set_last_error("matrix lives on device %d, context on device %d", qm->device, ctx->device);
        return kErrInvalidArg;
    }
    if (qm->ty != kGgmlQ4K && qm->ty != kGgmlQ5K && qm->ty != kGgmlQ6K) {
        set_last_error("indexed products take Q4_K / Q5_K / Q6_K expert stacks (ggml type %u given)", qm->ty);
        return kErrUnsupportedType;
    }
    if (k < 1 || k > 8) {
        set_last_error("k must be 1..=8");
        return kErrShape;
    }
    if (x_cols != qm->w.cols) {
        set_last_error("inner dim mismatch: x[..,%zu] vs W[..,%zu]", x_cols, qm->w.cols);
        return kErrShape;
    }
    if (rows_per_expert == 0 || rows_per_expert % 16 != 0 || qm->w.rows % rows_per_expert != 0) {
        set_last_error("the matrix's %zu rows are not a whole number of experts of %zu rows (a multiple of 16)", qm->w.rows,
                       rows_per_expert);
        return kErrShape;
    }
    if (t > 0 && (!x || !selw || !y)) {
        set_last_error("NULL activation, selection or result buffer");
        return kErrInvalidArg;
    }
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 3) || (reinterpret_cast<uintptr_t>(selw) & 3)) {
        set_last_error("activation buffer must be 16-byte aligned (selection and result 4-byte)");
        return kErrInvalidArg;
    }
    return kOk;
}

int32_t ferric_cuda_matmul_q_swiglu_id(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t t, size_t x_cols,
                                       const float* selw_dev, size_t k, size_t eff, float* y_dev)
{
    int32_t rc = check_id_args(ctx, qm, x_dev, selw_dev, y_dev, t, k, x_cols, 2 * eff);
    if (rc != kOk) return rc;
    if (eff % 16 != 0) {
        set_last_error("eff (%zu) must be a multiple of 16", eff);
        return kErrShape;
    }
    if (t == 0 || qm->w.nblk == 0) return kOk;
    DeviceGuard guard(ctx->device);
    if ((rc = ensure_scratch(ctx, frag_bytes(qm->ty, qm->w, t))) != kOk) return rc;
    if ((rc = launch_prep(ctx->stream, qm->ty, qm->w, x_dev, t, qm->w.cols, ctx->scratch, ctx->tune)) != kOk) return rc;
    IdSel id;
    id.selw = selw_dev;
    id.k = (int)k;
    id.rows_per_expert = (int)(2 * eff);
    id.n_expert = (int)(qm->w.rows / (2 * eff));
    id.x_per_pair = 0;
    ctx->launches += 2;
    return launch_gemv_id(ctx->stream, qm->ty, qm->w, ctx->scratch, t, t * k, y_dev, eff, kEpiSwiglu, ctx->tune, id);
}

int32_t ferric_cuda_matmul_q_id_wsum(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t t, size_t k,
                                     size_t x_cols, const float* selw_dev, size_t out_pe, float* y_dev)
{
    int32_t rc = check_id_args(ctx, qm, x_dev, selw_dev, y_dev, t, k, x_cols, out_pe);
    if (rc != kOk) return rc;
    if (t == 0) return kOk;
    DeviceGuard guard(ctx->device);
    if (qm->w.nblk == 0) {
        FERRIC_CUDA_TRY(cudaMemsetAsync(y_dev, 0, t * out_pe * sizeof(float), ctx->stream));
        return kOk;
    }
    const size_t pairs = t * k, frag = (frag_bytes(qm->ty, qm->w, pairs) + 255) / 256 * 256;
    if ((rc = ensure_scratch(ctx, frag + pairs * out_pe * sizeof(float))) != kOk) return rc;
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctx->scratch) + frag);
    if ((rc = launch_prep(ctx->stream, qm->ty, qm->w, x_dev, pairs, qm->w.cols, ctx->scratch, ctx->tune)) != kOk) return rc;
    IdSel id;
    id.selw = selw_dev;
    id.k = (int)k;
    id.rows_per_expert = (int)out_pe;
    id.n_expert = (int)(qm->w.rows / out_pe);
    id.x_per_pair = 1;
    if ((rc = launch_gemv_id(ctx->stream, qm->ty, qm->w, ctx->scratch, pairs, pairs, part, out_pe, kEpiStore, ctx->tune, id)) != kOk) return rc;
    ctx->launches += 3;
    return launch_id_wsum(ctx->stream, part, selw_dev, t, k, out_pe, y_dev, ctx->tune);
}

// ---------------------------------------------------------------------------------------------
// Chained products: a decoder layer's matmuls with the glue between them (activation preparation,
// residual add, RMSNorm statistics) done inside the products' own launches.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace ferric {
int32_t chain_setup(ferric_cuda_ctx* ctx, const ferric_chain_link* link, size_t m, bool pushed, Chain* chain,
                    const void** frag_in, Epilogue* epi, size_t* ldy_out)
{
    if (!ctx || !link || !link->qm) {
        set_last_error("chain_matmul: NULL context, link or matrix");
        return kErrInvalidArg;
    }
    const ferric_qmatrix* qm = link->qm;
    if (qm->device != ctx->device) {
        set_last_error("matrix lives on device %d, context on device %d", qm->device, ctx->device);
        return kErrInvalidArg;
    }
    if (!has_prepared_form(qm->ty)) {
        set_last_error("Q8_0 and dense matrices have no prepared form, so they cannot be chain links");
        return kUnsupported;
    }
    if (link->swiglu && qm->w.rows % 32 != 0) return kUnsupported;
    if (m > kChainMaxRows) {
        set_last_error("a chained product takes at most %zu activation rows (%zu given)", kChainMaxRows, m);
        return kErrShape;
    }
    if (link->in_slot != 0 && link->in_slot != 1) {
        set_last_error("in_slot must be 0 or 1");
        return kErrInvalidArg;
    }
    if (ctx->chain_slot_bytes == 0 || ctx->scratch_bytes < 2 * ctx->chain_slot_bytes) {
        set_last_error("call ferric_cuda_chain_reserve before the first chain link");
        return kErrInvalidArg;
    }
    const size_t out_cols = link->swiglu ? qm->w.rows / 2 : qm->w.rows;
    size_t ldy = link->ldy ? link->ldy : out_cols;
    if (ldy < out_cols || (ldy & 3)) {
        set_last_error("ldy %zu must cover the %zu result columns and be a multiple of 4", ldy, out_cols);
        return kErrShape;
    }
    if (!pushed && m > 0 && out_cols > 0 && (!link->y_dev || (reinterpret_cast<uintptr_t>(link->y_dev) & 15))) {
        set_last_error("chain_matmul: y_dev must be a 16-byte aligned device buffer");
        return kErrInvalidArg;
    }
    if (frag_bytes(qm->ty, qm->w, m) > ctx->chain_slot_bytes || qm->w.nblk > kChainMaxBlocks) {
        set_last_error("chain_matmul: the product's prepared activations (%zu bytes) do not fit the reserved slot (%zu)",
                       frag_bytes(qm->ty, qm->w, m), ctx->chain_slot_bytes);
        return kErrShape;
    }
    *chain = Chain();
    if (link->in_rms) {
        chain->ssq_in = ctx->chain_ssq;
        chain->ssq_blocks = (int)qm->w.nblk;
        chain->eps = link->eps;
        chain->d = (float)qm->w.cols;
    }
    ChainJob& j = chain->job;
    if (link->next != FERRIC_CHAIN_NONE) {
        const ferric_qmatrix* nx = link->next_qm;
        if (link->next != FERRIC_CHAIN_PREPARE && link->next != FERRIC_CHAIN_RESIDUAL) {
            set_last_error("chain_matmul: unknown `next` %d", link->next);
            return kErrInvalidArg;
        }
        if (!nx || nx->device != ctx->device || !has_prepared_form(nx->ty)) {
            set_last_error("chain_matmul: next_qm must be a Q4_K / Q5_K / Q6_K matrix on the context's device");
            return kErrInvalidArg;
        }
        if (nx->w.cols > out_cols || (link->next == FERRIC_CHAIN_RESIDUAL && nx->w.cols != out_cols)) {
            set_last_error("chain_matmul: the next product reads %zu columns, this one yields %zu", nx->w.cols, out_cols);
            return kErrShape;
        }
        if (frag_bytes(nx->ty, nx->w, m) > ctx->chain_slot_bytes || nx->w.nblk > kChainMaxBlocks) {
            set_last_error("chain_matmul: the next product's prepared activations do not fit the reserved slot");
            return kErrShape;
        }
        if (pushed && (link->next != FERRIC_CHAIN_RESIDUAL || link->swiglu)) {
            set_last_error("a pushed chain link must be a plain residual link");
            return kErrInvalidArg;
        }
        if (link->next == FERRIC_CHAIN_RESIDUAL &&
            (!link->h_dev || ((reinterpret_cast<uintptr_t>(link->h_dev) | reinterpret_cast<uintptr_t>(link->norm_weight_dev)) & 15))) {
            set_last_error("chain_matmul: a residual link needs h_dev (16-byte aligned, as norm_weight_dev)");
            return kErrInvalidArg;
        }
        j.kind = link->next == FERRIC_CHAIN_PREPARE ? 1 : pushed ? 3 : 2;
        j.out_ty = nx->ty == kGgmlQ6K ? (int)kGgmlQ6K : (int)kGgmlQ4K;
        j.blocks = (int)nx->w.nblk;
        j.tiles = (int)gemv_padded_tiles(m);
        j.tickets = ctx->chain_tickets;
        j.done = ctx->chain_done;
        j.y = link->y_dev;
        j.ldy = ldy;
        j.frag = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(ctx->scratch) + (size_t)(1 - link->in_slot) * ctx->chain_slot_bytes);
        j.h = link->h_dev;
        j.weight = link->norm_weight_dev;
        j.ssq = ctx->chain_ssq;
    } else if (pushed) {
        set_last_error("a pushed chain link must be a residual link");
        return kErrInvalidArg;
    }
    *frag_in = reinterpret_cast<const uint8_t*>(ctx->scratch) + (size_t)link->in_slot * ctx->chain_slot_bytes;
    *epi = link->swiglu ? kEpiSwiglu : pushed ? kEpiPush : kEpiStore;
    *ldy_out = ldy;
    return kOk;
}
}  // namespace ferric

extern "C" {

int32_t ferric_cuda_chain_reserve(ferric_cuda_ctx* ctx, size_t slot_bytes)
{
    if (!ctx) {
        set_last_error("NULL context");
        return kErrInvalidArg;
    }
    DeviceGuard guard(ctx->device);
    const size_t slot = (slot_bytes + 255) / 256 * 256 + 256;
    int32_t rc = ensure_scratch(ctx, 2 * slot);
    if (rc != kOk) return rc;
    ctx->chain_slot_bytes = slot;
    return kOk;
}

int32_t ferric_cuda_chain_matmul(ferric_cuda_ctx* ctx, const ferric_chain_link* link, size_t m)
{
    Chain chain;
    const void* frag = nullptr;
    Epilogue epi = kEpiStore;
    size_t ldy = 0;
    int32_t rc = chain_setup(ctx, link, m, false, &chain, &frag, &epi, &ldy);
    if (rc != kOk) return rc;
    if (m == 0 || link->qm->w.rows == 0) return kOk;
    if (link->qm->w.nblk == 0) {
        set_last_error("chain_matmul: empty K range");
        return kErrShape;
    }
    DeviceGuard guard(ctx->device);
    ctx->launches++;
    return launch_gemv(ctx->stream, link->qm->ty, link->qm->w, frag, m, link->y_dev, ldy, epi, ctx->tune, PushDst(), &chain);
}

// ---------------------------------------------------------------------------------------------
// matmul_q for callers that must not allocate.
//
// Some hosts hand this library a device whose memory is already fully spoken for -- a serving
// process that carved HBM into KV-cache pages at start-up, a real-time loop in which the implicit
// device synchronisation of cudaMalloc / cudaFree is not acceptable, a sandboxed plugin that is
// not permitted to call the allocator at all.  For them the activation-fragment scratch of the
// Q4_K / Q6_K product lives in a fixed array inside the library image instead of in memory the
// context grows on demand.  Every GPU that loads the library carries the array until the process
// exits.
// ---------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 2u << 20;  // 2 MiB: e.g. 8 activation rows x 32768 columns
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; its device address has to be looked up, per device,
// with that device current.  Done once per device and cached.
int32_t noalloc_scratch_ptr(int device, void** out)
{
    if (device < 0 || device >= kMaxDevices) {
        set_last_error("device %d out of range for the fixed scratch table", device);
        return kErrInvalidArg;
    }
    void* p = __atomic_load_n(&g_noalloc_ptr[device], __ATOMIC_ACQUIRE);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);  // the caller made `device` current
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        __atomic_store_n(&g_noalloc_ptr[device], p, __ATOMIC_RELEASE);
    }
    *out = p;
    return kOk;
}
}  // namespace

int32_t ferric_cuda_matmul_q_noalloc(ferric_cuda_ctx* ctx, const ferric_qmatrix* qm, const float* x_dev, size_t m,
                                     size_t x_cols, float* y_dev)
{
    int32_t rc = check_matmul_args(ctx, qm, x_dev, m, x_cols, y_dev);
    if (rc != kOk) return rc;
    if (m == 0 || qm->w.rows == 0) return kOk;
    DeviceGuard guard(ctx->device);
    if (!has_prepared_form(qm->ty)) {  // these formats need no scratch at all
        ctx->launches++;
        if (qm->ty == kGgmlF32) return launch_gemv_f32(ctx->stream, qm->w, x_dev, m, qm->w.cols, y_dev, qm->w.rows, ctx->tune);
        return launch_gemv_q8_0(ctx->stream, qm->w, x_dev, m, qm->w.cols, y_dev, qm->w.rows, ctx->tune);
    }
    if (qm->w.nblk == 0) {
        FERRIC_CUDA_TRY(cudaMemsetAsync(y_dev, 0, m * qm->w.rows * sizeof(float), ctx->stream));
        return kOk;
    }
    const size_t need = frag_bytes(qm->ty, qm->w, m);
    if (need > kNoAllocScratchBytes) {
        set_last_error("matmul_q_noalloc: %zu activation rows x %zu columns need %zu bytes of scratch, the fixed "
                       "array holds %zu; use ferric_cuda_matmul_q or split the batch", m, x_cols, need,
                       kNoAllocScratchBytes);
        return kErrShape;
    }
    void* scratch = nullptr;
    if ((rc = noalloc_scratch_ptr(ctx->device, &scratch)) != kOk) return rc;
    // The preparation kernel rewrites every fragment the product reads (all padded tiles, every
    // super-block), so nothing left over from an earlier call needs clearing first.
    if ((rc = launch_prep(ctx->stream, qm->ty, qm->w, x_dev, m, qm->w.cols, scratch, ctx->tune)) != kOk) return rc;
    rc = launch_gemv(ctx->stream, qm->ty, qm->w, scratch, m, y_dev, qm->w.rows, kEpiStore, ctx->tune);
    ctx->launches += 2;
    return rc;
}

}  // extern "C"
