/*
 * ferric_cuda.h -- C ABI of libferric_cuda: the sm_100a backend for Ferric's packed-quant
 * (GGUF Q4_K / Q6_K / Q8_0) weight x activation product.
 *
 * Each entry point names the reference interface it stands in for (paths relative to the
 * dcharlot-physicalai-bmi/ferric source tree).  Conventions follow the reference's own C ABI
 * (crates/ferric-ffi/src/lib.rs:99-132, libferric.h): opaque handles, explicit *_free, nothing
 * unwinds or aborts across the boundary.  Where the Rust side returns Result<_, String> or
 * panics on a shape error, these functions return a status code and leave the message in
 * ferric_cuda_last_error() (thread-local).
 *
 * Threading: one context per device per thread of control; calls on a context are ordered by
 * its CUDA stream and are asynchronous like the reference's dispatch queue
 * (crates/ferric-tensor/src/lib.rs:1712-1770) -- results are visible after ferric_cuda_ctx_sync
 * or after the caller synchronises the stream.  A ferric_qmatrix is immutable once built and
 * may be used by any context on the same device.
 *
 * There is no CPU fallback behind any of these functions: without a CUDA device they fail with
 * FERRIC_ERR_CUDA.
 */
#ifndef FERRIC_CUDA_H
#define FERRIC_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ---------------------------------------------------------------------------- */
#define FERRIC_OK 0
#define FERRIC_ERR_INVALID_ARG 1      /* NULL handle / pointer, misaligned activation buffer */
#define FERRIC_ERR_UNSUPPORTED_TYPE 2 /* Err("unsupported ggml type ..") / Err("QMatrix: no native matmul ..") */
#define FERRIC_ERR_SHAPE 3            /* the reference's assert!s: cols % block, byte length, inner dim */
#define FERRIC_ERR_CUDA 4
#define FERRIC_ERR_OOM 5
#define FERRIC_UNSUPPORTED 6          /* try_matmul_swiglu returning None */
#define FERRIC_ERR_TIMEOUT 7          /* a bounded device-side wait ran out */

/* ggml type ids carried by this path (crates/ferric-gguf/src/lib.rs:18-34). */
#define FERRIC_GGML_F32 0u
#define FERRIC_GGML_F16 1u
#define FERRIC_GGML_Q8_0 8u
#define FERRIC_GGML_Q4_K 12u
#define FERRIC_GGML_Q5_K 13u
#define FERRIC_GGML_Q6_K 14u
#define FERRIC_GGML_BF16 30u

typedef struct ferric_cuda_ctx ferric_cuda_ctx;
typedef struct ferric_qmatrix ferric_qmatrix;

/* Message of the last failing call on this thread ("" if none). */
const char *ferric_cuda_last_error(void);

/* ---- ferric-gguf: sizes and decoders ---------------------------------------------------- */

/* type_size(ty, n) -> Result<usize, String>   crates/ferric-gguf/src/lib.rs:471-494
 * (types 0, 1, 8, 12, 14, 30; any other id is FERRIC_ERR_UNSUPPORTED_TYPE). */
int32_t ferric_gguf_type_size(uint32_t ggml_type, size_t n, size_t *out_bytes);

/* deq_raw(raw, n, ty) -> Result<Vec<f32>, String>   crates/ferric-gguf/src/lib.rs:497-520
 * raw and out are HOST buffers; the decode itself runs on the context's device (bit-exact
 * with the reference's CPU decoders).  Types 8, 12, 14. */
int32_t ferric_gguf_deq_raw(ferric_cuda_ctx *ctx, const uint8_t *raw, size_t raw_len, size_t n,
                            uint32_t ggml_type, float *out);

/* ---- ferric-core: the device context ---------------------------------------------------- */

/* Context::new()   crates/ferric-core/src/lib.rs:109-151.  Owns a non-blocking stream. */
int32_t ferric_cuda_ctx_create(int device, ferric_cuda_ctx **out);
/* Same, but launches go to a caller-owned stream (cudaStream_t passed as void*; NULL = the
 * legacy default stream), e.g. the stream of the framework hosting the activations. */
int32_t ferric_cuda_ctx_create_on_stream(int device, void *cuda_stream, ferric_cuda_ctx **out);
/* Redirect later launches to another stream of the same device. */
int32_t ferric_cuda_ctx_set_stream(ferric_cuda_ctx *ctx, void *cuda_stream);
void *ferric_cuda_ctx_stream(const ferric_cuda_ctx *ctx);
/* Block until everything queued on the context's stream is done (the reference's
 * flush + readback point, crates/ferric-tensor/src/lib.rs:1816-1836). */
int32_t ferric_cuda_ctx_sync(ferric_cuda_ctx *ctx);
void ferric_cuda_ctx_free(ferric_cuda_ctx *ctx);

/* Capability record, the counterpart of Context's fields (crates/ferric-core/src/lib.rs:19-43). */
typedef struct ferric_cuda_caps {
    int32_t device;
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    uint64_t l2_bytes;
    uint64_t total_mem_bytes;
    uint64_t max_smem_per_block;
} ferric_cuda_caps;
int32_t ferric_cuda_ctx_caps(const ferric_cuda_ctx *ctx, ferric_cuda_caps *out);

/* Grow the context's activation-fragment scratch to at least `bytes` now, so later calls do not
 * allocate (needed before capturing calls into a CUDA graph).  Growing moves the scratch: a graph
 * captured earlier keeps the old address and must not be replayed after a later call has grown
 * it -- reserve the largest size any captured or later call will need (the maximum of
 * ferric_cuda_qmatrix_scratch_bytes(qm, m) over them) before the first capture. */
int32_t ferric_cuda_ctx_reserve_scratch(ferric_cuda_ctx *ctx, size_t bytes);
/* Launch counters since creation: kernels this library launched on the context. */
uint64_t ferric_cuda_ctx_launches(const ferric_cuda_ctx *ctx);

/* prof(ctx, label) / prof_report()   crates/ferric-tensor/src/lib.rs:3017-3046: per-op timing buckets.  When enabled
 * (the reference's FERRIC_PROFILE), ferric_cuda_prof synchronises the context's stream and charges the time since the
 * previous mark to `label` (the first mark only starts the clock) -- it serialises the stream, so it measures where the
 * work is, not the fastest achievable.  ferric_cuda_prof_report writes the buckets, largest first, as text (at most
 * cap - 1 bytes, full length in *len) and, when the whole text fitted, resets them. */
int32_t ferric_cuda_prof_enable(ferric_cuda_ctx *ctx, int32_t on);
int32_t ferric_cuda_prof(ferric_cuda_ctx *ctx, const char *label);
int32_t ferric_cuda_prof_report(ferric_cuda_ctx *ctx, char *buf, size_t cap, size_t *len);

/* ---- ferric-tensor: QMatrix ------------------------------------------------------------- */

/* QMatrix::block_bytes(ty) -> Option<(values, bytes)>   crates/ferric-tensor/src/dtype.rs:873-889
 * rows 8 / 12 / 14.  FERRIC_UNSUPPORTED stands for None. */
int32_t ferric_cuda_qmatrix_block_bytes(uint32_t ggml_type, size_t *values_per_block, size_t *bytes_per_block);

/* QMatrix::from_bytes(ctx, bytes, ggml_type, rows, cols) -> Result<QMatrix, String>
 * crates/ferric-tensor/src/dtype.rs:893-908 -> QShard::build :839-857 -> Q4_KWeights / Q6_KWeights /
 * Q8_0Weights::from_bytes :1388-1420 / :1147-1166 / :1270-1286.
 * `bytes` (HOST) are raw GGUF block bytes, row-major [rows = out, cols = in]; they are copied and
 * re-packed into the device layout, the pointer is not kept.  Errors: cols not a multiple of the
 * block size or len != rows * cols / block_values * block_bytes -> FERRIC_ERR_SHAPE; a type with
 * no packed kernel -> FERRIC_ERR_UNSUPPORTED_TYPE. */
int32_t ferric_cuda_qmatrix_from_bytes(ferric_cuda_ctx *ctx, const uint8_t *bytes, size_t len, uint32_t ggml_type,
                                       size_t rows, size_t cols, ferric_qmatrix **out);

/* The same constructor restricted to the sub-matrix rows [row0, row0 + nrows) x columns
 * [col0, col0 + ncols) of the full tensor: a tensor-parallel shard (a row range for
 * column-parallel Q/K/V/gate/up, a K range for row-parallel O/down) built straight from the
 * whole tensor's bytes.  col0 and ncols must be block multiples.  Generalises the row sharding
 * of QMatrix::from_bytes (crates/ferric-tensor/src/dtype.rs:899-905). */
int32_t ferric_cuda_qmatrix_from_bytes_view(ferric_cuda_ctx *ctx, const uint8_t *bytes, size_t len,
                                            uint32_t ggml_type, size_t rows, size_t cols, size_t row0, size_t nrows,
                                            size_t col0, size_t ncols, ferric_qmatrix **out);

/* As from_bytes, but `bytes_dev` already live in this device's memory (weights produced or
 * staged on the device); they are read during the call's stream work and not kept. */
int32_t ferric_cuda_qmatrix_from_device_bytes(ferric_cuda_ctx *ctx, const uint8_t *bytes_dev, size_t len,
                                              uint32_t ggml_type, size_t rows, size_t cols, ferric_qmatrix **out);

/* QMatrix::from_dense(ctx, w, rows, cols)   crates/ferric-tensor/src/dtype.rs:912-926 (DenseWeight :817-834): the
 * fallback for GGUF quants with no packed kernel -- the loader dequantises them to f32 and hands the row-major
 * [rows, cols] weight here (HOST pointer, copied).  matmul_q on such a matrix is a plain f32 product; it reports ggml
 * type FERRIC_GGML_F32, nbytes = rows * cols * 4, has no prepared form, no fused SwiGLU and no bf16 product
 * (FERRIC_UNSUPPORTED), as in the reference. */
int32_t ferric_cuda_qmatrix_from_dense(ferric_cuda_ctx *ctx, const float *w_host, size_t rows, size_t cols, ferric_qmatrix **out);

/* QMatrix::rows / cols / nbytes / n_shards   crates/ferric-tensor/src/dtype.rs:927-930.
 * nbytes is the on-disk format size (rows * cols / 256 * 144 for Q4_K, :1421). */
size_t ferric_cuda_qmatrix_rows(const ferric_qmatrix *qm);
size_t ferric_cuda_qmatrix_cols(const ferric_qmatrix *qm);
size_t ferric_cuda_qmatrix_nbytes(const ferric_qmatrix *qm);
size_t ferric_cuda_qmatrix_n_shards(const ferric_qmatrix *qm);
uint32_t ferric_cuda_qmatrix_ggml_type(const ferric_qmatrix *qm);
void ferric_cuda_qmatrix_free(ferric_qmatrix *qm);

/* Bytes of context scratch any product call (matmul_q*, matmul_q_bf16) with m activation rows needs for this matrix. */
size_t ferric_cuda_qmatrix_scratch_bytes(const ferric_qmatrix *qm, size_t m);

/* Tensor::matmul_q(&QMatrix)   crates/ferric-tensor/src/dtype.rs:935-944 -> matmul_q4_k :1426-1473,
 * matmul_q6_k :1172-1194, matmul_q8_0 :1292-1313.
 * y[m, rows] = x[m, cols] . W^T, f32 in, f32 out, both DEVICE buffers, contiguous row-major,
 * 16-byte aligned.  m >= 0.  `x_cols` is the activation's inner dimension; a mismatch with the
 * matrix is the reference's "inner dim mismatch" panic -> FERRIC_ERR_SHAPE.
 * Few activation rows (and Q8_0 at any m) run the GEMV kernels, in passes of 4 rows; Q4_K / Q5_K from 9 rows and Q6_K from 13
 * run a tensor-core kernel on integer-valued f16 operands (FERRIC_CUDA_GEMV_TC_MIN_M in the environment moves
 * that threshold, 0 switches the kernel off); ferric_cuda_gemm_status reports its bounded waits. */
int32_t ferric_cuda_matmul_q(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t m,
                             size_t x_cols, float *y_dev);

/* The same product with explicit row strides (in floats) for x and y, so a column slice of a
 * wider activation tensor feeds the matmul without a copy (the reference makes such inputs
 * contiguous first, crates/ferric-tensor/src/dtype.rs:1427).  ldx must be a multiple of 4;
 * 0 means "contiguous". */
int32_t ferric_cuda_matmul_q_ld(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t m,
                                size_t x_cols, size_t ldx, float *y_dev, size_t ldy);

/* The two halves of matmul_q, for callers that feed one activation tensor to several matrices
 * of the same format and inner dimension (fused q|k|v is one matrix in the reference,
 * crates/ferric-llama/src/qwen35.rs:380-402; split projections are not, qwen3.rs:192-228):
 * prepare_x converts x[m, x_cols] into the context's activation scratch once;
 * matmul_q_prepared multiplies any such matrix with what is in the scratch (swiglu != 0 selects
 * the fused gate/up epilogue, FERRIC_UNSUPPORTED as for matmul_q_swiglu).  Q8_0 has no prepared
 * form (FERRIC_UNSUPPORTED). */
int32_t ferric_cuda_prepare_x(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t m,
                              size_t x_cols, size_t ldx);
int32_t ferric_cuda_matmul_q_prepared(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, size_t m, float *y_dev,
                                      size_t ldy, int32_t swiglu);

/* Tensor::add_rmsnorm(other, weight, eps) -> (sum, norm)   crates/ferric-tensor/src/lib.rs:372-384
 * (kernel :2057-2075), and Tensor::rmsnorm :346-353 when b_dev is NULL.  sum = a + b,
 * norm = sum / sqrt(mean(sum^2) + eps) * weight; weight_dev NULL means all ones
 * (rmsnorm_weightless, :340-344); sum_dev may be NULL or alias a_dev. */
int32_t ferric_cuda_add_rmsnorm(ferric_cuda_ctx *ctx, const float *a_dev, const float *b_dev, const float *weight_dev,
                                float eps, size_t rows, size_t d, float *sum_dev, float *norm_dev);

/* add_rmsnorm fused with prepare_x: norm = rmsnorm(a + b) * weight (row length = the matrix's
 * inner dimension) is converted straight into the context's activation scratch, ready for
 * matmul_q_prepared on `qm` or any matrix of the same format and inner dimension -- the
 * `x.add_rmsnorm(..)` -> `matmul_q` pair of a decoder layer (crates/ferric-llama/src/qwen35.rs:986-996)
 * in one launch.  b_dev, weight_dev, sum_dev (may alias a_dev) and norm_dev may each be NULL.
 * The prepared form is the GEMV's: matmul_q_prepared runs the GEMV kernels in passes of 4 rows whatever m is, so from the
 * tensor-core kernel's threshold on (9 rows, Q6_K 13) the pair ferric_cuda_add_rmsnorm + ferric_cuda_matmul_q is faster. */
int32_t ferric_cuda_add_rmsnorm_prepare(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *a_dev,
                                        const float *b_dev, const float *weight_dev, float eps, size_t m,
                                        float *sum_dev, float *norm_dev);

/* ---- chained decoder-layer products ----------------------------------------------------------- */
/* The reference batches a decoder layer's kernels -- norm, projections, residual adds -- into one submit
 * (crates/ferric-llama/src/qwen35.rs:985-996, the layer loop :953-1014).  Here the glue between the products moves into
 * the products' own launches, so a layer is one launch per matrix and nothing else:
 *   - a link may PREPARE: once a 256-wide block of its result is complete, the warp that stored the block's last tile
 *     converts it into the activation form of the next product (what ferric_cuda_prepare_x would do in a launch of
 *     its own) -- e.g. q|k|v -> o, gate|up+SwiGLU -> down;
 *   - or be a RESIDUAL link: the block is added to the residual stream h in place (Tensor::add_rmsnorm's sum,
 *     crates/ferric-tensor/src/lib.rs:372-384), its sum of squares recorded, and h * norm_weight prepared for the next
 *     product WITHOUT the 1/rms factor -- that scalar commutes with the product, so the next link (in_rms = 1) applies
 *     1 / sqrt(mean(h^2) + eps) to its result instead -- e.g. o -> gate|up, down -> the next layer's q|k|v.
 * The context's scratch holds two prepared-activation slots; a link reads slot `in_slot` and prepares into the other.
 * ferric_cuda_add_rmsnorm_prepare / ferric_cuda_prepare_x write slot 0 (already normalised: in_rms = 0 for their
 * consumer), which is how a chain starts.  Up to 4 activation rows (one pass of the GEMV); Q4_K / Q5_K / Q6_K. */
#define FERRIC_CHAIN_NONE 0
#define FERRIC_CHAIN_PREPARE 1
#define FERRIC_CHAIN_RESIDUAL 2
typedef struct ferric_chain_link {
    const ferric_qmatrix *qm;     /* this product's matrix */
    int32_t swiglu;               /* 1: [gate | up] matrix, result silu(gate . x) * (up . x) (try_matmul_swiglu) */
    int32_t in_slot;              /* slot holding the prepared input: 0 or 1 */
    int32_t in_rms;               /* 1: input prepared by a RESIDUAL link; scale the result by 1 / sqrt(mean(h^2) + eps) */
    float eps;                    /* RMSNorm epsilon (with in_rms) */
    float *y_dev;                 /* result [m, rows] (rows / 2 with swiglu), 16-byte aligned */
    size_t ldy;                   /* its row stride in floats, 0 = contiguous */
    int32_t next;                 /* FERRIC_CHAIN_NONE / _PREPARE / _RESIDUAL */
    const ferric_qmatrix *next_qm; /* the consumer of what this link prepares: its format and inner dimension; PREPARE
                                     feeds it the first `cols(next_qm)` result columns, RESIDUAL needs cols == rows here */
    float *h_dev;                 /* RESIDUAL: residual stream [m, rows], contiguous, updated in place */
    const float *norm_weight_dev; /* RESIDUAL: RMSNorm weight [rows] or NULL (weightless) */
} ferric_chain_link;
/* Size both slots for prepared activations of up to `slot_bytes` (the largest
 * ferric_cuda_qmatrix_scratch_bytes(qm, m) of any matrix in the chain).  Call before the first link and before any
 * capture; other calls that grow the scratch afterwards invalidate it as they do a captured graph. */
int32_t ferric_cuda_chain_reserve(ferric_cuda_ctx *ctx, size_t slot_bytes);
/* One link: y = x . W^T from slot in_slot (+ epilogue), then the link's job.  Asynchronous on the context's stream;
 * links on one context must be issued one after the other (they share the block tickets). */
int32_t ferric_cuda_chain_matmul(ferric_cuda_ctx *ctx, const ferric_chain_link *link, size_t m);

/* No counterpart in the reference.  matmul_q for hosts that cannot let this library allocate: a
 * server that has already divided the device's memory among its own pools, a latency-critical
 * loop that cannot take the device-wide stall of cudaMalloc / cudaFree, a restricted plugin host.
 * The Q4_K / Q6_K activation scratch is a fixed 2 MiB array inside the library (held by every GPU
 * that loads it, until exit) rather than context memory grown on demand; the call makes no
 * cudaMalloc, cudaFree or other allocating call.  Same arguments and result as
 * ferric_cuda_matmul_q.  Limits and rules:
 *  - the product must need no more than 2 MiB of scratch (ferric_cuda_qmatrix_scratch_bytes(qm, m);
 *    e.g. m <= 8 at 32768 columns, m <= 2 at 131072) -- larger requests fail with FERRIC_ERR_SHAPE
 *    and a message, nothing is launched;
 *  - the first call on each device looks up the array's device address; make that first call
 *    outside any stream capture;
 *  - all contexts and threads share the one array per device: two such calls that overlap on the
 *    GPU (different streams) race on it, so order them.  Nothing needs clearing between calls --
 *    each call overwrites every byte it later reads. */
int32_t ferric_cuda_matmul_q_noalloc(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t m,
                                     size_t x_cols, float *y_dev);

/* Prefill product on the tensor cores: y[m, rows] (f32) = x . W^T with bf16 activations x[m, cols]
 * (raw bf16 bits, 16-byte aligned) and the weights dequantised to bf16, round to nearest even.
 * Replaces the reference's cooperative-matrix prefill kernels Tensor::matmul_q4_k_coop
 * (crates/ferric-tensor/src/dtype.rs:1818-1834, WGSL :2059-2096), matmul_q6_k_coop (:1199-1214) and
 * matmul_q8_0_coop (:1316-1330), which dequantise weight tiles
 * into workgroup memory and multiply them with 8x8x8 subgroup-matrix ops; here a CTA (above
 * 256 activation rows: a pair of CTAs) owns 128 (256) weight rows x up to 512 activation rows,
 * K advances in chunks of 64, and the multiply is tcgen05.mma with the f32 accumulator in tensor
 * memory.  Q4_K, Q5_K, Q6_K and Q8_0 (the last with columns in multiples of 256; anything else returns
 * FERRIC_UNSUPPORTED, the reference's fall-back to the plain kernel); any m >= 1 works but the kernel is
 * meant for m >= 128.  Asynchronous on the context's stream.  Tiles of a partly filled last wave
 * are cut along K; their pieces meet in the context's scratch (up to 37 MB, grown on demand --
 * ferric_cuda_ctx_reserve_scratch beforehand when capturing).  FERRIC_CUDA_GEMM_PAIR=0 in the
 * environment keeps every tile on a single CTA, FERRIC_CUDA_GEMM_SPLIT=0 never cuts a tile. */
int32_t ferric_cuda_matmul_q_bf16(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const uint16_t *x_bf16_dev, size_t m,
                                  size_t x_cols, float *y_dev);

/* Every wait inside the tensor-core kernel is bounded.  This call synchronises the stream and
 * reports (and clears) the code a block left if one of its waits ran out: *code 0 and FERRIC_OK
 * when none did, FERRIC_ERR_TIMEOUT otherwise.  No counterpart in the reference. */
int32_t ferric_cuda_gemm_status(ferric_cuda_ctx *ctx, int32_t *code);

/* The same product with HOST activation and result buffers: copies x in, runs, copies y out and
 * returns when y is complete. */
int32_t ferric_cuda_matmul_q_host(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_host, size_t m,
                                  size_t x_cols, float *y_host);

/* Tensor::try_matmul_swiglu(&QMatrix) -> Option<Tensor>   crates/ferric-tensor/src/dtype.rs:949-959
 * (-> matmul_q4_k_swiglu :1551-1574, matmul_q6_k_swiglu :1802-1817).  The matrix is [gate rows |
 * up rows] = [2*n_ff, cols]; y[m, n_ff] = silu(gate . x) * (up . x).  FERRIC_UNSUPPORTED (the
 * reference's None) for Q8_0 or when n_ff is not a multiple of 16; the caller then runs
 * matmul_q followed by ferric_cuda_swiglu, as Proj::gate_up_swiglu does
 * (crates/ferric-llama/src/qwen3.rs:219-227). */
int32_t ferric_cuda_matmul_q_swiglu(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t m,
                                    size_t x_cols, float *y_dev);

/* Tensor::matmul_q4_k_swiglu_id   crates/ferric-tensor/src/dtype.rs:1620-1637 (kernel :2463-2516), for Q4_K, Q5_K and
 * Q6_K stacks: batched selected-expert gate|up + SwiGLU of a mixture-of-experts layer.  The matrix packs ALL experts'
 * fused gate|up weights, expert-major: rows = n_expert * 2 * eff (expert e: eff gate rows, then eff up rows).
 * x[t, cols]: one hidden row per token; selw[t, 2k] is the router's output (Tensor::moe_topk, :1582-1612): the k
 * weights, then the k expert indices stored as f32.  y[t, k, eff] = silu(gate_e . x_t) * (up_e . x_t) for every
 * (token, selected expert).  k in 1..8 (the reference's assert), eff a multiple of 16; an index outside the stack
 * yields zeros.  All buffers on the device. */
int32_t ferric_cuda_matmul_q_swiglu_id(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t t,
                                       size_t x_cols, const float *selw_dev, size_t k, size_t eff, float *y_dev);
/* Tensor::matmul_q6_k_id_wsum   crates/ferric-tensor/src/dtype.rs:1660-1677 (kernel :2538-2566; its Q4_K twin
 * :2569-...): the selected experts' down projections with the weighted sum fused.  The matrix packs all experts' down
 * weights, expert-major (rows = n_expert * out_pe); x[t, k, cols] holds row (t, s) = token t's slot-s SwiGLU output;
 * y[t, out_pe] = sum over s, in slot order, of w_{t,s} * (down_{e_{t,s}} . x_{t,s}).  out_pe a multiple of 16. */
int32_t ferric_cuda_matmul_q_id_wsum(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, const float *x_dev, size_t t, size_t k,
                                     size_t x_cols, const float *selw_dev, size_t out_pe, float *y_dev);

/* Tensor::swiglu(d)   crates/ferric-tensor/src/lib.rs:726-737: gu[t, 2d] -> out[t, d]. */
int32_t ferric_cuda_swiglu(ferric_cuda_ctx *ctx, const float *gu_dev, size_t t, size_t d, float *out_dev);

/* Device-side deq_raw of a loaded matrix: out[rows * cols] f32, bit-exact with
 * crates/ferric-gguf/src/lib.rs:497-520 applied to the bytes the matrix was built from. */
int32_t ferric_cuda_dequant_f32(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, float *out_dev);
/* The same values rounded to bf16 with the reference's rule
 * (crates/ferric-tensor/src/dtype.rs:4159-4163): out[rows * cols] uint16 bf16 bits. */
int32_t ferric_cuda_dequant_bf16(ferric_cuda_ctx *ctx, const ferric_qmatrix *qm, uint16_t *out_dev);

/* ---- GGUF ingest --------------------------------------------------------------------------- */
/* ferric_gguf::parse   crates/ferric-gguf/src/lib.rs:105-132 (bounds-safe cursor :59-103, stride guard
 * :387-431): header, metadata and tensor table of a GGUF file held in memory.  `bytes` is borrowed:
 * it must stay valid for the life of the handle.  Errors as the reference reports them: "not a GGUF
 * file" (FERRIC_ERR_INVALID_ARG), "GGUF header truncated or malformed" and the two stride refusals
 * (FERRIC_ERR_SHAPE). */
typedef struct ferric_gguf ferric_gguf;
int32_t ferric_gguf_parse(const uint8_t *bytes, size_t len, ferric_gguf **out);
/* GgufFile::open   :533-554.  The file is memory-mapped read-only; tensor bytes are served from the
 * mapping without a copy. */
int32_t ferric_gguf_open(const char *path, ferric_gguf **out);
void ferric_gguf_free(ferric_gguf *g);
size_t ferric_gguf_n_tensors(const ferric_gguf *g);
size_t ferric_gguf_data_start(const ferric_gguf *g); /* GgufFile::data_start :562 */
size_t ferric_gguf_n_meta(const ferric_gguf *g);

/* TensorInfo :40-45, plus the element count and the byte size by this library's type table
 * (0 for a type it does not know).  `name` points into the handle. */
typedef struct {
    const char *name;
    uint32_t n_dims;
    uint64_t dims[4]; /* fastest-varying first: a listed [in, out] is a row-major [out, in] weight */
    uint32_t ggml_type;
    uint64_t offset; /* relative to ferric_gguf_data_start */
    uint64_t n_elements;
    uint64_t nbytes;
} ferric_gguf_tensor;
int32_t ferric_gguf_tensor_at(const ferric_gguf *g, size_t index, ferric_gguf_tensor *out);
int32_t ferric_gguf_tensor_by_name(const ferric_gguf *g, const char *name, ferric_gguf_tensor *out); /* Gguf::tensor :444 */
/* Gguf::raw / GgufFile::raw   :447-453, :566-573: the tensor's packed bytes exactly as stored --
 * a pointer into the file, valid until ferric_gguf_free. */
int32_t ferric_gguf_raw(const ferric_gguf *g, const char *name, const uint8_t **data, size_t *nbytes);

/* Metadata (enum Meta :37).  A getter of the wrong kind fails with FERRIC_ERR_INVALID_ARG.
 * String getters copy at most cap - 1 bytes, terminate, and report the full length in *len. */
enum { FERRIC_GGUF_META_U = 0, FERRIC_GGUF_META_I = 1, FERRIC_GGUF_META_F = 2, FERRIC_GGUF_META_BOOL = 3,
       FERRIC_GGUF_META_STR = 4, FERRIC_GGUF_META_ARR = 5 };
int32_t ferric_gguf_meta_key_at(const ferric_gguf *g, size_t index, char *buf, size_t cap, size_t *len);
int32_t ferric_gguf_meta_kind(const ferric_gguf *g, const char *key, int32_t *kind);
int32_t ferric_gguf_meta_u64(const ferric_gguf *g, const char *key, uint64_t *out);
int32_t ferric_gguf_meta_i64(const ferric_gguf *g, const char *key, int64_t *out);
int32_t ferric_gguf_meta_f64(const ferric_gguf *g, const char *key, double *out);
int32_t ferric_gguf_meta_bool(const ferric_gguf *g, const char *key, int32_t *out);
int32_t ferric_gguf_meta_str(const ferric_gguf *g, const char *key, char *buf, size_t cap, size_t *len);
int32_t ferric_gguf_meta_arr_len(const ferric_gguf *g, const char *key, size_t *n);
int32_t ferric_gguf_meta_arr_str(const ferric_gguf *g, const char *key, size_t index, char *buf, size_t cap, size_t *len);
int32_t ferric_gguf_meta_arr_f64(const ferric_gguf *g, const char *key, size_t index, double *out);

/* The model loaders' qm / qm_cat   crates/ferric-llama/src/qwen35.rs:366-402: one device matrix from
 * one named weight, or from several same-format weights of equal input width stacked along the
 * output dimension (q|k|v, gate|up) -- rows = sum of dims[1], cols = dims[0].  Mixed formats, a
 * differing input width or a missing tensor fail as in the reference; a format without a packed
 * kernel here fails with FERRIC_ERR_UNSUPPORTED_TYPE (the reference dequantises to a dense matrix
 * instead, which this library does not do). */
int32_t ferric_cuda_qmatrix_from_gguf(ferric_cuda_ctx *ctx, const ferric_gguf *g, const char *const *names, size_t n_names,
                                      ferric_qmatrix **out);

/* Proj   crates/ferric-llama/src/qwen3.rs:192-228: a projection that is logically one matmul with several stacked
 * outputs (q|k|v, gate|up).  Proj::load (:199-208): when every named weight has the same quant format the bytes are
 * stacked into ONE matrix (Fused: qm_cat, or qm for a single name); real Q4_K_M files mix formats inside q|k|v (V in
 * Q6_K beside Q4_K Q and K, :188-191), and then each weight becomes a matrix of its own (Split).  Up to 8 names. */
typedef struct ferric_proj ferric_proj;
int32_t ferric_cuda_proj_from_gguf(ferric_cuda_ctx *ctx, const ferric_gguf *g, const char *const *names, size_t n_names,
                                   ferric_proj **out);
/* The same from matrices the caller built (a Split projection of `n_parts` parts, or Fused with one); the projection
 * takes ownership of them and frees them with ferric_cuda_proj_free.  All parts: same device, same input dim. */
int32_t ferric_cuda_proj_from_parts(ferric_qmatrix *const *parts, size_t n_parts, ferric_proj **out);
size_t ferric_cuda_proj_n_parts(const ferric_proj *p); /* 1 = Proj::Fused */
size_t ferric_cuda_proj_rows(const ferric_proj *p);    /* sum of the parts' rows */
size_t ferric_cuda_proj_cols(const ferric_proj *p);
const ferric_qmatrix *ferric_cuda_proj_part(const ferric_proj *p, size_t i);
void ferric_cuda_proj_free(ferric_proj *p);
/* Proj::matmul (:209-218): y[m, rows] = x . W^T, one product per part written at the part's column offset (the
 * reference concatenates the parts' results); parts with the same activation form share one preparation of x. */
int32_t ferric_cuda_proj_matmul(ferric_cuda_ctx *ctx, const ferric_proj *p, const float *x_dev, size_t m, size_t x_cols,
                                float *y_dev);
/* Proj::gate_up_swiglu (:221-228): y[m, n_ff] = silu(gate . x) * (up . x); one fused kernel when gate|up is a single
 * Q4_K / Q5_K / Q6_K matrix (try_matmul_swiglu), otherwise the plain products followed by Tensor::swiglu. */
int32_t ferric_cuda_proj_gate_up_swiglu(ferric_cuda_ctx *ctx, const ferric_proj *p, const float *x_dev, size_t m,
                                        size_t x_cols, size_t n_ff, float *y_dev);

/* ---- tensor-parallel exchange (one process per GPU) ------------------------------------- */
/* The reference shards a QMatrix by rows and concatenates (crates/ferric-tensor/src/dtype.rs:893-908,
 * :935-944) and moves activations between devices through host buffers
 * (crates/ferric-tensor/src/sched.rs:209-265); it has no reduction across devices.  Sharding the
 * o / down projections along K needs one: the f32 [m, hidden] partial sums of all ranks are added.
 * These entry points do that with the library's own kernels over CUDA-IPC peer memory. */
typedef struct ferric_tp_group ferric_tp_group;

/* Allocate this rank's two exchange buffers of `elems` floats (kind 0 and 1) plus flags. */
int32_t ferric_cuda_tp_create(ferric_cuda_ctx *ctx, int32_t rank, int32_t world, size_t elems, ferric_tp_group **out);
/* 64-byte CUDA IPC handle of this rank's exchange memory, to be sent to every peer by the host. */
int32_t ferric_cuda_tp_export(ferric_tp_group *g, uint8_t *handle64);
/* Map the peers' exchange memory: `handles` holds world x 64 bytes in rank order. */
int32_t ferric_cuda_tp_connect(ferric_tp_group *g, const uint8_t *handles);
/* The same for ranks that live in this process (one thread or one loop driving several GPUs): `groups` holds the
 * `world` groups in rank order, this one included; peer access between their devices is switched on as needed. */
int32_t ferric_cuda_tp_connect_local(ferric_tp_group *g, ferric_tp_group *const *groups);
/* Device address of this rank's exchange buffer `kind`: pass it as y_dev of the row-parallel matmul. */
void *ferric_cuda_tp_partial(ferric_tp_group *g, int32_t kind);
/* Announce to all peers that exchange buffer `kind` holds this rank's next partial (stream-ordered).  Each kind has
 * one buffer, which is safe only while consecutive exchanges of this signalled form alternate between the kinds (a
 * decoder layer's o / down pattern): signalling the same kind twice in a row is refused with FERRIC_ERR_INVALID_ARG. */
int32_t ferric_cuda_tp_signal(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind);
/* ferric_cuda_add_rmsnorm_prepare with b = the sum over all ranks of exchange buffer `kind`
 * (waits, bounded, for every rank's announcement; sums in rank order, identically on every rank). */
int32_t ferric_cuda_tp_add_rmsnorm_prepare(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind,
                                           const ferric_qmatrix *qm, const float *a_dev, const float *weight_dev,
                                           float eps, size_t m, float *sum_dev, float *norm_dev);
/* The same exchange, pushed (the lower-latency form for a few activation rows): the row-parallel product
 * x_dev[m, cols] . W^T is not written to a buffer of this rank; its epilogue stores every value, paired with the
 * exchange's sequence number, into the receive region of every rank (this one included).  Q4_K / Q5_K / Q6_K;
 * m x rows must fit the group's `elems`. */
int32_t ferric_cuda_tp_matmul_push(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind, const ferric_qmatrix *qm,
                                   const float *x_dev, size_t m, size_t ldx);
/* ferric_cuda_add_rmsnorm_prepare with b = the sum over all ranks of what they pushed for exchange `kind`: polls
 * (bounded) the pairs in this rank's own memory, sums in rank order, then closes the exchange.  Every
 * tp_matmul_push of a kind must be followed by exactly one of these before the next push of that kind. */
int32_t ferric_cuda_tp_add_rmsnorm_prepare_pushed(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind,
                                                  const ferric_qmatrix *qm, const float *a_dev,
                                                  const float *weight_dev, float eps, size_t m, float *sum_dev,
                                                  float *norm_dev);
/* For many activation rows (the batched decode path): (sum, norm) = add_rmsnorm(a, all-reduce over the ranks of
 * partial_dev[rows, d]) by the library's own kernels in two pushed steps -- every rank stores slice s of its partial into
 * rank s's memory, rank s adds the copies in rank order and stores the sums into every rank's memory, and the add +
 * RMSNorm reads them there.  rows x d must fit the group's `elems`; d a multiple of 4; buffers 16-byte aligned;
 * sum_dev is required (it may be a_dev), norm_dev and weight_dev may be NULL. */
int32_t ferric_cuda_tp_allreduce_add_rmsnorm(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind,
                                             const float *partial_dev, const float *a_dev, const float *weight_dev,
                                             float eps, size_t rows, size_t d, float *sum_dev, float *norm_dev);
/* The same exchange one step at a time (`steps`: 1 scatter, 2 reduce, 4 consume, or-ed together), for a host that
 * drives several ranks on one GPU and therefore must not queue a step that waits for a kernel it has not launched. */
int32_t ferric_cuda_tp_allreduce_add_rmsnorm_steps(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind,
                                                   const float *partial_dev, const float *a_dev,
                                                   const float *weight_dev, float eps, size_t rows, size_t d,
                                                   float *sum_dev, float *norm_dev, int32_t steps);
/* The row-parallel product of this rank, x[m, cols] . W^T, whose result goes straight into the scatter step of that
 * exchange: where the product's K range is cut across CTAs (the tensor-core decode kernel on a matrix with few row
 * tiles -- the o and down shards of a decoder layer), the kernel that adds the K pieces stores the sums, as the exchange's
 * (value, number) pairs, into the slice owners' memory instead of a local buffer (*fused = 1); otherwise the product
 * lands in the group's partial buffer and the scatter step runs after it (*fused = 0).  Either way step 1 is done:
 * continue with ferric_cuda_tp_allreduce_add_rmsnorm_steps(.., steps = 2 | 4) (its partial_dev is not read then).
 * No counterpart in the reference (its model parallelism only concatenates, crates/ferric-tensor/src/sched.rs:209-240).
 * m x rows must fit the group's `elems`, rows a multiple of 4, x 16-byte aligned; ldx = 0 means dense rows. */
int32_t ferric_cuda_tp_matmul_scatter(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind, const ferric_qmatrix *qm,
                                      const float *x_dev, size_t m, size_t ldx, int32_t *fused);
/* A RESIDUAL chain link (ferric_cuda_chain_matmul) whose product is row-parallel: the epilogue pushes the partial
 * sums to every rank as ferric_cuda_tp_matmul_push does, and the link's job polls (bounded) all ranks' pairs for its
 * block in this rank's memory, adds them in rank order to h and prepares the next product -- product, all-reduce,
 * residual add and preparation in one launch.  link->y_dev is not used.  The last job closes the exchange. */
int32_t ferric_cuda_tp_chain_matmul(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t kind, const ferric_chain_link *link,
                                    size_t m);
/* Synchronise the context and report whether any wait on a peer ran out (FERRIC_ERR_TIMEOUT).  Every wait is bounded
 * (about a second by default; FERRIC_CUDA_PEER_WAIT_SPINS in the environment, read when the context is created, sets
 * the number of polling rounds); once one ran out, later kernels of the group do not wait again. */
int32_t ferric_cuda_tp_status(ferric_cuda_ctx *ctx, ferric_tp_group *g, int32_t *timed_out);
/* After a time-out: synchronise, then clear the status word, the exchange counters and every receive region of this
 * rank, so that the ranks count exchanges from zero again.  Every rank of the group must do this, with no exchange in
 * flight, before the next one. */
int32_t ferric_cuda_tp_reset(ferric_cuda_ctx *ctx, ferric_tp_group *g);
void ferric_cuda_tp_free(ferric_tp_group *g);

#ifdef __cplusplus
}
#endif
#endif /* FERRIC_CUDA_H */
