// Internal launch interface between the C ABI (ffi.cu) and the kernel translation units.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace ferric {

constexpr uint32_t kGgmlF32 = 0, kGgmlQ8_0 = 8, kGgmlQ4K = 12, kGgmlQ5K = 13, kGgmlQ6K = 14;
// The formats whose product runs from prepared activation fragments (the tensor-core GEMV kernels).
inline bool has_prepared_form(uint32_t ty) { return ty == kGgmlQ4K || ty == kGgmlQ5K || ty == kGgmlQ6K; }

// One packed weight matrix in device memory.  rows x cols logical; nblk = blocks per row
// (256-weight super-blocks for Q4_K/Q6_K, 32-weight blocks for Q8_0).
struct DeviceWeights {
    uint8_t* units = nullptr;    // Q4_K / Q6_K: ceil(rows/16) * nblk units, zero padded past `rows`
    int8_t* q8_qs = nullptr;     // Q8_0: [rows][cols] int8
    uint16_t* q8_d = nullptr;    // Q8_0: [rows][cols/32] f16 bits
    float* dense = nullptr;      // dense f32 (QMatrix::from_dense): [rows][cols] row-major
    size_t rows = 0, cols = 0, nblk = 0;
    size_t row_tiles() const { return (rows + 15) / 16; }
};

// Tensor-parallel exchange seen from one rank: the f32 partial sums of every rank (its own
// included) in peer-mapped memory, the arrival flags peers write into this rank's memory, this
// rank's own count of exchanges so far, and a status word for waits that give up.
constexpr int kMaxRanks = 8;
struct PeerSum {
    const float* part[kMaxRanks] = {};
    const unsigned* flags = nullptr;   // [world], local memory, written by peers
    const unsigned* epoch = nullptr;   // local: how many exchanges of this kind this rank has signalled
    int* status = nullptr;             // set to 1 if a wait ran out
    int world = 0;                     // 0 = no exchange
    int wait_spins = 4000000;          // polls of a peer's flag before the wait gives up (about a second)
};

// The same exchange done by pushing: the row-parallel product's epilogue stores every output value, paired with the
// exchange's sequence number, straight into each rank's receive region; the consumer polls the pairs in its own memory.
// An 8-byte store arrives whole, so a pair whose number matches carries its value: no flag, no fence, no signal kernel,
// and only a one-way trip over NVLink on the critical path.  Receive regions are double-buffered on the number's parity.
struct PushDst {                      // producer side (kernel parameter)
    uint2* dst[kMaxRanks] = {};       // rank r's receive region for (kind, source = this rank), parity 0
    const unsigned* epoch = nullptr;  // exchanges of this kind completed on this rank; the stamp is *epoch + 1
    size_t parity_stride = 0;         // pairs between the two parities of a region
    int world = 0;
};
struct PushSrc {                      // consumer side
    const uint2* recv = nullptr;      // local memory: [parity][world][elems] pairs for this kind
    unsigned* epoch = nullptr;        // bumped by the last CTA of the consumer
    unsigned* ticket = nullptr;       // CTA counter for that
    int* status = nullptr;            // set to 1 if a wait ran out
    size_t elems = 0;
    int world = 0;                    // 0 = not a push exchange
    int wait_spins = 1000000;         // polling rounds (each a trip to L2 for every rank's pairs) before a wait gives up
};

// The two-step pushed all-reduce of a whole activation matrix (kernels_tpwide.cu), seen from one rank.
struct WideDst {
    uint2* stage1[kMaxRanks] = {};    // rank r's stage-1 region for (kind, source = this rank), parity 0
    uint2* stage2[kMaxRanks] = {};    // rank r's stage-2 region for this kind, parity 0
    const uint2* recv1 = nullptr;     // local stage 1 for this kind: [parity][source rank][slice]
    const uint2* recv2 = nullptr;     // local stage 2 for this kind: [parity][elems]
    unsigned* epoch = nullptr;        // exchanges of this kind completed on this rank
    unsigned* ticket = nullptr;
    int* status = nullptr;
    size_t slice = 0;                 // floats per rank's slice, a multiple of 4
    size_t parity_stride1 = 0, parity_stride2 = 0;   // pairs
    int world = 0, rank = 0;
    int wait_spins = 1000000;         // polling rounds (about a second) before a wait gives up
};
// (sum, norm) = add_rmsnorm(a, all-reduce(partial)) over the ranks of `dst`; rows x d floats, d a multiple of 4.
// `steps`: 1 scatter, 2 reduce, 4 consume (7 = the whole exchange).
int32_t launch_wide_allreduce_add_rmsnorm(cudaStream_t st, const float* partial, const float* a, const float* weight, float eps,
                                          size_t rows, size_t d, float* sum, float* norm, const WideDst& dst,
                                          const struct GemvTuning& tune, int steps = 7);

enum Epilogue : int { kEpiStore = 0, kEpiSwiglu = 1, kEpiPush = 2 };

// A link of a decoder layer's chain of products: what one GEMV launch does besides the product itself, so that the
// layer needs no launches between its products.
//  * Input side: the activations may have been prepared un-normalised (h * weight) by the preceding link's residual
//    job; the product is then scaled by 1 / sqrt(mean(h^2) + eps), with the squares summed per 256-wide block by that
//    job -- the scalar commutes with the product, so nothing has to wait for the whole row before it is converted.
//  * Output side, the "job": every warp that stores a 16-row tile of the result takes a ticket of the tile's 256-wide
//    block; the warp that takes the sixteenth turns the block into the next product's activation fragments, optionally
//    adding it to the residual stream first (kinds 2, 3).  Kind 3 reads the block from the pairs all ranks pushed.
struct ChainJob {
    int kind = 0;                   // 0 none, 1 prepare y, 2 h += y and prepare h * weight, 3 as 2 with y = sum over ranks of the pushed pairs
    int out_ty = 0;                 // fragment format of the next product: kGgmlQ4K (also Q5_K) or kGgmlQ6K
    int blocks = 0;                 // 256-wide blocks of the result that feed the next product (= its super-blocks per row)
    int tiles = 0;                  // activation tiles of two rows (padded as the GEMV pads them)
    unsigned* tickets = nullptr;    // [blocks], zero between launches
    unsigned* done = nullptr;       // kind 3: jobs finished; the last one closes the exchange
    const float* y = nullptr;       // kinds 1, 2: the product's own result, row stride ldy
    size_t ldy = 0;
    uint2* frag = nullptr;          // the next product's fragments
    float* h = nullptr;             // kinds 2, 3: residual stream [m, 256 * blocks], updated in place
    const float* weight = nullptr;  // RMSNorm weight or null
    float* ssq = nullptr;           // kinds 2, 3: [activation row][blocks] sums of squares of the updated residual
    PushSrc pushed;                 // kind 3
};
// Indexed (mixture-of-experts) products: the matrix stacks every expert's rows, expert-major, and each launch "pass"
// (blockIdx.y) is one (token, expert slot) pair whose expert index is read on the device from the router's output
// selw[token][w_0..w_{k-1} | idx_0..idx_{k-1}] (indices stored as f32).
struct IdSel {
    const float* selw = nullptr;   // null: not an indexed product
    int k = 0;                     // expert slots per token
    int n_expert = 0;              // an index outside [0, n_expert) yields zeros
    int rows_per_expert = 0;       // matrix rows per expert (2 * eff for gate|up)
    int x_per_pair = 0;            // 1: activation row = pair number (x is [T, k, in]); 0: activation row = token
};
struct Chain {
    IdSel id;
    const float* ssq_in = nullptr;  // [activation row][ssq_blocks], or null: no scaling
    int ssq_blocks = 0;
    float eps = 0.0f, d = 1.0f;     // row length of the normalised vector, as a float
    ChainJob job;
};
constexpr size_t kChainMaxBlocks = 1024;   // super-blocks per row a chained product may have on either side
constexpr size_t kChainMaxRows = 4;        // activation rows of a chained product (one GEMV pass of two tiles)

// Workspace of the unit-balanced GEMV: warps whose run of units starts or ends inside a row tile leave their partial
// sums here, and the last one to arrive at a tile (a ticket per tile) adds them in warp order and stores the result.
struct SplitWs {
    float* partial = nullptr;     // [pass][warp][2 slots][tiles per pass x 64]
    unsigned* tickets = nullptr;  // [pass][row tile], zero between launches
};
constexpr size_t kSplitWsFloats = 1u << 20;   // 4 MiB of partial sums per context
constexpr size_t kSplitTickets = 1u << 14;

// Tunables read once from the environment (FERRIC_CUDA_*), the counterpart of the reference's
// FERRIC_* kernel-selection flags (docs/FLAGS.md, crates/ferric-tensor/src/dtype.rs:2173-2187).
struct GemvTuning {
    int wk = 0;        // warps of a CTA that split K (0 = choose from the shape)
    int sm_count = 148;
    int push_cluster = 0;   // CTAs (a cluster) sharing one tile of the pushed exchange's consumer: 1, 2, 4 or 8; 0 = from the world size
    bool stream = false;    // Q6_K plain / pushed GEMV in its unit-balanced form (FERRIC_CUDA_GEMV_STREAM=1; measured no faster)
    int stream_ctas = 0;    // its grid; 0 = one CTA per resident slot (FERRIC_CUDA_GEMV_STREAM_CTAS, for tests on small matrices)
    SplitWs split_ws;       // the context's workspace for that (not a tunable: it rides here to reach the launchers)
    int wait_spins = 0;     // bound of every wait on a peer, in polling rounds (FERRIC_CUDA_PEER_WAIT_SPINS; 0 = the defaults, about a second)
    bool pdl = true;   // programmatic dependent launch between consecutive kernels (FERRIC_CUDA_PDL=0 disables)
};

int32_t launch_repack(cudaStream_t st, uint32_t ty, const uint8_t* src, DeviceWeights& w, size_t src_nblk,
                      size_t row0, size_t blk0);
int32_t launch_dequant_weights(cudaStream_t st, uint32_t ty, const DeviceWeights& w, void* out, bool bf16);
int32_t launch_dequant_raw(cudaStream_t st, uint32_t ty, const uint8_t* raw, size_t n, void* out, bool bf16);

// Bytes of activation-fragment scratch a matmul with m activation rows needs for this matrix.
size_t frag_bytes(uint32_t ty, const DeviceWeights& w, size_t m);
// x[m, cols] (f32, row stride ldx) -> tensor-core B fragments in `frag`.
int32_t launch_prep(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx,
                    void* frag, const GemvTuning& tune);
// Fused (sum, norm) = add_rmsnorm(a, b, weight) and activation preparation of `norm` (row length
// w.cols) in one kernel; sum / norm may be null when the caller does not need them in memory.
int32_t launch_norm_prep(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* a, const float* b,
                         const float* weight, float eps, size_t m, float* sum, float* norm, void* frag,
                         const GemvTuning& tune, const PeerSum& peers = PeerSum(), const PushSrc& pushed = PushSrc());
// One CTA: bump this rank's exchange count and publish it to every peer's flag slot for this rank.
int32_t launch_tp_signal(cudaStream_t st, unsigned* epoch, unsigned* const* peer_flag_slots, int world,
                         const GemvTuning& tune);
// y[m, rows] (row stride ldy) = x . W^T from prepared fragments.  With kEpiSwiglu the matrix is
// [gate rows | up rows] and y is [m, rows/2] = silu(gate) * up.
// With kEpiPush y is not written: the values go to every rank named by `push` (ldy = row length there).
// `chain` (one pass of at most kChainMaxRows activation rows only) adds the input scaling and the output job above.
int32_t launch_gemv(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const void* frag, size_t m, float* y,
                    size_t ldy, Epilogue epi, const GemvTuning& tune, const PushDst& push = PushDst(),
                    const Chain* chain = nullptr);
// Activation tiles (of two rows) the GEMV works on for m rows, padded to whole passes.
size_t gemv_padded_tiles(size_t m);
// Indexed products (IdSel): `pairs` = tokens x k launch passes over an expert-major matrix; y[pair][rows per expert]
// (rows per expert / 2 with kEpiSwiglu), row stride ldy.
int32_t launch_gemv_id(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const void* frag, size_t m, size_t pairs, float* y,
                       size_t ldy, Epilogue epi, const GemvTuning& tune, const IdSel& id);
// out[t][o] = sum over s in slot order of selw[t][s] * part[t * k + s][o]
int32_t launch_id_wsum(cudaStream_t st, const float* part, const float* selw, size_t t, size_t k, size_t out_pe, float* out,
                       const GemvTuning& tune);
// Q8_0 needs no fragments: y = x . W^T straight from f32 activations.
int32_t launch_gemv_q8_0(cudaStream_t st, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y,
                         size_t ldy, const GemvTuning& tune);
// Dense f32 weights [rows, cols] (the fallback for formats without a packed kernel): y = x . W^T.
int32_t launch_gemv_f32(cudaStream_t st, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y,
                        size_t ldy, const GemvTuning& tune);
// out[t, d] = silu(gu[t, d]) * gu[t, d + ..] on a [t, 2d] tensor (the unfused twin).
int32_t launch_swiglu(cudaStream_t st, const float* gu, size_t t, size_t d, float* out, const GemvTuning& tune);

// (sum, norm) = (a + b, rmsnorm(a + b) * weight); b and weight may be null (no add / unit weight),
// sum may be null.
int32_t launch_add_rmsnorm(cudaStream_t st, const float* a, const float* b, const float* weight, float eps,
                           size_t rows, size_t d, float* sum, float* norm, const GemvTuning& tune);

// Prefill product on the tcgen05 tensor cores: y[m, rows] (f32, row stride ldy) = x . W^T with Q4_K or Q6_K weights
// dequantised to bf16 (round to nearest even) and bf16 activations x[m, cols] (row stride ldx elements).
// `workspace` holds gemm_workspace_bytes() bytes (0 when no tile of the launch is cut along K); without it no tile is cut.
size_t gemm_workspace_bytes(const DeviceWeights& w, size_t m, int sm_count);
int32_t launch_gemm_bf16(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const uint16_t* x_bf16, size_t m, size_t ldx,
                         float* y, size_t ldy, void* workspace, int sm_count);
// Batched decode product on the tensor cores on integer-valued f16 operands (Q4_K, Q5_K from 9 rows, Q6_K from 13): preparation,
// product and, for K-split or SwiGLU, a finish kernel.  `scratch` holds gemv_tc_scratch_bytes() bytes.
bool gemv_tc_eligible(uint32_t ty, const DeviceWeights& w, size_t m);
size_t gemv_tc_scratch_bytes(uint32_t ty, const DeviceWeights& w, size_t m, Epilogue epi, int sm_count);
// With `scatter` (plain store, K cut across CTAs, rows a multiple of 4) the finish kernel stores the result not into y but, as
// step 1 of the two-step pushed all-reduce, into the slice owners' memory, and *scattered says that it did.
int32_t launch_gemv_tc(cudaStream_t st, uint32_t ty, const DeviceWeights& w, const float* x, size_t m, size_t ldx, float* y, size_t ldy,
                       Epilogue epi, void* scratch, const GemvTuning& tune, int* launches, const WideDst* scatter = nullptr,
                       bool* scattered = nullptr);
// Synchronise the stream and fetch-and-clear the code a GEMM CTA left when one of its bounded waits ran out.
int32_t gemm_status(cudaStream_t st, int* code);

}  // namespace ferric
