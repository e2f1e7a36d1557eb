/*
 * ferric_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-file CPU restatement of the reference's (dcharlot-physicalai-bmi/ferric) own
 * CPU arithmetic for the quantized-GGUF matmul path.  It exists so the CUDA kernels have something
 * to be compared against bit for bit (dequantised weights) and within tolerance (dot products).
 * Nothing in the shipped library links, loads or calls this file; only tests/, the smoke check and
 * the bench's CPU-baseline leg do.
 *
 * Build with:  gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC -pthread
 * (-ffp-contract=off matters: the reference is Rust, which never contracts a*b+c into an FMA, so
 * every mul/add below must round separately.)
 *
 * Parity status: PINNED by the reference's own known-answer tests, restated in tests/ and
 * tests/golden/ (f16 specials, the hand-built Q4_K block, the Q8_0 quantise round trip, bf16 RNE,
 * packed-vs-dequant agreement, thread/span invariance).  The reference holds no golden values for
 * Q6_K or Q5_K; their layouts here follow the reference decoders line by line and are cross-checked
 * bit for bit against an independently written numpy decoder (for those two formats that
 * cross-check, not a reference vector, is the pin).
 *
 * Each function names the reference file:line it follows (paths relative to the reference root).
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FO_OK 0
#define FO_ERR_TYPE -1   /* unsupported ggml type (reference: Err(String)) */
#define FO_ERR_SHAPE -2  /* a reference assert!/panic: cols not a block multiple, wrong byte length */
#define FO_ERR_ARG -3

enum { GGML_F32 = 0, GGML_F16 = 1, GGML_Q8_0 = 8, GGML_Q4_K = 12, GGML_Q5_K = 13, GGML_Q6_K = 14, GGML_BF16 = 30 };

/* ---------------------------------------------------------------------------------------------
 * IEEE binary16 -> f32, including subnormals, inf and nan.
 * crates/ferric-tensor/src/cpu_simd.rs:29-48 (hand-rolled twin of half::f16::to_f32 used by
 * crates/ferric-gguf/src/lib.rs:605 `rd_f16`).
 * ------------------------------------------------------------------------------------------- */
float fo_f16_to_f32(uint16_t bits)
{
    uint32_t sign = (uint32_t)(bits >> 15) & 1u;
    uint32_t exp = (uint32_t)(bits >> 10) & 0x1Fu;
    uint32_t man = (uint32_t)bits & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign << 31;
        } else {
            /* subnormal: value = man * 2^-24; shift until the implicit bit appears */
            uint32_t m = man, k = 0;
            while ((m & 0x400u) == 0) { m <<= 1; k++; }
            out = (sign << 31) | ((113u - k) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) {
        out = (sign << 31) | 0x7F800000u | (man << 13);
    } else {
        out = (sign << 31) | ((exp + 127u - 15u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* f32 -> binary16, round to nearest even (what half::f16::from_f32 does; needed only by the
 * fixture generators below, which the reference writes with f16::from_f32:
 * crates/ferric-tensor/examples/q4_k.rs:15-18, q6_k.rs:14-15, crates/ferric-gguf/src/lib.rs:990). */
uint16_t fo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t e = (x >> 23) & 0xFFu;
    uint32_t m = x & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? (0x200u | (m >> 13)) : 0));
    int32_t ne = (int32_t)e - 127 + 15;
    if (ne >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (ne <= 0) {
        if (ne < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - ne);
        uint32_t hm = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t h = ((uint32_t)ne << 10) | (m >> 13);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

/* f32 -> bf16 bits, round to nearest even with the reference's add-bias rule.
 * crates/ferric-tensor/src/dtype.rs:4159-4163 (`bf16_rne` in QUANTIZE_WGSL). */
uint16_t fo_bf16_rne(float x)
{
    uint32_t b;
    memcpy(&b, &x, 4);
    uint32_t r = b + 0x7FFFu + ((b >> 16) & 1u);
    return (uint16_t)(r >> 16);
}

float fo_bf16_to_f32(uint16_t h)
{
    uint32_t b = (uint32_t)h << 16; /* crates/ferric-tensor/src/dtype.rs:4149-4150 */
    float f;
    memcpy(&f, &b, 4);
    return f;
}

/* ---------------------------------------------------------------------------------------------
 * On-disk bytes for n elements.  crates/ferric-gguf/src/lib.rs:471-494, restricted to the types
 * this path carries (the three packed formats plus the three plain float types deq_raw widens).
 * ------------------------------------------------------------------------------------------- */
int fo_type_size(uint32_t ty, size_t n, size_t *out)
{
    switch (ty) {
    case GGML_F32: *out = n * 4; return FO_OK;
    case GGML_F16: *out = n * 2; return FO_OK;
    case GGML_BF16: *out = n * 2; return FO_OK;
    case GGML_Q8_0: *out = n / 32 * 34; return FO_OK;
    case GGML_Q4_K: *out = n / 256 * 144; return FO_OK;
    case GGML_Q5_K: *out = n / 256 * 176; return FO_OK;
    case GGML_Q6_K: *out = n / 256 * 210; return FO_OK;
    default: return FO_ERR_TYPE;
    }
}

/* (values per block, bytes per block) for a type with a native packed matmul.
 * crates/ferric-tensor/src/dtype.rs:873-889, rows 8 / 12 / 14. */
int fo_block_bytes(uint32_t ty, size_t *vals, size_t *bytes)
{
    switch (ty) {
    case GGML_Q8_0: *vals = 32; *bytes = 34; return FO_OK;
    case GGML_Q4_K: *vals = 256; *bytes = 144; return FO_OK;
    case GGML_Q5_K: *vals = 256; *bytes = 176; return FO_OK;
    case GGML_Q6_K: *vals = 256; *bytes = 210; return FO_OK;
    default: return FO_ERR_TYPE;
    }
}

/* Q8_0: [f16 d][i8 qs[32]], value = q * d.  crates/ferric-gguf/src/lib.rs:608-615. */
static void deq_q8_0(const uint8_t *raw, size_t n, float *out)
{
    size_t nb = n / 32;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = raw + b * 34;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int j = 0; j < 32; j++) out[b * 32 + j] = (float)(int8_t)blk[2 + j] * d;
    }
}

/* Q6_K: [ql[128]][qh[64]][i8 scales[16]][f16 d], value = d * scale * (q - 32).
 * crates/ferric-gguf/src/lib.rs:721-746.  The product is formed left to right: (d*scale)*q. */
static void deq_q6_k(const uint8_t *raw, size_t n, float *out)
{
    size_t nb = n / 256;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = raw + b * 210;
        float d = fo_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float *y = out + b * 256;
        for (int half = 0; half < 2; half++) {
            const uint8_t *qlh = ql + half * 64, *qhh = qh + half * 32;
            const int8_t *sch = sc + half * 8;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (int)((qlh[l] & 0xF) | (((qhh[l] >> 0) & 3) << 4)) - 32;
                int q2 = (int)((qlh[l + 32] & 0xF) | (((qhh[l] >> 2) & 3) << 4)) - 32;
                int q3 = (int)((qlh[l] >> 4) | (((qhh[l] >> 4) & 3) << 4)) - 32;
                int q4 = (int)((qlh[l + 32] >> 4) | (((qhh[l] >> 6) & 3) << 4)) - 32;
                float t;
                t = d * (float)sch[is];     y[l]      = t * (float)q1;
                t = d * (float)sch[is + 2]; y[l + 32] = t * (float)q2;
                t = d * (float)sch[is + 4]; y[l + 64] = t * (float)q3;
                t = d * (float)sch[is + 6]; y[l + 96] = t * (float)q4;
            }
            y += 128;
        }
    }
}

/* The 6-bit (scale, min) pair j of a Q4_K block's 12 packed bytes.
 * crates/ferric-gguf/src/lib.rs:795-804 (`get_sc_min`). */
static void q4k_sc_min(const uint8_t *s, int j, uint8_t *sc, uint8_t *mn)
{
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* Q4_K: [f16 d][f16 dmin][scales[12]][qs[128]]; four 64-value groups, low nibbles (sub-block is)
 * then high nibbles (is+1); value = (d*sc)*q - (dmin*m).  crates/ferric-gguf/src/lib.rs:793-825. */
static void deq_q4_k(const uint8_t *raw, size_t n, float *out)
{
    size_t nb = n / 256;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = raw + b * 144;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = fo_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        float *y = out + b * 256;
        int is = 0;
        for (int grp = 0; grp < 4; grp++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_sc_min(scales, is, &sc1, &m1);
            q4k_sc_min(scales, is + 1, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
            float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) { float p = d1 * (float)(qs[l] & 0x0F); y[l] = p - mm1; }
            for (int l = 0; l < 32; l++) { float p = d2 * (float)(qs[l] >> 4); y[l + 32] = p - mm2; }
            y += 64; qs += 32; is += 2;
        }
    }
}

/* Q5_K: [f16 d][f16 dmin][scales[12]][qh[32]][qs[128]] = 176 bytes; Q4_K with a fifth bit: group jg takes bit 2*jg
 * of qh[l] for its low-nibble values and bit 2*jg+1 for its high-nibble values, worth 16.
 * crates/ferric-gguf/src/lib.rs:690-716. */
static void deq_q5_k(const uint8_t *raw, size_t n, float *out)
{
    size_t nb = n / 256;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = raw + b * 176;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = fo_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        float *y = out + b * 256;
        int is = 0;
        for (int jg = 0; jg < 4; jg++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_sc_min(scales, is, &sc1, &m1);
            q4k_sc_min(scales, is + 1, &sc2, &m2);
            float d1 = d * (float)sc1, mm1 = dmin * (float)m1;
            float d2 = d * (float)sc2, mm2 = dmin * (float)m2;
            uint8_t b1 = (uint8_t)(1u << (2 * jg)), b2 = (uint8_t)(1u << (2 * jg + 1));
            for (int l = 0; l < 32; l++) {
                float p = d1 * (float)((qs[l] & 0x0F) + ((qh[l] & b1) ? 16 : 0));
                y[l] = p - mm1;
            }
            for (int l = 0; l < 32; l++) {
                float p = d2 * (float)((qs[l] >> 4) + ((qh[l] & b2) ? 16 : 0));
                y[l + 32] = p - mm2;
            }
            y += 64; qs += 32; is += 2;
        }
    }
}

/* Dispatch on ggml type id; unknown type is an error, never a silent zero.
 * crates/ferric-gguf/src/lib.rs:497-520.  `raw_len` is checked against type_size so a short
 * buffer is reported instead of read past (the reference slices and would panic). */
int fo_deq_raw(const uint8_t *raw, size_t raw_len, size_t n, uint32_t ty, float *out)
{
    size_t need;
    if (fo_type_size(ty, n, &need) != FO_OK) return FO_ERR_TYPE;
    if (raw_len < need) return FO_ERR_SHAPE;
    switch (ty) {
    case GGML_F32: memcpy(out, raw, n * 4); return FO_OK;
    case GGML_F16:
        for (size_t i = 0; i < n; i++) out[i] = fo_f16_to_f32((uint16_t)(raw[2 * i] | (raw[2 * i + 1] << 8)));
        return FO_OK;
    case GGML_BF16:
        for (size_t i = 0; i < n; i++) out[i] = fo_bf16_to_f32((uint16_t)(raw[2 * i] | (raw[2 * i + 1] << 8)));
        return FO_OK;
    case GGML_Q8_0: deq_q8_0(raw, n, out); return FO_OK;
    case GGML_Q4_K: deq_q4_k(raw, n, out); return FO_OK;
    case GGML_Q5_K: deq_q5_k(raw, n, out); return FO_OK;
    case GGML_Q6_K: deq_q6_k(raw, n, out); return FO_OK;
    default: return FO_ERR_TYPE;
    }
}

/* Dequantise straight to bf16 bits: bf16_rne(deq_raw(..)), the rounding the prefill kernel's
 * dequant-to-bf16 stage must reproduce bit for bit. */
int fo_deq_raw_bf16(const uint8_t *raw, size_t raw_len, size_t n, uint32_t ty, uint16_t *out)
{
    float *tmp = (float *)malloc((n ? n : 1) * sizeof(float));
    if (!tmp) return FO_ERR_ARG;
    int rc = fo_deq_raw(raw, raw_len, n, ty, tmp);
    if (rc == FO_OK) for (size_t i = 0; i < n; i++) out[i] = fo_bf16_rne(tmp[i]);
    free(tmp);
    return rc;
}

/* c[i,j] = (sum_l a[i,l] * b[j,l]) * scale, sequential f32, l ascending.
 * crates/ferric-core/src/kernels.rs:906-916 (`cpu::matmul_bt`). */
void fo_matmul_bt(const float *a, const float *b, size_t m, size_t n, size_t k, float scale, float *c)
{
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float acc = 0.0f;
            for (size_t l = 0; l < k; l++) acc += a[i * k + l] * b[j * k + l];
            c[i * n + j] = acc * scale;
        }
}

/* ---------------------------------------------------------------------------------------------
 * Shape checks of the packed weight constructors: cols a block multiple, exact byte length.
 * crates/ferric-tensor/src/dtype.rs:1389-1390 (Q4_K), :1148-1149 (Q6_K), :1271-1272 (Q8_0).
 * ------------------------------------------------------------------------------------------- */
static int check_packed(uint32_t ty, size_t len, size_t rows, size_t cols, size_t *row_bytes)
{
    size_t vals, bytes;
    if (fo_block_bytes(ty, &vals, &bytes) != FO_OK) return FO_ERR_TYPE;
    if (cols % vals != 0) return FO_ERR_SHAPE;
    *row_bytes = cols / vals * bytes;
    if (len != rows * *row_bytes) return FO_ERR_SHAPE;
    return FO_OK;
}

/* ---- row kernels -------------------------------------------------------------------------- */

/* The literal reference CPU semantics for y = x . W^T on a packed weight: dequantise the row
 * (deq_raw), then the sequential f32 dot of matmul_bt.  This is what the reference's own kernel
 * tests compare the GPU against (crates/ferric-tensor/examples/q4_k.rs:48-51, q6_k.rs:27-30,
 * q8_0.rs:15-18).  `scratch` holds one dequantised row. */
static float row_dequant_dot(const float *x, const uint8_t *rowbytes, size_t cols, uint32_t ty, float *scratch)
{
    switch (ty) {
    case GGML_Q8_0: deq_q8_0(rowbytes, cols, scratch); break;
    case GGML_Q4_K: deq_q4_k(rowbytes, cols, scratch); break;
    case GGML_Q5_K: deq_q5_k(rowbytes, cols, scratch); break;
    default: deq_q6_k(rowbytes, cols, scratch); break;
    }
    float acc = 0.0f;
    for (size_t l = 0; l < cols; l++) acc += x[l] * scratch[l];
    return acc;
}

/* Same, but the row is rounded to bf16 first and x is bf16 bits: the reference product for the
 * tensor-core prefill configuration (bf16 operands, f32 accumulate). */
static float row_dequant_dot_bf16(const uint16_t *xb, const uint8_t *rowbytes, size_t cols, uint32_t ty, float *scratch)
{
    switch (ty) {
    case GGML_Q8_0: deq_q8_0(rowbytes, cols, scratch); break;
    case GGML_Q4_K: deq_q4_k(rowbytes, cols, scratch); break;
    case GGML_Q5_K: deq_q5_k(rowbytes, cols, scratch); break;
    default: deq_q6_k(rowbytes, cols, scratch); break;
    }
    float acc = 0.0f;
    for (size_t l = 0; l < cols; l++) acc += fo_bf16_to_f32(xb[l]) * fo_bf16_to_f32(fo_bf16_rne(scratch[l]));
    return acc;
}

/* One Q8_0 row in the reference's CPU matvec order: a 32-wide partial per block, scaled once.
 * crates/ferric-tensor/src/cpu_simd.rs:57-72 (`row_q8_0`). */
static float row_fused_q8_0(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 32;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 34;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        const float *xs = x + b * 32;
        float part = 0.0f;
        for (int j = 0; j < 32; j++) part += xs[j] * (float)(int8_t)blk[2 + j];
        acc += part * d;
    }
    return acc;
}

/* Q4_K row in the same fused shape (the reference has no CPU Q4_K matvec; this extends row_q8_0's
 * structure using the per-sub-block factoring of the reference's own Q4_K kernel,
 * crates/ferric-tensor/src/dtype.rs:2283-2294: ds*sum(x*q) - mm*sum(x)). */
static float row_fused_q4_k(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 144;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = fo_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        const float *xs = x + b * 256;
        for (int grp = 0; grp < 4; grp++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_sc_min(scales, 2 * grp, &sc1, &m1);
            q4k_sc_min(scales, 2 * grp + 1, &sc2, &m2);
            float dot1 = 0.0f, sum1 = 0.0f, dot2 = 0.0f, sum2 = 0.0f;
            for (int l = 0; l < 32; l++) {
                dot1 += xs[l] * (float)(qs[l] & 0x0F); sum1 += xs[l];
                dot2 += xs[l + 32] * (float)(qs[l] >> 4); sum2 += xs[l + 32];
            }
            acc += (d * (float)sc1) * dot1 - (dmin * (float)m1) * sum1;
            acc += (d * (float)sc2) * dot2 - (dmin * (float)m2) * sum2;
            xs += 64; qs += 32;
        }
    }
    return acc;
}

/* Q6_K row, fused: per 16-value sub-block an integer-valued partial, scaled by d*scale. */
static float row_fused_q6_k(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 210;
        float d = fo_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
        const int8_t *sc = (const int8_t *)(blk + 192);
        const float *xs = x + b * 256;
        for (int half = 0; half < 2; half++) {
            const uint8_t *qlh = blk + half * 64, *qhh = blk + 128 + half * 32;
            for (int k = 0; k < 4; k++)
                for (int is = 0; is < 2; is++) {
                    float part = 0.0f;
                    for (int j = 0; j < 16; j++) {
                        int l = is * 16 + j;
                        int lo = (k & 1) ? qlh[l + 32] : qlh[l];
                        lo = (k & 2) ? (lo >> 4) : (lo & 0xF);
                        int q = (lo | (((qhh[l] >> (2 * k)) & 3) << 4)) - 32;
                        part += xs[half * 128 + k * 32 + l] * (float)q;
                    }
                    acc += part * (d * (float)sc[half * 8 + is + 2 * k]);
                }
        }
    }
    return acc;
}

/* ---- shader-order rows: the reference GPU kernels' arithmetic, lane-sequential ------------- */

/* Flat Q4_K kernel: per code word, acc = acc + ds*dot(x4, nib4) - mm*(x.x+x.y+x.z+x.w).
 * crates/ferric-tensor/src/dtype.rs:2283-2294 (Q4_K_INNER) inside :2995-3019. */
static float row_shader_q4_k(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 144;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = fo_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        for (int s = 0; s < 8; s++) {
            uint8_t sc, mn;
            q4k_sc_min(scales, s, &sc, &mn);
            float ds = d * (float)sc, mm = dmin * (float)mn;
            const uint8_t *cw = qs + 32 * (s >> 1);
            int hi = s & 1;
            const float *xv = x + b * 256 + 32 * s;
            for (int w = 0; w < 8; w++) {
                float nib[4];
                for (int j = 0; j < 4; j++) nib[j] = (float)(hi ? (cw[4 * w + j] >> 4) : (cw[4 * w + j] & 0xF));
                const float *xw = xv + 4 * w;
                float dot = xw[0] * nib[0] + xw[1] * nib[1] + xw[2] * nib[2] + xw[3] * nib[3];
                float sum = xw[0] + xw[1] + xw[2] + xw[3];
                acc = acc + ds * dot - mm * sum;
            }
        }
    }
    return acc;
}

/* Flat Q6_K kernel: acc = acc + x*d*scale*q, four per l.
 * crates/ferric-tensor/src/dtype.rs:3061-3079 (Q6_K_BODY) inside :3423-3442. */
static float row_shader_q6_k(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 256;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 210;
        float d = fo_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
        const int8_t *sc = (const int8_t *)(blk + 192);
        for (int hf = 0; hf < 2; hf++) {
            const uint8_t *ql = blk + 64 * hf, *qh = blk + 128 + 32 * hf;
            const int8_t *sch = sc + 8 * hf;
            const float *xh = x + b * 256 + 128 * hf;
            for (int l = 0; l < 32; l++) {
                int is = l >> 4, h = qh[l];
                int q1 = (int)((ql[l] & 0xF) | ((h & 3) << 4)) - 32;
                int q2 = (int)((ql[l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql[l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
                acc = acc + xh[l] * d * (float)sch[is] * (float)q1;
                acc = acc + xh[32 + l] * d * (float)sch[is + 2] * (float)q2;
                acc = acc + xh[64 + l] * d * (float)sch[is + 4] * (float)q3;
                acc = acc + xh[96 + l] * d * (float)sch[is + 6] * (float)q4;
            }
        }
    }
    return acc;
}

/* Flat Q8_0 kernel: per word, acc = acc + d*dot(x4, sext4(word)).
 * crates/ferric-tensor/src/dtype.rs:3473-3497. */
static float row_shader_q8_0(const float *x, const uint8_t *blocks, size_t cols)
{
    size_t nb = cols / 32;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = blocks + b * 34;
        float d = fo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int w = 0; w < 8; w++) {
            const float *xw = x + b * 32 + 4 * w;
            const int8_t *q = (const int8_t *)(blk + 2 + 4 * w);
            float dot = xw[0] * (float)q[0] + xw[1] * (float)q[1] + xw[2] * (float)q[2] + xw[3] * (float)q[3];
            acc = acc + d * dot;
        }
    }
    return acc;
}

/* ---- threaded driver: contiguous row spans, results in row order ---------------------------
 * crates/ferric-tensor/src/cpu_simd.rs:92-112 (`matvec_q8_0_threaded`): threads clamp to
 * [1, rows], per = ceil(rows/threads), thread t owns rows [t*per, min(rows,(t+1)*per)). */
enum { FO_MODE_DEQUANT_DOT = 0, FO_MODE_FUSED = 1, FO_MODE_SHADER = 2, FO_MODE_BF16 = 3 };

typedef struct {
    const uint8_t *w;
    const void *x;
    float *y;
    size_t rows, cols, row_bytes, m, lo, hi;
    uint32_t ty;
    int mode;
} span_job;

static void *span_worker(void *arg)
{
    span_job *j = (span_job *)arg;
    float *scratch = (float *)malloc((j->cols ? j->cols : 1) * sizeof(float));
    for (size_t r = j->lo; r < j->hi; r++) {
        const uint8_t *rb = j->w + r * j->row_bytes;
        for (size_t t = 0; t < j->m; t++) {
            float v;
            if (j->mode == FO_MODE_BF16) {
                v = row_dequant_dot_bf16((const uint16_t *)j->x + t * j->cols, rb, j->cols, j->ty, scratch);
            } else {
                const float *x = (const float *)j->x + t * j->cols;
                /* Q5_K has neither a CPU kernel nor a separately restated shader order: every mode is the reference product */
                if (j->mode == FO_MODE_DEQUANT_DOT || j->ty == GGML_Q5_K) v = row_dequant_dot(x, rb, j->cols, j->ty, scratch);
                else if (j->mode == FO_MODE_FUSED)
                    v = j->ty == GGML_Q8_0 ? row_fused_q8_0(x, rb, j->cols)
                      : j->ty == GGML_Q4_K ? row_fused_q4_k(x, rb, j->cols) : row_fused_q6_k(x, rb, j->cols);
                else
                    v = j->ty == GGML_Q8_0 ? row_shader_q8_0(x, rb, j->cols)
                      : j->ty == GGML_Q4_K ? row_shader_q4_k(x, rb, j->cols) : row_shader_q6_k(x, rb, j->cols);
            }
            j->y[t * j->rows + r] = v;
        }
    }
    free(scratch);
    return NULL;
}

/* y[m, rows] = x[m, cols] . W^T for a packed weight given as raw GGUF block bytes.
 * mode 0: dequantise-then-sequential-dot (the reference product, see row_dequant_dot);
 * mode 1: fused per-block rows in the cpu_simd shape; mode 2: the flat GPU kernels' order;
 * mode 3: bf16 operands (x is uint16 bf16 bits).  `threads` as in matvec_q8_0_threaded. */
int fo_matmul_q(const uint8_t *w, size_t len, uint32_t ty, size_t rows, size_t cols,
                const void *x, size_t m, float *y, int threads, int mode)
{
    size_t row_bytes;
    int rc = check_packed(ty, len, rows, cols, &row_bytes);
    if (rc != FO_OK) return rc;
    if (mode < 0 || mode > 3) return FO_ERR_ARG;
    size_t nt = threads < 1 ? 1 : (size_t)threads;
    if (nt > (rows ? rows : 1)) nt = rows ? rows : 1;
    size_t per = (rows + nt - 1) / nt;
    span_job *jobs = (span_job *)calloc(nt, sizeof(span_job));
    pthread_t *tid = (pthread_t *)calloc(nt, sizeof(pthread_t));
    size_t used = 0;
    for (size_t t = 0; t < nt; t++) {
        size_t lo = t * per, hi = lo + per < rows ? lo + per : rows;
        if (lo >= hi) break;
        span_job j = { w, x, y, rows, cols, row_bytes, m, lo, hi, ty, mode };
        jobs[used] = j;
        if (nt == 1) span_worker(&jobs[used]);
        else pthread_create(&tid[used], NULL, span_worker, &jobs[used]);
        used++;
    }
    if (nt > 1) for (size_t t = 0; t < used; t++) pthread_join(tid[t], NULL);
    free(jobs);
    free(tid);
    return FO_OK;
}

/* A contiguous span [lo, hi) of output rows only (m = 1): crates/ferric-tensor/src/cpu_simd.rs:118-122. */
int fo_matvec_span(const uint8_t *w, size_t len, uint32_t ty, size_t rows, size_t cols,
                   const float *x, size_t lo, size_t hi, float *y, int threads, int mode)
{
    size_t row_bytes;
    int rc = check_packed(ty, len, rows, cols, &row_bytes);
    if (rc != FO_OK) return rc;
    if (lo > hi || hi > rows) return FO_ERR_ARG;
    return fo_matmul_q(w + lo * row_bytes, (hi - lo) * row_bytes, ty, hi - lo, cols, x, 1, y, threads, mode);
}

/* out[t, j] = silu(gu[t, j]) * gu[t, d + j] with silu(g) = g / (1 + exp(-g)).
 * crates/ferric-tensor/src/lib.rs:2603-2618 (SWIGLU_WGSL); gate rows are stacked first, then up
 * (crates/ferric-llama/src/qwen35.rs:431). */
void fo_swiglu(const float *gu, size_t t, size_t d, float *out)
{
    for (size_t r = 0; r < t; r++)
        for (size_t c = 0; c < d; c++) {
            float g = gu[r * 2 * d + c], u = gu[r * 2 * d + d + c];
            out[r * d + c] = (g / (1.0f + expf(-g))) * u;
        }
}

/* (sum, norm) = (a + b, rmsnorm(a + b) * weight): one sequential f32 pass per row for the mean of
 * squares, inv = 1 / sqrt(ms / d + eps), norm = s * inv * w.  b NULL = plain rmsnorm, w NULL = ones.
 * crates/ferric-tensor/src/lib.rs:2057-2075 (ADD_RMSNORM_WGSL), :2018-2032 (RMSNORM_WGSL). */
void fo_add_rmsnorm(const float *a, const float *b, const float *w, float eps, size_t rows, size_t d,
                    float *sum, float *norm)
{
    for (size_t r = 0; r < rows; r++) {
        size_t base = r * d;
        float ms = 0.0f;
        for (size_t j = 0; j < d; j++) {
            float s = b ? a[base + j] + b[base + j] : a[base + j];
            if (sum) sum[base + j] = s;
            ms = ms + s * s;
        }
        float inv = 1.0f / sqrtf(ms / (float)d + eps);
        for (size_t j = 0; j < d; j++) {
            float s = b ? a[base + j] + b[base + j] : a[base + j];
            norm[base + j] = s * inv * (w ? w[j] : 1.0f);
        }
    }
}

/* ---- fixture generators used by the reference's own kernel tests --------------------------- */

/* crates/ferric-gguf/src/lib.rs:985-997 (`quant_q8_0`); out holds ceil(n/32)*34 bytes. */
void fo_quant_q8_0(const float *x, size_t n, uint8_t *out)
{
    for (size_t b0 = 0; b0 < n; b0 += 32) {
        size_t len = n - b0 < 32 ? n - b0 : 32;
        float amax = 0.0f;
        for (size_t i = 0; i < len; i++) { float a = fabsf(x[b0 + i]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        uint16_t h = fo_f32_to_f16(d);
        *out++ = (uint8_t)(h & 0xFF);
        *out++ = (uint8_t)(h >> 8);
        for (size_t i = 0; i < 32; i++) {
            int8_t q = 0;
            if (d != 0.0f) {
                float v = (i < len ? x[b0 + i] : 0.0f) / d;
                float r = roundf(v); /* Rust f32::round: half away from zero */
                if (r < -127.0f) r = -127.0f;
                if (r > 127.0f) r = 127.0f;
                q = (int8_t)r;
            }
            *out++ = (uint8_t)q;
        }
    }
}

/* crates/ferric-tensor/examples/q4_k.rs:13-37 (`q4k_block(seed)`): one 144-byte super-block. */
void fo_q4k_block(uint32_t seed, uint8_t *b)
{
    float d = 0.05f + 0.01f * (float)(seed % 7);
    float dmin = 0.02f + 0.005f * (float)(seed % 5);
    uint16_t hd = fo_f32_to_f16(d), hm = fo_f32_to_f16(dmin);
    b[0] = (uint8_t)(hd & 0xFF); b[1] = (uint8_t)(hd >> 8);
    b[2] = (uint8_t)(hm & 0xFF); b[3] = (uint8_t)(hm >> 8);
    uint8_t s[12];
    memset(s, 0, 12);
    for (uint32_t j = 0; j < 8; j++) {
        uint8_t sc = (uint8_t)((seed * 2654435761u + j * 40503u) % 64u);
        uint8_t mn = (uint8_t)((seed * 40503u + j * 2654435761u) % 64u);
        if (j < 4) {
            s[j] |= sc & 63;
            s[j + 4] |= mn & 63;
        } else {
            s[j + 4] |= (uint8_t)((sc & 0x0F) | ((mn & 0x0F) << 4));
            s[j - 4] |= (uint8_t)((sc >> 4) << 6);
            s[j] |= (uint8_t)((mn >> 4) << 6);
        }
    }
    memcpy(b + 4, s, 12);
    for (uint32_t i = 0; i < 128; i++) b[16 + i] = (uint8_t)((seed + i * 2246822519u) % 256u);
}

/* crates/ferric-tensor/examples/q6_k.rs:9-17 (`q6k_block(seed)`): one 210-byte super-block. */
void fo_q6k_block(uint32_t seed, uint8_t *b)
{
    for (uint32_t i = 0; i < 128; i++) b[i] = (uint8_t)((seed + i * 2246822519u) % 256u);
    for (uint32_t i = 0; i < 64; i++) b[128 + i] = (uint8_t)((seed * 40503u + i * 97u) % 256u);
    for (uint32_t i = 0; i < 16; i++) b[192 + i] = (uint8_t)(int8_t)((int32_t)((seed + i * 7u) % 64u) - 32);
    uint16_t hd = fo_f32_to_f16(0.04f + 0.01f * (float)(seed % 6));
    b[208] = (uint8_t)(hd & 0xFF);
    b[209] = (uint8_t)(hd >> 8);
}

/* crates/ferric-tensor/src/cpu_simd.rs:136-156 (`synth`): an LCG-built Q8_0 weight plus the exact
 * f32 values it encodes (ground truth that does not pass through the decoder under test). */
void fo_q8_0_synth(size_t rows, size_t cols, uint32_t seed, uint8_t *raw, float *vals)
{
    uint32_t s = seed * 2654435761u + 1u;
    size_t nb = cols / 32;
    for (size_t r = 0; r < rows; r++)
        for (size_t b = 0; b < nb; b++) {
            s = s * 1664525u + 1013904223u;
            uint16_t dbits = (uint16_t)(0x1C00u | ((s >> 16) & 0x3Fu));
            *raw++ = (uint8_t)(dbits & 0xFF);
            *raw++ = (uint8_t)(dbits >> 8);
            float d = fo_f16_to_f32(dbits);
            for (int j = 0; j < 32; j++) {
                s = s * 1664525u + 1013904223u;
                uint8_t c = (uint8_t)((s >> 16) & 0xFFu);
                *raw++ = c;
                vals[r * cols + b * 32 + j] = (float)(int8_t)c * d;
            }
        }
}
