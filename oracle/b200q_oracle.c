/*
 * CPU oracle for the GGUF fused quant-matmul path (Q4_K / Q6_K / Q8_0).
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are
 * compared against and the timed CPU baseline; nothing in the product library
 * links, imports or calls it.
 *
 * It restates, in plain C, the host reference that brotensor's own parity
 * tests use as their FP32 ground truth (brotensor's CPU backend has no quant
 * ops):
 *   Q4_K  scale unpack   tests/test_q4k_parity.cpp:73-83
 *   Q4_K  block decode   tests/test_q4k_parity.cpp:166-180
 *   Q6_K  index mapping  tests/test_q6k_parity.cpp:60-66
 *   Q6_K  block decode   tests/test_q6k_parity.cpp:139-151
 *   Q8_0  block decode   tests/test_q8_0_parity.cpp:64-69
 *   matmul               tests/test_q4k_parity.cpp:267-274, 326-335
 *                        (sequential FP32 accumulation, k ascending)
 *   fp16/bf16 <-> fp32   src/tensor.cpp:162-260 (round to nearest even)
 *
 * Two formats have no decoder anywhere in brotensor (its loader carries them as opaque storage,
 * src/gguf.cpp:111-130): Q4_0 and Q5_K. Their decoders below restate ggml's published block
 * definitions (block_q4_0 / dequantize_row_q4_0, block_q5_K / dequantize_row_q5_K of ggml-quants.c;
 * ggml is not part of the reference tree). For these two, parity is pinned to that specification
 * and to a second, independently written numpy restatement in tests/test_formats_extra.py - not to
 * reference code.
 *
 * Parity is pinned: tests/test_oracle.py checks every function here against
 * golden vectors produced by the reference's own functions (compiled from the
 * reference sources into oracle/_ref) and, when that library is present,
 * against the reference functions directly on random blocks.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FMT_Q4_0 10
#define FMT_Q8_0 14
#define FMT_Q4_K 22
#define FMT_Q5_K 23
#define FMT_Q6_K 24

/* ---- scalar conversions -------------------------------------------------- */

float oracle_fp16_to_fp32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else { /* subnormal: value = man * 2^-24 */
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

uint16_t oracle_fp32_to_fp16(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t e8 = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (e8 == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x0200u : 0u));
    int32_t e = (int32_t)e8 - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e;
        uint32_t half = 1u << (shift - 1);
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t r = man >> shift;
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint32_t out = ((uint32_t)e << 10) | r;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++out; /* carry may bump exponent */
    if (out >= 0x7C00u) out = 0x7C00u;
    return (uint16_t)(sign | out);
}

float oracle_bf16_to_fp32(uint16_t b) {
    uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

uint16_t oracle_fp32_to_bf16(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    if ((x & 0x7F800000u) == 0x7F800000u && (x & 0x7FFFFFu)) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

/* ---- block geometry -------------------------------------------------------- */

int oracle_block_elems(int fmt) {
    return (fmt == FMT_Q8_0 || fmt == FMT_Q4_0) ? 32 : (fmt == FMT_Q4_K || fmt == FMT_Q6_K || fmt == FMT_Q5_K) ? 256 : 0;
}
int oracle_block_bytes(int fmt) {
    return fmt == FMT_Q8_0 ? 34 : fmt == FMT_Q4_0 ? 18 : fmt == FMT_Q4_K ? 144 : fmt == FMT_Q5_K ? 176 : fmt == FMT_Q6_K ? 210 : 0;
}

/* ---- Q4_K ------------------------------------------------------------------ */

/* 12 packed bytes -> eight 6-bit scales and eight 6-bit mins. */
void oracle_q4k_unpack_sc_m(const uint8_t s[12], uint8_t sc[8], uint8_t m[8]) {
    for (int j = 0; j < 8; ++j) {
        if (j < 4) {
            sc[j] = s[j] & 0x3F;
            m[j] = s[j + 4] & 0x3F;
        } else {
            sc[j] = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
            m[j] = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
        }
    }
}

/* Inverse of the unpack (tests/test_q4k_parity.cpp:54-71); used by generators. */
void oracle_q4k_pack_sc_m(uint8_t s[12], const uint8_t sc[8], const uint8_t m[8]) {
    memset(s, 0, 12);
    for (int j = 0; j < 4; ++j) {
        s[j] = sc[j] & 0x3F;
        s[j + 4] = m[j] & 0x3F;
    }
    for (int j = 4; j < 8; ++j) {
        s[j + 4] = (uint8_t)((sc[j] & 0x0F) | ((m[j] & 0x0F) << 4));
        s[j - 4] |= (uint8_t)(((sc[j] >> 4) & 3) << 6);
        s[j] |= (uint8_t)(((m[j] >> 4) & 3) << 6);
    }
}

/* 144-byte block: fp16 d @0, fp16 dmin @2, scales[12] @4, qs[128] @16. */
void oracle_q4k_dequant_block(const uint8_t* blk, float* dst) {
    uint16_t dh, mh;
    memcpy(&dh, blk, 2);
    memcpy(&mh, blk + 2, 2);
    const float d = oracle_fp16_to_fp32(dh);
    const float dmin = oracle_fp16_to_fp32(mh);
    uint8_t sc[8], m[8];
    oracle_q4k_unpack_sc_m(blk + 4, sc, m);
    const uint8_t* qs = blk + 16;
    for (int t = 0; t < 256; ++t) {
        const int is = t >> 5, l = t & 31;
        const uint8_t qb = qs[(is >> 1) * 32 + l];
        const int nib = (is & 1) ? (qb >> 4) : (qb & 0x0F);
        /* Every intermediate is exact in FP32 (11+6+4 and 11+6 significant
         * bits), so the value does not depend on contraction or order. */
        dst[t] = d * (float)sc[is] * (float)nib - dmin * (float)m[is];
    }
}

/* ---- Q6_K ------------------------------------------------------------------ */

/* 210-byte block: ql[128] @0, qh[64] @128, int8 scales[16] @192, fp16 d @208. */
void oracle_q6k_dequant_block(const uint8_t* blk, float* dst) {
    uint16_t dh;
    memcpy(&dh, blk + 208, 2);
    const float d = oracle_fp16_to_fp32(dh);
    const uint8_t* ql = blk;
    const uint8_t* qh = blk + 128;
    const int8_t* scales = (const int8_t*)(blk + 192);
    for (int e = 0; e < 256; ++e) {
        const int group = e >> 7;
        const int quad = (e & 127) >> 5;
        const int l = e & 31;
        const int sb = group * 8 + quad * 2 + (l >> 4);
        const uint8_t ql_b = ql[group * 64 + (quad & 1) * 32 + l];
        const uint8_t qh_b = qh[group * 32 + l];
        const int raw4 = (quad < 2) ? (ql_b & 0x0F) : (ql_b >> 4);
        const int hi2 = (qh_b >> (quad * 2)) & 3;
        const int val6 = (raw4 | (hi2 << 4)) - 32;
        dst[e] = d * (float)scales[sb] * (float)val6;
    }
}

/* ---- Q8_0 ------------------------------------------------------------------ */

/* 34-byte block: fp16 d @0, int8 qs[32] @2. */
void oracle_q8_0_dequant_block(const uint8_t* blk, float* dst) {
    uint16_t dh;
    memcpy(&dh, blk, 2);
    const float d = oracle_fp16_to_fp32(dh);
    const int8_t* qs = (const int8_t*)(blk + 2);
    for (int i = 0; i < 32; ++i) dst[i] = d * (float)qs[i];
}

/* ---- Q4_0 (ggml block_q4_0) -------------------------------------------------- */

/* 18-byte block: fp16 d @0, qs[16] @2. Element j < 16 is the low nibble of qs[j], element j + 16 its
 * high nibble; value d * (nibble - 8). */
void oracle_q4_0_dequant_block(const uint8_t* blk, float* dst) {
    uint16_t dh;
    memcpy(&dh, blk, 2);
    const float d = oracle_fp16_to_fp32(dh);
    const uint8_t* qs = blk + 2;
    for (int j = 0; j < 16; ++j) {
        dst[j] = d * (float)((int)(qs[j] & 0x0F) - 8);
        dst[j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
    }
}

/* ---- Q5_K (ggml block_q5_K) -------------------------------------------------- */

/* 176-byte block: fp16 d @0, fp16 dmin @2, scales[12] @4 (the Q4_K packing), qh[32] @16, qs[128] @48.
 * For each 64-element group j = 0..3: the low nibbles of qs[32 j .. 32 j + 31] with bit 2 j of qh[l] as
 * fifth bit are sub-block 2 j, the high nibbles with bit 2 j + 1 sub-block 2 j + 1;
 * value d * sc * q - dmin * m. */
void oracle_q5k_dequant_block(const uint8_t* blk, float* dst) {
    uint16_t dh, mh;
    memcpy(&dh, blk, 2);
    memcpy(&mh, blk + 2, 2);
    const float d = oracle_fp16_to_fp32(dh);
    const float dmin = oracle_fp16_to_fp32(mh);
    uint8_t sc[8], m[8];
    oracle_q4k_unpack_sc_m(blk + 4, sc, m);
    const uint8_t* qh = blk + 16;
    const uint8_t* ql = blk + 48;
    for (int j = 0; j < 4; ++j) {
        for (int l = 0; l < 32; ++l) {
            const int lo = (ql[32 * j + l] & 0x0F) + (((qh[l] >> (2 * j)) & 1) ? 16 : 0);
            const int hi = (ql[32 * j + l] >> 4) + (((qh[l] >> (2 * j + 1)) & 1) ? 16 : 0);
            dst[64 * j + l] = d * (float)sc[2 * j] * (float)lo - dmin * (float)m[2 * j];
            dst[64 * j + 32 + l] = d * (float)sc[2 * j + 1] * (float)hi - dmin * (float)m[2 * j + 1];
        }
    }
}

/* ---- row / matrix level ---------------------------------------------------- */

static void dequant_block(int fmt, const uint8_t* blk, float* dst) {
    if (fmt == FMT_Q4_K) oracle_q4k_dequant_block(blk, dst);
    else if (fmt == FMT_Q6_K) oracle_q6k_dequant_block(blk, dst);
    else if (fmt == FMT_Q5_K) oracle_q5k_dequant_block(blk, dst);
    else if (fmt == FMT_Q4_0) oracle_q4_0_dequant_block(blk, dst);
    else oracle_q8_0_dequant_block(blk, dst);
}

/* W: rows x (K/elems) blocks, row-major. out: rows x K fp32. Returns 0 or -1. */
int oracle_dequant_f32(int fmt, const uint8_t* W, int64_t rows, int K, float* out) {
    const int be = oracle_block_elems(fmt), bb = oracle_block_bytes(fmt);
    if (!be || K % be) return -1;
    const int bpr = K / be;
    for (int64_t r = 0; r < rows; ++r)
        for (int b = 0; b < bpr; ++b)
            dequant_block(fmt, W + ((size_t)r * bpr + b) * bb, out + (size_t)r * K + (size_t)b * be);
    return 0;
}

/* Same, rounded to fp16 (kind 1) or bf16 (kind 4) bit patterns. */
int oracle_dequant_16(int fmt, const uint8_t* W, int64_t rows, int K, int kind, uint16_t* out) {
    const int be = oracle_block_elems(fmt), bb = oracle_block_bytes(fmt);
    if (!be || K % be) return -1;
    const int bpr = K / be;
    float tmp[256];
    for (int64_t r = 0; r < rows; ++r)
        for (int b = 0; b < bpr; ++b) {
            dequant_block(fmt, W + ((size_t)r * bpr + b) * bb, tmp);
            uint16_t* o = out + (size_t)r * K + (size_t)b * be;
            for (int i = 0; i < be; ++i) o[i] = kind == 1 ? oracle_fp32_to_fp16(tmp[i]) : oracle_fp32_to_bf16(tmp[i]);
        }
    return 0;
}

typedef struct {
    int fmt, M, N, K;
    const uint8_t* W;
    const float* X;    /* M x K */
    const float* bias; /* N or NULL */
    float* Y;          /* M x N, fp32-accumulated */
    double* Y64;       /* optional M x N, fp64-accumulated */
    int64_t r0, r1;
} mm_job;

static void* mm_worker(void* p) {
    mm_job* j = (mm_job*)p;
    const int be = oracle_block_elems(j->fmt), bb = oracle_block_bytes(j->fmt);
    const int bpr = j->K / be;
    float* row = (float*)malloc((size_t)j->K * sizeof(float));
    for (int64_t r = j->r0; r < j->r1; ++r) {
        for (int b = 0; b < bpr; ++b) dequant_block(j->fmt, j->W + ((size_t)r * bpr + b) * bb, row + (size_t)b * be);
        for (int m = 0; m < j->M; ++m) {
            const float* x = j->X + (size_t)m * j->K;
            float s = 0.0f;
            for (int k = 0; k < j->K; ++k) s += row[k] * x[k]; /* built with -ffp-contract=off */
            j->Y[(size_t)m * j->N + r] = j->bias ? s + j->bias[r] : s;
            if (j->Y64) {
                double s2 = 0.0;
                for (int k = 0; k < j->K; ++k) s2 += (double)row[k] * (double)x[k];
                j->Y64[(size_t)m * j->N + r] = j->bias ? s2 + (double)j->bias[r] : s2;
            }
        }
    }
    free(row);
    return NULL;
}

/*
 * Y(M,N) = X(M,K) * dequant(W(N,K))^T (+ bias(N)), decoded row by row, each
 * dot product accumulated sequentially in FP32 exactly as the reference tests
 * do. Rows are split over `threads` pthreads (1 = the scalar reference order;
 * results do not depend on the thread count because rows are independent).
 */
int oracle_matmul(int fmt, const uint8_t* W, const float* X, const float* bias, float* Y, double* Y64,
                  int M, int N, int K, int threads) {
    const int be = oracle_block_elems(fmt);
    if (!be || K % be || M < 0 || N < 0) return -1;
    if (threads < 1) threads = 1;
    if (threads > N) threads = N > 0 ? N : 1;
    mm_job* jobs = (mm_job*)calloc((size_t)threads, sizeof(mm_job));
    pthread_t* th = (pthread_t*)calloc((size_t)threads, sizeof(pthread_t));
    for (int t = 0; t < threads; ++t) {
        mm_job j = {fmt, M, N, K, W, X, bias, Y, Y64, (int64_t)N * t / threads, (int64_t)N * (t + 1) / threads};
        jobs[t] = j;
    }
    if (threads == 1) {
        mm_worker(&jobs[0]);
    } else {
        for (int t = 0; t < threads; ++t) pthread_create(&th[t], NULL, mm_worker, &jobs[t]);
        for (int t = 0; t < threads; ++t) pthread_join(th[t], NULL);
    }
    free(jobs);
    free(th);
    return 0;
}
