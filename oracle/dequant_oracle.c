/*
 * CPU oracle for the GGUF block decode path -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A plain-C restatement of the arithmetic in the reference's
 * src/phfe/inference/gguf_loader.py (decode functions at :407-554, final cast
 * at :377-378).  Only tests, the smoke check and the CPU-baseline leg of the
 * benchmark may load this file; the CUDA library never links or calls it.
 *
 * Parity status: pinned.  tests/golden/ holds vectors produced by executing the
 * reference's own Python functions; tests/test_oracle.py checks this file
 * against every one of them bit for bit.
 *
 * All IEEE conversions are done with integer arithmetic so that the result
 * does not depend on compiler flags, x87/SSE modes or _Float16 support.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ggml type ids and block geometry: gguf_loader.py:33-65 */
enum {
    ORACLE_F32 = 0,
    ORACLE_F16 = 1,
    ORACLE_Q4_0 = 2,
    ORACLE_Q4_1 = 3,
    ORACLE_Q8_0 = 8,
    ORACLE_BF16 = 30,
    /* Formats the reference names (gguf_loader.py:37-46) but cannot decode.  Restated from ggml's
     * published dequantize_row_q5_0 / q5_1 / q2_K / q3_K / q4_K / q5_K / q6_K; pinned against the
     * gguf-py package's dequantize() (tests/golden/decode_<type>_ggml.npz), not against the reference. */
    ORACLE_Q5_0 = 6,
    ORACLE_Q5_1 = 7,
    ORACLE_Q2_K = 10,
    ORACLE_Q3_K = 11,
    ORACLE_Q4_K = 12,
    ORACLE_Q5_K = 13,
    ORACLE_Q6_K = 14
};

/* OR-ed into Q4_0 / Q4_1: ggml's own element order (ggml-quants.c dequantize_row_q4_0 /
 * dequantize_row_q4_1 as published: y[j] from the low nibble of qs[j], y[j+16] from the high
 * nibble) instead of the reference's interleaved order.  Not a reference behaviour; pinned
 * against the gguf-py package's dequantize() in tests/golden. */
#define ORACLE_GGML_ORDER 0x100

enum { ORACLE_OUT_F32 = 0, ORACLE_OUT_F16 = 1, ORACLE_OUT_BF16 = 2 };

static int block_elems(int t)
{
    switch (t & ~ORACLE_GGML_ORDER) {
    case ORACLE_F32: case ORACLE_F16: case ORACLE_BF16: return 1;
    case ORACLE_Q4_0: case ORACLE_Q4_1: case ORACLE_Q8_0: case ORACLE_Q5_0: case ORACLE_Q5_1: return 32;
    case ORACLE_Q2_K: case ORACLE_Q3_K: case ORACLE_Q4_K: case ORACLE_Q5_K: case ORACLE_Q6_K: return 256;
    default: return 0;
    }
}

static int block_bytes(int t)
{
    switch (t & ~ORACLE_GGML_ORDER) {
    case ORACLE_F32: return 4;
    case ORACLE_F16: case ORACLE_BF16: return 2;
    case ORACLE_Q4_0: return 18;
    case ORACLE_Q4_1: return 20;
    case ORACLE_Q8_0: return 34;
    case ORACLE_Q5_0: return 22;
    case ORACLE_Q5_1: return 24;
    case ORACLE_Q2_K: return 84;
    case ORACLE_Q3_K: return 110;
    case ORACLE_Q4_K: return 144;
    case ORACLE_Q5_K: return 176;
    case ORACLE_Q6_K: return 210;
    default: return 0;
    }
}

/* GGUFTensorInfo.nbytes, gguf_loader.py:131-139: ceil(numel/blk) * blk_bytes. */
int64_t oracle_nbytes(int ggml_type, int64_t numel)
{
    int be = block_elems(ggml_type);
    if (be == 0) return -1;
    return (numel + be - 1) / be * (int64_t)block_bytes(ggml_type);
}

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* Exact binary16 -> binary32 widening (what numpy float16 -> Python float ->
 * float32 does at gguf_loader.py:455-456, :500-501, :542). */
static float half_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        /* subnormal: man * 2^-24, exact in binary32 */
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round to nearest even, overflow to infinity,
 * subnormals kept (torch.Tensor.to(torch.float16) on CPU, gguf_loader.py:378). */
static uint16_t f32_to_half(float f)
{
    uint32_t x = f32_to_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {                       /* inf or NaN */
        if (ax > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  /* >= 65520 rounds to inf */
    if (ax < 0x33000001u) return sign;             /* <= 2^-25 rounds to zero (tie to even) */
    int32_t e = (int32_t)(ax >> 23) - 127;         /* unbiased exponent */
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;     /* 24-bit significand */
    int shift;                                     /* bits dropped from m */
    uint32_t base;
    if (e >= -14) { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
    else { shift = 13 + (-14 - e); base = 0; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    /* a carry out of the mantissa correctly bumps the exponent field */
    return (uint16_t)(sign | (base + q));
}

/* binary32 -> bfloat16, round to nearest even (torch.Tensor.to(torch.bfloat16)). */
static uint16_t f32_to_bf16(float f)
{
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u); /* quiet NaN */
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

static inline uint16_t rd_u16(const uint8_t *p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

/* One block of 32 values into v[32]; formulas follow the reference exactly. */
static void decode_block(int t, const uint8_t *b, float *v)
{
    if (t & ORACLE_GGML_ORDER) {
        /* same arithmetic as below, ggml's element order */
        int q41 = (t & ~ORACLE_GGML_ORDER) == ORACLE_Q4_1;
        double d = (double)half_to_f32(rd_u16(b));
        double m = q41 ? (double)half_to_f32(rd_u16(b + 2)) : 0.0;
        const uint8_t *qs = b + (q41 ? 4 : 2);
        for (int j = 0; j < 16; j++) {
            int lo = qs[j] & 0x0f, hi = qs[j] >> 4;
            if (q41) { v[j] = (float)((double)lo * d + m); v[j + 16] = (float)((double)hi * d + m); }
            else { v[j] = (float)((double)(lo - 8) * d); v[j + 16] = (float)((double)(hi - 8) * d); }
        }
        return;
    }
    if (t == ORACLE_Q4_0) {
        /* gguf_loader.py:451-474: out[2j] = ((qs[j]&15)-8)*d, out[2j+1] = ((qs[j]>>4)-8)*d.
         * The reference multiplies int16 by a Python float (float64) and stores to
         * float32; the product has at most 4+11 significant bits, so it is exact. */
        double d = (double)half_to_f32(rd_u16(b));
        for (int j = 0; j < 16; j++) {
            int lo = (b[2 + j] & 0x0f) - 8;
            int hi = (b[2 + j] >> 4) - 8;
            v[2 * j] = (float)((double)lo * d);
            v[2 * j + 1] = (float)((double)hi * d);
        }
    } else if (t == ORACLE_Q4_1) {
        /* gguf_loader.py:496-517: q*d + m evaluated in float64 (exact there: the
         * sum spans < 53 bits), then one rounding to float32. */
        double d = (double)half_to_f32(rd_u16(b));
        double m = (double)half_to_f32(rd_u16(b + 2));
        for (int j = 0; j < 16; j++) {
            int lo = b[4 + j] & 0x0f;
            int hi = b[4 + j] >> 4;
            v[2 * j] = (float)((double)lo * d + m);
            v[2 * j + 1] = (float)((double)hi * d + m);
        }
    } else { /* ORACLE_Q8_0, gguf_loader.py:538-552: float32(int8) * d in float32 */
        float d = half_to_f32(rd_u16(b));
        for (int j = 0; j < 32; j++) v[j] = (float)(int8_t)b[2 + j] * d;
    }
}

/* 6-bit scale and minimum of sub-block j of a Q4_K / Q5_K block (12 packed bytes at s). */
static void k4_scale_min(const uint8_t *s, int j, int *sc, int *mn)
{
    if (j < 4) { *sc = s[j] & 63; *mn = s[j + 4] & 63; }
    else { *sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4); *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

/* Element k of one Q5_0 / Q5_1 / K-quant block.  All products before the last operation are
 * exact in float (fp16 scale x small integers), so fmaf / one multiply gives the single rounding
 * that ggml's float code and gguf-py's float32 NumPy code both produce. */
static float extra_element(int t, const uint8_t *b, int k)
{
    if (t == ORACLE_Q5_0 || t == ORACLE_Q5_1) {
        int o = (t == ORACLE_Q5_0) ? 2 : 4;
        uint32_t qh = (uint32_t)b[o] | ((uint32_t)b[o + 1] << 8) | ((uint32_t)b[o + 2] << 16) | ((uint32_t)b[o + 3] << 24);
        int byte = b[o + 4 + (k & 15)];
        int q = ((k & 16) ? (byte >> 4) : (byte & 15)) | (int)(((qh >> k) & 1u) << 4);
        float d = half_to_f32(rd_u16(b));
        if (t == ORACLE_Q5_0) return d * (float)(q - 16);
        return fmaf(d, (float)q, half_to_f32(rd_u16(b + 2)));
    }
    int sb = k >> 5, l = k & 31;
    if (t == ORACLE_Q4_K || t == ORACLE_Q5_K) {
        int sc, mn;
        k4_scale_min(b + 4, sb, &sc, &mn);
        int byte = b[(t == ORACLE_Q4_K ? 16 : 48) + 32 * (sb >> 1) + l];
        int q = (sb & 1) ? (byte >> 4) : (byte & 15);
        if (t == ORACLE_Q5_K) q |= ((b[16 + l] >> sb) & 1) << 4;
        float dl = half_to_f32(rd_u16(b)) * (float)sc;
        float ml = half_to_f32(rd_u16(b + 2)) * (float)mn;
        return fmaf(dl, (float)q, -ml);
    }
    if (t == ORACLE_Q6_K) {
        int half = sb >> 2, r = sb & 3;
        int lo = b[64 * half + 32 * (r & 1) + l], hi = b[128 + 32 * half + l];
        int q = (((r >> 1) ? (lo >> 4) : (lo & 15)) | (((hi >> (2 * r)) & 3) << 4)) - 32;
        float dl = half_to_f32(rd_u16(b + 208)) * (float)(int8_t)b[192 + (k >> 4)];
        return dl * (float)q;
    }
    int half = k >> 7, r = (k >> 5) & 3;
    if (t == ORACLE_Q2_K) {
        int q = (b[16 + 32 * half + l] >> (2 * r)) & 3;
        int s = b[k >> 4];
        float dl = half_to_f32(rd_u16(b + 80)) * (float)(s & 15);
        float ml = half_to_f32(rd_u16(b + 82)) * (float)(s >> 4);
        return fmaf(dl, (float)q, -ml);
    }
    /* ORACLE_Q3_K */
    int j = k >> 4;
    int q = (((b[32 + 32 * half + l] >> (2 * r)) & 3) | (((b[l] >> sb) & 1) << 2)) - 4;
    int low = (j < 8) ? (b[96 + j] & 15) : (b[96 + j - 8] >> 4);
    int high = (b[104 + (j & 3)] >> (2 * (j >> 2))) & 3;
    float dl = half_to_f32(rd_u16(b + 108)) * (float)((low | (high << 4)) - 32);
    return dl * (float)q;
}

static int is_extra(int t)
{
    return t == ORACLE_Q5_0 || t == ORACLE_Q5_1 || (t >= ORACLE_Q2_K && t <= ORACLE_Q6_K);
}

/*
 * Decode `numel` elements of ggml type `ggml_type` from `src` into float32.
 * Returns 0, -1 for an unsupported type, -2 when src_bytes is shorter than
 * ceil(numel/32) blocks (the reference raises ValueError for Q4_0 at
 * gguf_loader.py:444-446; numpy raises for the others).
 */
int oracle_decode_f32(int ggml_type, const uint8_t *src, int64_t src_bytes,
                      int64_t numel, float *out, int n_threads)
{
    int64_t need = oracle_nbytes(ggml_type, numel);
    if (need < 0) return -1;
    if ((ggml_type & ORACLE_GGML_ORDER) && (ggml_type & ~ORACLE_GGML_ORDER) != ORACLE_Q4_0 &&
        (ggml_type & ~ORACLE_GGML_ORDER) != ORACLE_Q4_1) return -1;
    if (src_bytes < need) return -2;
    (void)n_threads;
#ifdef _OPENMP
    if (n_threads < 1) n_threads = 1;
#endif
    if (ggml_type == ORACLE_F32) {                 /* gguf_loader.py:407-410 */
        memcpy(out, src, (size_t)numel * 4);
        return 0;
    }
    if (ggml_type == ORACLE_F16) {                 /* gguf_loader.py:413-416 */
#pragma omp parallel for num_threads(n_threads) schedule(static)
        for (int64_t i = 0; i < numel; i++) out[i] = half_to_f32(rd_u16(src + 2 * i));
        return 0;
    }
    if (ggml_type == ORACLE_BF16) {                /* gguf_loader.py:419-427: u16 << 16 */
#pragma omp parallel for num_threads(n_threads) schedule(static)
        for (int64_t i = 0; i < numel; i++)
            out[i] = bits_to_f32((uint32_t)rd_u16(src + 2 * i) << 16);
        return 0;
    }
    if (is_extra(ggml_type)) {
        int be = block_elems(ggml_type), xb = block_bytes(ggml_type);
#pragma omp parallel for num_threads(n_threads) schedule(static)
        for (int64_t i = 0; i < numel; i++)
            out[i] = extra_element(ggml_type, src + (i / be) * xb, (int)(i % be));
        return 0;
    }
    int bb = block_bytes(ggml_type);
    int64_t n_blocks = (numel + 31) / 32;
#pragma omp parallel for num_threads(n_threads) schedule(static)
    for (int64_t blk = 0; blk < n_blocks; blk++) {
        float v[32];
        decode_block(ggml_type, src + blk * bb, v);
        int64_t base = blk * 32;
        int n = (numel - base) < 32 ? (int)(numel - base) : 32;   /* output[:numel] */
        memcpy(out + base, v, (size_t)n * 4);
    }
    return 0;
}

/* The `.to(dtype)` step of read_tensor (gguf_loader.py:378) for 16-bit targets. */
int oracle_cast(const float *in, int64_t n, int out_dtype, void *out, int n_threads)
{
    (void)n_threads;
#ifdef _OPENMP
    if (n_threads < 1) n_threads = 1;
#endif
    if (out_dtype == ORACLE_OUT_F32) { memcpy(out, in, (size_t)n * 4); return 0; }
    uint16_t *o = (uint16_t *)out;
    if (out_dtype == ORACLE_OUT_F16) {
#pragma omp parallel for num_threads(n_threads) schedule(static)
        for (int64_t i = 0; i < n; i++) o[i] = f32_to_half(in[i]);
        return 0;
    }
    if (out_dtype == ORACLE_OUT_BF16) {
#pragma omp parallel for num_threads(n_threads) schedule(static)
        for (int64_t i = 0; i < n; i++) o[i] = f32_to_bf16(in[i]);
        return 0;
    }
    return -1;
}

/* Widen a 16-bit result back to float32 (used for the double rounding that
 * param.copy_(tensor) performs when param.dtype != dtype, gguf_loader.py:758-759). */
int oracle_widen(const void *in, int64_t n, int in_dtype, float *out)
{
    const uint16_t *p = (const uint16_t *)in;
    if (in_dtype == ORACLE_OUT_F32) { memcpy(out, in, (size_t)n * 4); return 0; }
    if (in_dtype == ORACLE_OUT_F16) { for (int64_t i = 0; i < n; i++) out[i] = half_to_f32(p[i]); return 0; }
    if (in_dtype == ORACLE_OUT_BF16) { for (int64_t i = 0; i < n; i++) out[i] = bits_to_f32((uint32_t)p[i] << 16); return 0; }
    return -1;
}

/*
 * read_tensor's arithmetic in one call: decode to float32, then cast.
 * `scratch` must hold numel floats when out_dtype is 16-bit (may alias nothing).
 */
int oracle_read_tensor(int ggml_type, const uint8_t *src, int64_t src_bytes, int64_t numel,
                       int out_dtype, void *out, float *scratch, int n_threads)
{
    if (out_dtype == ORACLE_OUT_F32)
        return oracle_decode_f32(ggml_type, src, src_bytes, numel, (float *)out, n_threads);
    int rc = oracle_decode_f32(ggml_type, src, src_bytes, numel, scratch, n_threads);
    if (rc) return rc;
    return oracle_cast(scratch, numel, out_dtype, out, n_threads);
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
