// Block formats the reference names (src/phfe/inference/gguf_loader.py:37-46) but cannot
// decode: Q5_0, Q5_1 and the 256-element K-quants Q2_K, Q3_K, Q4_K, Q5_K, Q6_K.  The
// arithmetic restates ggml's published dequantize_row_* routines; element order is ggml's.
// Every product that is formed before the final operation is exact in fp32 (an fp16 scale
// times a 4..8-bit integer, times another small integer), so each output is one IEEE
// rounding of the exact value and does not depend on how a compiler contracts the C code:
//   Q5_0  y = (q5 - 16) * d                       Q5_1  y = q5 * d + m
//   Q2_K  y = (d * sc4) * q2 - (dmin * m4)        Q3_K  y = (d * (sc6 - 32)) * (q3 - 4)
//   Q4_K  y = (d * sc6) * q4 - (dmin * m6)        Q5_K  y = (d * sc6) * q5 - (dmin * m6)
//   Q6_K  y = (d * sc8) * (q6 - 32)
// Included by dequant_kernels.cuh; relies on its helpers (ld16, half_bits_to_f32, pack2 ...).
#pragma once

namespace pfhe {

enum : int { T_Q5_0 = 6, T_Q5_1 = 7, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14 };

template <> struct Fmt<T_Q5_0> { static constexpr int kElems = 32,  kBytes = 22;  };
template <> struct Fmt<T_Q5_1> { static constexpr int kElems = 32,  kBytes = 24;  };
template <> struct Fmt<T_Q2_K> { static constexpr int kElems = 256, kBytes = 84;  };
template <> struct Fmt<T_Q3_K> { static constexpr int kElems = 256, kBytes = 110; };
template <> struct Fmt<T_Q4_K> { static constexpr int kElems = 256, kBytes = 144; };
template <> struct Fmt<T_Q5_K> { static constexpr int kElems = 256, kBytes = 176; };
template <> struct Fmt<T_Q6_K> { static constexpr int kElems = 256, kBytes = 210; };

template <int T> struct IsExtra { static constexpr bool value = (T == T_Q5_0 || T == T_Q5_1 || T == T_Q2_K || T == T_Q3_K ||
                                                                T == T_Q4_K || T == T_Q5_K || T == T_Q6_K); };

// What the quantised integer is offset by before scaling, and whether a minimum is subtracted / added.
template <int T> struct ExtraTraits;
template <> struct ExtraTraits<T_Q5_0> { static constexpr float kBias = 16.0f; static constexpr int kMin = 0; };
template <> struct ExtraTraits<T_Q5_1> { static constexpr float kBias = 0.0f;  static constexpr int kMin = +1; };  // + m
template <> struct ExtraTraits<T_Q2_K> { static constexpr float kBias = 0.0f;  static constexpr int kMin = -1; };  // - ml
template <> struct ExtraTraits<T_Q3_K> { static constexpr float kBias = 4.0f;  static constexpr int kMin = 0; };
template <> struct ExtraTraits<T_Q4_K> { static constexpr float kBias = 0.0f;  static constexpr int kMin = -1; };
template <> struct ExtraTraits<T_Q5_K> { static constexpr float kBias = 0.0f;  static constexpr int kMin = -1; };
template <> struct ExtraTraits<T_Q6_K> { static constexpr float kBias = 32.0f; static constexpr int kMin = 0; };

// Formats whose per-group multiplier is costly to unpack get it computed once per tile into a
// shared-memory table (kGroups entries per block) instead of once per 16-byte unit.
template <int T> struct ScaleTable { static constexpr int kGroups = 0; };
template <> struct ScaleTable<T_Q4_K> { static constexpr int kGroups = 8; };
template <> struct ScaleTable<T_Q5_K> { static constexpr int kGroups = 8; };
// (measured: it lifts Q4_K / Q5_K -> 16-bit from 0.80 / 0.77 to 0.93 / 0.88 of the copy peak, but costs
// Q2_K / Q3_K, whose 16 groups per block make the table pass dearer than the inline unpack.)

__device__ __forceinline__ uint32_t ld8(const uint8_t *p) { return *p; }

// Bits 0..3 of x moved to bit 0 of bytes 0..3 (the partial products land on distinct bits, so nothing carries).
__device__ __forceinline__ uint32_t spread4(uint32_t x) { return ((x & 0xFu) * 0x00204081u) & 0x01010101u; }

// Scale and minimum of sub-block j (0..7) from the 12 packed bytes of Q4_K / Q5_K.
__device__ __forceinline__ void k4_scale_min(const uint8_t *s, int j, uint32_t *sc, uint32_t *mn)
{
    if (j < 4) {
        *sc = ld8(s + j) & 63u;
        *mn = ld8(s + j + 4) & 63u;
    } else {
        const uint32_t hi = ld8(s + j + 4);
        *sc = (hi & 0xFu) | ((ld8(s + j - 4) >> 6) << 4);
        *mn = (hi >> 4) | ((ld8(s + j) >> 6) << 4);
    }
}

// The per-(sub-)block multiplier `dl` and offset `ml` that apply to element e0 (and the elements
// that share its 16- or 32-element group) of a block.
template <int T> __device__ __forceinline__ void extra_scales(const uint8_t *blk, int e0, float *dl, float *ml)
{
    *ml = 0.0f;
    if constexpr (T == T_Q5_0) {
        *dl = half_bits_to_f32(ld16<true>(blk));
    } else if constexpr (T == T_Q5_1) {
        *dl = half_bits_to_f32(ld16<true>(blk));
        *ml = half_bits_to_f32(ld16<true>(blk + 2));
    } else if constexpr (T == T_Q4_K || T == T_Q5_K) {
        uint32_t sc, mn;
        k4_scale_min(blk + 4, e0 >> 5, &sc, &mn);
        *dl = __fmul_rn(half_bits_to_f32(ld16<true>(blk)), (float)sc);
        *ml = __fmul_rn(half_bits_to_f32(ld16<true>(blk + 2)), (float)mn);
    } else if constexpr (T == T_Q6_K) {
        const int sc = (int)(int8_t)ld8(blk + 192 + (e0 >> 4));
        *dl = __fmul_rn(half_bits_to_f32(ld16<true>(blk + 208)), (float)sc);
    } else if constexpr (T == T_Q2_K) {
        const uint32_t s = ld8(blk + (e0 >> 4));
        *dl = __fmul_rn(half_bits_to_f32(ld16<true>(blk + 80)), (float)(s & 0xFu));
        *ml = __fmul_rn(half_bits_to_f32(ld16<true>(blk + 82)), (float)(s >> 4));
    } else {  // T_Q3_K
        const int j = e0 >> 4;
        const uint32_t low = (j < 8) ? (ld8(blk + 96 + j) & 0xFu) : (ld8(blk + 96 + j - 8) >> 4);
        const uint32_t high = (ld8(blk + 104 + (j & 3)) >> (2 * (j >> 2))) & 3u;
        *dl = __fmul_rn(half_bits_to_f32(ld16<true>(blk + 108)), (float)((int)(low | (high << 4)) - 32));
    }
}

// N (4 or 8) consecutive quantised integers starting at element e0 of a block, one per byte of
// w[0] (and w[1]); unsigned, before the bias of ExtraTraits is taken off.  e0 is a multiple of N.
template <int T, int N> __device__ __forceinline__ void extra_quants(const uint8_t *blk, int e0, uint32_t *w)
{
    auto load_n = [&](const uint8_t *p, uint32_t *out) {          // N bytes from a 2-byte aligned address
        out[0] = ld16<true>(p) | (ld16<true>(p + 2) << 16);
        if constexpr (N == 8) out[1] = ld16<true>(p + 4) | (ld16<true>(p + 6) << 16);
    };
    constexpr int W = N / 4;
    if constexpr (T == T_Q5_0 || T == T_Q5_1) {
        constexpr int kQh = (T == T_Q5_0) ? 2 : 4;
        const uint32_t qh = ld16<true>(blk + kQh) | (ld16<true>(blk + kQh + 2) << 16);
        uint32_t raw[2];
        load_n(blk + kQh + 4 + (e0 & 15), raw);
        const uint32_t sh = (e0 >> 4) * 4;                         // elements 16..31 use the high nibbles
        const uint32_t bits = qh >> e0;                            // element e <-> bit e
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = ((raw[i] >> sh) & 0x0F0F0F0Fu) | (spread4(bits >> (4 * i)) << 4);
    } else if constexpr (T == T_Q4_K || T == T_Q5_K) {
        const int sb = e0 >> 5, l0 = e0 & 31;
        constexpr int kQs = (T == T_Q4_K) ? 16 : 48;
        uint32_t raw[2];
        load_n(blk + kQs + 32 * (sb >> 1) + l0, raw);
        const uint32_t sh = (sb & 1) * 4;
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = (raw[i] >> sh) & 0x0F0F0F0Fu;
        if constexpr (T == T_Q5_K) {
            uint32_t hb[2];
            load_n(blk + 16 + l0, hb);
#pragma unroll
            for (int i = 0; i < W; ++i) w[i] |= ((hb[i] >> sb) & 0x01010101u) << 4;
        }
    } else if constexpr (T == T_Q6_K) {
        const int g = e0 >> 5, l0 = e0 & 31, half = g >> 2, r = g & 3;
        uint32_t lo[2], hi[2];
        load_n(blk + 64 * half + 32 * (r & 1) + l0, lo);
        load_n(blk + 128 + 32 * half + l0, hi);
        const uint32_t sh = (r >> 1) * 4;
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = ((lo[i] >> sh) & 0x0F0F0F0Fu) | (((hi[i] >> (2 * r)) & 0x03030303u) << 4);
    } else if constexpr (T == T_Q2_K) {
        const int half = e0 >> 7, r = (e0 >> 5) & 3, l0 = e0 & 31;
        uint32_t raw[2];
        load_n(blk + 16 + 32 * half + l0, raw);
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = (raw[i] >> (2 * r)) & 0x03030303u;
    } else {  // T_Q3_K
        const int half = e0 >> 7, r = (e0 >> 5) & 3, l0 = e0 & 31;
        uint32_t raw[2], hm[2];
        load_n(blk + 32 + 32 * half + l0, raw);
        load_n(blk + l0, hm);
        const uint32_t hbit = e0 >> 5;                             // 0..7
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = ((raw[i] >> (2 * r)) & 0x03030303u) | (((hm[i] >> hbit) & 0x01010101u) << 2);
    }
}

template <int T> __device__ __forceinline__ float extra_finish(float q_plus_magic, float dl, float ml)
{
    const float q = __fsub_rn(q_plus_magic, 8388608.0f + ExtraTraits<T>::kBias);   // exact
    if constexpr (ExtraTraits<T>::kMin < 0) return __fmaf_rn(dl, q, -ml);          // one rounding of dl*q - ml
    else if constexpr (ExtraTraits<T>::kMin > 0) return __fmaf_rn(dl, q, ml);
    else return __fmul_rn(dl, q);
}

// Sixteen output bytes of an extra-format tensor: unit c of its block (VEC = 8 or 4 outputs),
// with the group's multiplier and offset already known.
template <int T, int MID, int OUT>
__device__ __forceinline__ uint4 extra_unit_scaled(const uint8_t *blk, int c, float dl, float ml)
{
    constexpr int VEC = 16 / OutT<OUT>::kSize;
    const int e0 = c * VEC;
    uint32_t w[2];
    extra_quants<T, VEC>(blk, e0, w);
    uint4 r;
    if constexpr (OUT == O_F32) {
        r.x = __float_as_uint(round_via<MID>(extra_finish<T>(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7540)), dl, ml)));
        r.y = __float_as_uint(round_via<MID>(extra_finish<T>(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7541)), dl, ml)));
        r.z = __float_as_uint(round_via<MID>(extra_finish<T>(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7542)), dl, ml)));
        r.w = __float_as_uint(round_via<MID>(extra_finish<T>(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7543)), dl, ml)));
    } else {
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = extra_finish<T>(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7540 + i)), dl, ml);
            v[4 + i] = extra_finish<T>(__uint_as_float(__byte_perm(w[1], 0x4B000000u, 0x7540 + i)), dl, ml);
        }
        r.x = pack2<MID, OUT>(v[0], v[1]); r.y = pack2<MID, OUT>(v[2], v[3]);
        r.z = pack2<MID, OUT>(v[4], v[5]); r.w = pack2<MID, OUT>(v[6], v[7]);
    }
    return r;
}

template <int T, int MID, int OUT>
__device__ __forceinline__ uint4 extra_unit(const uint8_t *blk, int c)
{
    float dl, ml;
    extra_scales<T>(blk, c * (16 / OutT<OUT>::kSize), &dl, &ml);
    return extra_unit_scaled<T, MID, OUT>(blk, c, dl, ml);
}

// One element (index k inside its block), byte reads only: the fallback path and ragged tails.
template <int T> __device__ __forceinline__ float extra_element(const uint8_t *b, int k)
{
    auto h16 = [&](int off) { return half_bits_to_f32((uint32_t)b[off] | ((uint32_t)b[off + 1] << 8)); };
    int q;
    float dl, ml = 0.0f;
    if constexpr (T == T_Q5_0 || T == T_Q5_1) {
        constexpr int kQh = (T == T_Q5_0) ? 2 : 4;
        const uint32_t qh = (uint32_t)b[kQh] | ((uint32_t)b[kQh + 1] << 8) | ((uint32_t)b[kQh + 2] << 16) | ((uint32_t)b[kQh + 3] << 24);
        const uint32_t byte = b[kQh + 4 + (k & 15)];
        q = (int)(((k & 16) ? (byte >> 4) : (byte & 15)) | (((qh >> k) & 1u) << 4));
        dl = h16(0);
        if constexpr (T == T_Q5_1) ml = h16(2);
    } else if constexpr (T == T_Q4_K || T == T_Q5_K) {
        const int sb = k >> 5, l = k & 31;
        constexpr int kQs = (T == T_Q4_K) ? 16 : 48;
        const uint8_t *s = b + 4;
        uint32_t sc, mn;
        if (sb < 4) { sc = s[sb] & 63u; mn = s[sb + 4] & 63u; }
        else { sc = (s[sb + 4] & 0xFu) | ((uint32_t)(s[sb - 4] >> 6) << 4); mn = (s[sb + 4] >> 4) | ((uint32_t)(s[sb] >> 6) << 4); }
        const uint32_t byte = b[kQs + 32 * (sb >> 1) + l];
        q = (int)((sb & 1) ? (byte >> 4) : (byte & 15));
        if constexpr (T == T_Q5_K) q |= (int)(((b[16 + l] >> sb) & 1u) << 4);
        dl = __fmul_rn(h16(0), (float)sc);
        ml = __fmul_rn(h16(2), (float)mn);
    } else if constexpr (T == T_Q6_K) {
        const int g = k >> 5, l = k & 31, half = g >> 2, r = g & 3;
        const uint32_t lo = b[64 * half + 32 * (r & 1) + l];
        const uint32_t hi = b[128 + 32 * half + l];
        q = (int)((((r >> 1) ? (lo >> 4) : (lo & 15))) | (((hi >> (2 * r)) & 3u) << 4));
        dl = __fmul_rn(h16(208), (float)(int)(int8_t)b[192 + (k >> 4)]);
    } else if constexpr (T == T_Q2_K) {
        const int half = k >> 7, r = (k >> 5) & 3, l = k & 31;
        q = (int)((b[16 + 32 * half + l] >> (2 * r)) & 3u);
        const uint32_t s = b[k >> 4];
        dl = __fmul_rn(h16(80), (float)(s & 0xFu));
        ml = __fmul_rn(h16(82), (float)(s >> 4));
    } else {  // T_Q3_K
        const int half = k >> 7, r = (k >> 5) & 3, l = k & 31, j = k >> 4;
        q = (int)(((b[32 + 32 * half + l] >> (2 * r)) & 3u) | (((b[l] >> (k >> 5)) & 1u) << 2));
        const uint32_t low = (j < 8) ? (b[96 + j] & 0xFu) : (b[96 + j - 8] >> 4);
        const uint32_t high = (b[104 + (j & 3)] >> (2 * (j >> 2))) & 3u;
        dl = __fmul_rn(h16(108), (float)((int)(low | (high << 4)) - 32));
    }
    const float qf = (float)(q - (int)ExtraTraits<T>::kBias);
    if constexpr (ExtraTraits<T>::kMin < 0) return __fmaf_rn(dl, qf, -ml);
    else if constexpr (ExtraTraits<T>::kMin > 0) return __fmaf_rn(dl, qf, ml);
    else return __fmul_rn(dl, qf);
}

}  // namespace pfhe
