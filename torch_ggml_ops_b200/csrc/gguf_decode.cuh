// Device-side decode of raw GGUF super-blocks (256 weights) to bf16, 32 weights at a time.
//
// The value produced for each weight is bf16_rne(w) with w the fp32 value the reference's
// decoder defines (reference: csrc/ck/gguf_decode.cuh:54-149; block field offsets
// csrc/vendor/llama_cpp/common.cuh:78-127).  Every product below is exact in fp32 (fp16
// super-scale x small integers), the only fp32 rounding is the Q4_K / Q5_K subtraction of the
// minimum, so the order of the exact operations is free and the result is bit-identical.
//
// A block is read from a shared-memory "window": the 16-byte-aligned span of global memory that
// covers it, copied verbatim.  Blocks of 110 / 210 / 82 bytes start on 2-byte boundaries only, so
// their fields are fetched as aligned 32-bit words and funnel-shifted into place.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tgo {

enum : int { QT_Q3_K = 11, QT_Q4_K = 12, QT_Q5_K = 13, QT_Q6_K = 14, QT_IQ2_S = 22 };

template <int QT> struct BlockFmt;
// kBytes: block size.  kAligned: every block starts 16-byte aligned.  kCopy: bytes that cover the
// block from the aligned address below its start.  kSlot: distance between block windows in shared
// memory: kCopy plus slack for the trailing funnel-shift word, and chosen so that the windows of
// consecutive rows start in different banks (a pitch of 128 bytes would put every row of a warp on
// the same bank).  kBox: bytes per window that the GEMM's TMA box loads copy (= kSlot: the box rows
// land back to back in shared memory, so the box width is the pitch).
template <> struct BlockFmt<QT_Q4_K> { static constexpr int kBytes = 144, kAligned = 1, kCopy = 144, kSlot = 144, kBox = 144; };
template <> struct BlockFmt<QT_Q5_K> { static constexpr int kBytes = 176, kAligned = 1, kCopy = 176, kSlot = 176, kBox = 176; };
template <> struct BlockFmt<QT_Q6_K> { static constexpr int kBytes = 210, kAligned = 0, kCopy = 224, kSlot = 240, kBox = 240; };
template <> struct BlockFmt<QT_Q3_K> { static constexpr int kBytes = 110, kAligned = 0, kCopy = 128, kSlot = 144, kBox = 144; };
template <> struct BlockFmt<QT_IQ2_S> { static constexpr int kBytes = 82, kAligned = 0, kCopy = 96, kSlot = 112, kBox = 112; };

__host__ __device__ constexpr int block_bytes_of(int qt) {
    return qt == QT_Q3_K ? 110 : qt == QT_Q4_K ? 144 : qt == QT_Q5_K ? 176 : qt == QT_Q6_K ? 210
         : qt == QT_IQ2_S ? 82 : -1;
}

// Shared-memory accesses by 32-bit shared-window address (one integer add per access instead of
// 64-bit generic pointer arithmetic).
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .u16 h; ld.shared.u16 h, [%1]; cvt.u32.u16 %0, h; }" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// N consecutive 32-bit words starting at a 2-byte-aligned shared-memory address.
template <int N>
__device__ __forceinline__ void ld_words(uint32_t a, uint32_t (&w)[N]) {
    const uint32_t base = a & ~3u;
    const uint32_t sh = (a & 2u) * 8u;
    uint32_t prev = lds32(base);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = lds32(base + 4 * (i + 1));
        w[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}
__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&r);
}

// 6-bit scale and minimum of 32-weight group g from the 12 packed bytes of Q4_K / Q5_K, given as
// three little-endian words (reference: csrc/ck/gguf_decode.cuh:13-31).
__device__ __forceinline__ void kquant_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int g,
                                                 int& sc, int& mn) {
    const int j = g & 3;
    const uint32_t a = (s0 >> (8 * j)) & 0xFFu;  // scales[j]
    const uint32_t b = (s1 >> (8 * j)) & 0xFFu;  // scales[4 + j]
    const uint32_t c = (s2 >> (8 * j)) & 0xFFu;  // scales[8 + j]
    if (g < 4) {
        sc = a & 63;
        mn = b & 63;
    } else {
        sc = (c & 15) | ((a >> 2) & 0x30);
        mn = (c >> 4) | ((b >> 2) & 0x30);
    }
}

// Byte b of v as the float 2^23 + byte (exact); the caller subtracts 2^23 (plus any offset).
__device__ __forceinline__ float byte_to_biased_float(uint32_t v, int b) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650u + b));
}
// Two weights at once with the packed fp32x2 instructions of sm_100 (each half is an ordinary
// IEEE fp32 operation, so results are bit-identical to the scalar formulas):
//   affine: (q - 0) * ds - mn as one fused multiply-add per half;  scaled: (q - off) * ds.
__device__ __forceinline__ uint32_t affine2(uint32_t v, int b0, int b1, float2 ds, float2 neg_mn) {
    const float2 f = make_float2(byte_to_biased_float(v, b0), byte_to_biased_float(v, b1));
    const float2 q = __fadd2_rn(f, make_float2(-8388608.0f, -8388608.0f));
    const float2 w = __ffma2_rn(ds, q, neg_mn);
    return pack_bf16(w.x, w.y);
}
__device__ __forceinline__ uint32_t scaled2(uint32_t v, int b0, int b1, float2 ds, float2 neg_bias) {
    const float2 f = make_float2(byte_to_biased_float(v, b0), byte_to_biased_float(v, b1));
    const float2 q = __fadd2_rn(f, neg_bias);
    const float2 w = __fmul2_rn(ds, q);
    return pack_bf16(w.x, w.y);
}
// Eight weights from two words of byte-sized quants: w = ds * q - mn.
__device__ __forceinline__ uint4 affine8(uint32_t v0, uint32_t v1, float ds, float mn) {
    const float2 ds2 = make_float2(ds, ds), nm2 = make_float2(-mn, -mn);
    uint4 o;
    o.x = affine2(v0, 0, 1, ds2, nm2);
    o.y = affine2(v0, 2, 3, ds2, nm2);
    o.z = affine2(v1, 0, 1, ds2, nm2);
    o.w = affine2(v1, 2, 3, ds2, nm2);
    return o;
}
// Eight weights from two words of byte-sized quants with an integer offset: w = ds * (q - off).
__device__ __forceinline__ uint4 scaled8(uint32_t v0, uint32_t v1, float ds, float off) {
    const float2 ds2 = make_float2(ds, ds), nb2 = make_float2(-8388608.0f - off, -8388608.0f - off);
    uint4 o;
    o.x = scaled2(v0, 0, 1, ds2, nb2);
    o.y = scaled2(v0, 2, 3, ds2, nb2);
    o.z = scaled2(v1, 0, 1, ds2, nb2);
    o.w = scaled2(v1, 2, 3, ds2, nb2);
    return o;
}

// decode32<QT>: weights 32g .. 32g+31 of the block at shared-memory address `blk`, as four
// 16-byte chunks of 8 bf16 each.  `grid` is the shared-memory address of the IQ2_S codebook
// (unused otherwise).
template <int QT>
__device__ __forceinline__ void decode32(uint32_t blk, int g, uint32_t grid, uint4 (&out)[4]);

template <>
__device__ __forceinline__ void decode32<QT_Q4_K>(uint32_t blk, int g, uint32_t, uint4 (&out)[4]) {
    const uint4 head = lds128(blk);  // d, dmin, scales[12]
    int sc, mn;
    kquant_scale_min(head.y, head.z, head.w, g, sc, mn);
    const float ds = half_bits_to_float(head.x & 0xFFFFu) * static_cast<float>(sc);
    const float dm = half_bits_to_float(head.x >> 16) * static_cast<float>(mn);
    const uint32_t qs = blk + 16 + (g >> 1) * 32;
    const uint4 a = lds128(qs), b = lds128(qs + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const int sh = 4 * (g & 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t v0 = (w[2 * c] >> sh) & 0x0F0F0F0Fu;
        const uint32_t v1 = (w[2 * c + 1] >> sh) & 0x0F0F0F0Fu;
        out[c] = affine8(v0, v1, ds, dm);
    }
}

template <>
__device__ __forceinline__ void decode32<QT_Q5_K>(uint32_t blk, int g, uint32_t, uint4 (&out)[4]) {
    const uint4 head = lds128(blk);
    int sc, mn;
    kquant_scale_min(head.y, head.z, head.w, g, sc, mn);
    const float ds = half_bits_to_float(head.x & 0xFFFFu) * static_cast<float>(sc);
    const float dm = half_bits_to_float(head.x >> 16) * static_cast<float>(mn);
    const uint4 ha = lds128(blk + 16), hb = lds128(blk + 32);
    const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
    const uint32_t qs = blk + 48 + (g >> 1) * 32;
    const uint4 a = lds128(qs), b = lds128(qs + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const int sh = 4 * (g & 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t v0 = ((w[2 * c] >> sh) & 0x0F0F0F0Fu) | (((h[2 * c] >> g) & 0x01010101u) << 4);
        const uint32_t v1 =
            ((w[2 * c + 1] >> sh) & 0x0F0F0F0Fu) | (((h[2 * c + 1] >> g) & 0x01010101u) << 4);
        out[c] = affine8(v0, v1, ds, dm);
    }
}

template <>
__device__ __forceinline__ void decode32<QT_Q6_K>(uint32_t blk, int g, uint32_t, uint4 (&out)[4]) {
    // weights i = 32g + j: chunk c = g>>2 of 128; ql byte c*64 + (g&1)*32 + j, nibble (g&3)>>1;
    // qh byte c*32 + j, bit pair g&3; one int8 scale per 16 weights.
    const int c128 = g >> 2;
    uint32_t ql[8], qh[8];
    ld_words<8>(blk + c128 * 64 + (g & 1) * 32, ql);
    ld_words<8>(blk + 128 + c128 * 32, qh);
    const uint32_t sc2 = lds16(blk + 192 + 2 * g);
    const float d = half_bits_to_float(lds16(blk + 208));
    const float ds0 = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(sc2 & 0xFFu)));
    const float ds1 = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(sc2 >> 8)));
    const int sl = 4 * ((g & 3) >> 1);
    const int shh = 2 * (g & 3);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t v0 = ((ql[2 * c] >> sl) & 0x0F0F0F0Fu) | (((qh[2 * c] >> shh) & 0x03030303u) << 4);
        const uint32_t v1 =
            ((ql[2 * c + 1] >> sl) & 0x0F0F0F0Fu) | (((qh[2 * c + 1] >> shh) & 0x03030303u) << 4);
        out[c] = scaled8(v0, v1, c < 2 ? ds0 : ds1, 32.0f);
    }
}

template <>
__device__ __forceinline__ void decode32<QT_Q3_K>(uint32_t blk, int g, uint32_t, uint4 (&out)[4]) {
    // weights i = 32g + j: low 2 bits qs[(g>>2)*32 + j] >> 2*(g&3); hmask[j] bit g set means
    // "do not subtract 4"; 6-bit scale (minus 32) per 16 weights.
    uint32_t hm[8], qs[8], s[3];
    ld_words<8>(blk, hm);
    ld_words<8>(blk + 32 + (g >> 2) * 32, qs);
    ld_words<3>(blk + 96, s);
    const float d = half_bits_to_float(lds16(blk + 108));
    float ds[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int sg = 2 * g + t;  // 16-weight group 0..15
        const int k = sg & 7;
        const uint32_t lsb = ((k < 4 ? s[0] : s[1]) >> (8 * (k & 3))) & 0xFFu;  // scales[sg & 7]
        const uint32_t ls = sg < 8 ? lsb : (lsb >> 4);
        const uint32_t hs = ((s[2] >> (8 * (sg & 3))) & 0xFFu) >> (2 * (sg >> 2));
        const int scale = static_cast<int>((ls & 15u) | ((hs & 3u) << 4)) - 32;
        ds[t] = d * static_cast<float>(scale);
    }
    const int sq = 2 * (g & 3);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t v0 = ((qs[2 * c] >> sq) & 0x03030303u) | (((hm[2 * c] >> g) & 0x01010101u) << 2);
        const uint32_t v1 =
            ((qs[2 * c + 1] >> sq) & 0x03030303u) | (((hm[2 * c + 1] >> g) & 0x01010101u) << 2);
        out[c] = scaled8(v0, v1, c < 2 ? ds[0] : ds[1], 4.0f);
    }
}

template <>
__device__ __forceinline__ void decode32<QT_IQ2_S>(uint32_t blk, int g, uint32_t grid, uint4 (&out)[4]) {
    // weights 32g..32g+31 = codebook groups 4g..4g+3 of 8 weights: index qs[gg] | 2 bits of
    // qh[g] << 8, sign byte qs[32 + gg]; one 4-bit scale per 16 weights in scales[g].
    uint32_t idxw[1], sgnw[1];
    ld_words<1>(blk + 2 + 4 * g, idxw);
    ld_words<1>(blk + 34 + 4 * g, sgnw);
    const uint32_t qh = lds8(blk + 66 + g);
    const uint32_t scb = lds8(blk + 74 + g);
    const float d = half_bits_to_float(lds16(blk));
    const float db0 = (d * (0.5f + static_cast<float>(scb & 15u))) * 0.25f;
    const float db1 = (d * (0.5f + static_cast<float>(scb >> 4))) * 0.25f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t idx = ((idxw[0] >> (8 * c)) & 0xFFu) | (((qh >> (2 * c)) & 3u) << 8);
        const uint2 mags = lds64(grid + idx * 8);
        const uint32_t m0 = mags.x, m1 = mags.y;
        const uint32_t sg = (sgnw[0] >> (8 * c)) & 0xFFu;
        const float db = c < 2 ? db0 : db1;
        const uint32_t dbb = __float_as_uint(db);
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            const uint32_t mw = e < 4 ? m0 : m1;
            const float2 f = make_float2(byte_to_biased_float(mw, e & 3), byte_to_biased_float(mw, (e & 3) + 1));
            const float2 mag = __fadd2_rn(f, make_float2(-8388608.0f, -8388608.0f));
            // +-db per weight: the sign bit of the sign byte moved onto the float's sign
            const float2 sdb = make_float2(__uint_as_float(dbb ^ ((sg << (31 - e)) & 0x80000000u)),
                                           __uint_as_float(dbb ^ ((sg << (30 - e)) & 0x80000000u)));
            const float2 w = __fmul2_rn(sdb, mag);
            o[e >> 1] = pack_bf16(w.x, w.y);
        }
        out[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// decode64: weights 64s .. 64s+63 of a Q4_K / Q5_K block in one pass over the raw bytes they share
// (one header load and one load of the 32 quant bytes instead of two of each): the first 32 come
// back decoded, the last 32 as byte-sized quants with their scale and minimum, to be finished by
// finish32 when the caller has room for them.  Same arithmetic as decode32, so the same bits.
struct Pending32 {
    uint32_t v[8];
    float ds, dm;
};
__device__ __forceinline__ void finish32(const Pending32& p, uint4 (&out)[4]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) out[c] = affine8(p.v[2 * c], p.v[2 * c + 1], p.ds, p.dm);
}
template <int QT>
__device__ __forceinline__ void decode64(uint32_t blk, int s, uint4 (&out)[4], Pending32& p);

template <>
__device__ __forceinline__ void decode64<QT_Q4_K>(uint32_t blk, int s, uint4 (&out)[4], Pending32& p) {
    const uint4 head = lds128(blk);
    int sc0, mn0, sc1, mn1;
    kquant_scale_min(head.y, head.z, head.w, 2 * s, sc0, mn0);
    kquant_scale_min(head.y, head.z, head.w, 2 * s + 1, sc1, mn1);
    const float d = half_bits_to_float(head.x & 0xFFFFu), dmin = half_bits_to_float(head.x >> 16);
    const float ds0 = d * static_cast<float>(sc0), dm0 = dmin * static_cast<float>(mn0);
    p.ds = d * static_cast<float>(sc1);
    p.dm = dmin * static_cast<float>(mn1);
    const uint32_t qs = blk + 16 + s * 32;
    const uint4 a = lds128(qs), b = lds128(qs + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) p.v[i] = (w[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int c = 0; c < 4; ++c) out[c] = affine8(w[2 * c] & 0x0F0F0F0Fu, w[2 * c + 1] & 0x0F0F0F0Fu, ds0, dm0);
}

template <>
__device__ __forceinline__ void decode64<QT_Q5_K>(uint32_t blk, int s, uint4 (&out)[4], Pending32& p) {
    const uint4 head = lds128(blk);
    int sc0, mn0, sc1, mn1;
    kquant_scale_min(head.y, head.z, head.w, 2 * s, sc0, mn0);
    kquant_scale_min(head.y, head.z, head.w, 2 * s + 1, sc1, mn1);
    const float d = half_bits_to_float(head.x & 0xFFFFu), dmin = half_bits_to_float(head.x >> 16);
    const float ds0 = d * static_cast<float>(sc0), dm0 = dmin * static_cast<float>(mn0);
    p.ds = d * static_cast<float>(sc1);
    p.dm = dmin * static_cast<float>(mn1);
    const uint4 ha = lds128(blk + 16), hb = lds128(blk + 32);
    const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
    const uint32_t qs = blk + 48 + s * 32;
    const uint4 a = lds128(qs), b = lds128(qs + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    const int g = 2 * s;
#pragma unroll
    for (int i = 0; i < 8; ++i) p.v[i] = ((w[i] >> 4) & 0x0F0F0F0Fu) | (((h[i] >> (g + 1)) & 0x01010101u) << 4);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t v0 = (w[2 * c] & 0x0F0F0F0Fu) | (((h[2 * c] >> g) & 0x01010101u) << 4);
        const uint32_t v1 = (w[2 * c + 1] & 0x0F0F0F0Fu) | (((h[2 * c + 1] >> g) & 0x01010101u) << 4);
        out[c] = affine8(v0, v1, ds0, dm0);
    }
}

}  // namespace tgo
