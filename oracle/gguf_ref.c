/*
 * CPU oracle: scalar restatement of the reference's GGUF super-block decode.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product path may link, import or
 * call this file; it exists so that tests, the smoke check and the CPU leg of
 * the benchmark have an independent statement of the arithmetic.
 *
 * Follows, value for value, the reference's project-owned decoder
 *   csrc/ck/gguf_decode.cuh:13-31   (6-bit scale / min unpack for Q4_K, Q5_K)
 *   csrc/ck/gguf_decode.cuh:55-80   (Q3_K)
 *   csrc/ck/gguf_decode.cuh:83-94   (Q4_K)
 *   csrc/ck/gguf_decode.cuh:97-110  (Q5_K)
 *   csrc/ck/gguf_decode.cuh:113-128 (Q6_K)
 *   csrc/ck/gguf_decode.cuh:131-149 (IQ2_S)
 * with the block field offsets of csrc/vendor/llama_cpp/common.cuh:78-127.
 * All arithmetic is fp32, one operation at a time (no contraction that could
 * change a result: every product here is exact in fp32, only the Q4_K/Q5_K
 * subtraction rounds).
 *
 * Pinning: checked bit-for-bit against gguf-py 0.19.0 (gguf.quants.dequantize)
 * and against the committed golden vectors in tests/golden/.  The reference's
 * own test oracle (a function of an un-pinned transformers fork) and its GGUF
 * checkpoint are not available, so parity with *that* boundary is unpinned.
 *
 * The IQ2_S codebook is not stored here: the caller passes the 1024-entry
 * table (taken at run time from the installed gguf package, hash-checked).
 */
#include <stdint.h>
#include <string.h>

enum { QT_Q3_K = 11, QT_Q4_K = 12, QT_Q5_K = 13, QT_Q6_K = 14, QT_IQ2_S = 22 };

static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t load_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

int64_t tgo_ref_block_bytes(int qtype) {
    switch (qtype) {
        case QT_Q3_K: return 110;
        case QT_Q4_K: return 144;
        case QT_Q5_K: return 176;
        case QT_Q6_K: return 210;
        case QT_IQ2_S: return 82;
        default: return -1;
    }
}

/* gguf_decode.cuh:13-31 */
static int kq_scale(const uint8_t *sc, int g) {
    if (g < 4) return sc[g] & 63;
    return (sc[8 + g - 4] & 15) | ((sc[g - 4] >> 2) & 0x30);
}
static int kq_min(const uint8_t *sc, int g) {
    if (g < 4) return sc[4 + g] & 63;
    return (sc[8 + g - 4] >> 4) | ((sc[4 + g - 4] >> 2) & 0x30);
}

static void dq_q4k(const uint8_t *b, float *out) {
    const float d = half_to_float(load_u16(b)), dmin = half_to_float(load_u16(b + 2));
    const uint8_t *sc = b + 4, *qs = b + 16;
    for (int i = 0; i < 256; ++i) {
        const int g = i >> 5;
        const int q = (qs[(g >> 1) * 32 + (i & 31)] >> (4 * (g & 1))) & 15;
        const float ds = d * (float)kq_scale(sc, g);
        const float mn = dmin * (float)kq_min(sc, g);
        const float prod = ds * (float)q;
        out[i] = prod - mn;
    }
}

static void dq_q5k(const uint8_t *b, float *out) {
    const float d = half_to_float(load_u16(b)), dmin = half_to_float(load_u16(b + 2));
    const uint8_t *sc = b + 4, *qh = b + 16, *qs = b + 48;
    for (int i = 0; i < 256; ++i) {
        const int g = i >> 5;
        const int lo = (qs[(g >> 1) * 32 + (i & 31)] >> (4 * (g & 1))) & 15;
        const int hi = (qh[i & 31] >> g) & 1;
        const int q = lo | (hi << 4);
        const float ds = d * (float)kq_scale(sc, g);
        const float mn = dmin * (float)kq_min(sc, g);
        const float prod = ds * (float)q;
        out[i] = prod - mn;
    }
}

static void dq_q6k(const uint8_t *b, float *out) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    const float d = half_to_float(load_u16(b + 208));
    for (int i = 0; i < 256; ++i) {
        const int c = i >> 7, r = i & 127;
        const int lo = (ql[c * 64 + (r & 63)] >> (4 * (r >> 6))) & 15;
        const int hi = (qh[c * 32 + (i & 31)] >> (2 * ((r >> 5) & 3))) & 3;
        const int q = (lo | (hi << 4)) - 32;
        const float ds = d * (float)sc[i >> 4];
        out[i] = ds * (float)q;
    }
}

static void dq_q3k(const uint8_t *b, float *out) {
    const uint8_t *hm = b, *qs = b + 32, *sc = b + 96;
    const float d = half_to_float(load_u16(b + 108));
    for (int i = 0; i < 256; ++i) {
        const int sg = i >> 4;
        const int ls = sg < 8 ? sc[sg] : (sc[sg - 8] >> 4);
        const int hs = sc[8 + (sg & 3)] >> (2 * (sg >> 2));
        const int scale = ((ls & 15) | ((hs & 3) << 4)) - 32;
        const int low = (qs[(i >> 7) * 32 + (i & 31)] >> (2 * ((i & 127) >> 5))) & 3;
        const int high = ((hm[i & 31] >> (i >> 5)) & 1) ^ 1;
        const int q = low - (high << 2);
        const float ds = d * (float)scale;
        out[i] = ds * (float)q;
    }
}

static void dq_iq2s(const uint8_t *b, const uint64_t *grid, float *out) {
    const float d = half_to_float(load_u16(b));
    const uint8_t *qs = b + 2, *qh = b + 66, *sc = b + 74;
    for (int i = 0; i < 256; ++i) {
        const int gg = i >> 3, ge = i & 7;
        const int high = (qh[gg >> 2] >> (2 * (gg & 3))) & 3;
        const int idx = qs[gg] | (high << 8);
        const int mag = (int)((grid[idx] >> (8 * ge)) & 255);
        const int sign = ((qs[32 + gg] >> ge) & 1) ? -1 : 1;
        const int sg = i >> 4;
        const int s = (sc[sg >> 1] >> (4 * (sg & 1))) & 15;
        const float dd = d * (0.5f + (float)s);
        const float db = dd * 0.25f;
        out[i] = db * (float)(mag * sign);
    }
}

/* Decode n_blocks consecutive super-blocks into n_blocks*256 floats.
 * grid may be NULL unless qtype == IQ2_S.  Returns 0, or -1 on a bad type. */
int tgo_ref_dequantize(const uint8_t *packed, int64_t n_blocks, int qtype,
                       const uint64_t *grid, float *out) {
    const int64_t bb = tgo_ref_block_bytes(qtype);
    if (bb < 0) return -1;
    if (qtype == QT_IQ2_S && grid == 0) return -2;
    for (int64_t i = 0; i < n_blocks; ++i) {
        const uint8_t *b = packed + i * bb;
        float *o = out + i * 256;
        switch (qtype) {
            case QT_Q3_K: dq_q3k(b, o); break;
            case QT_Q4_K: dq_q4k(b, o); break;
            case QT_Q5_K: dq_q5k(b, o); break;
            case QT_Q6_K: dq_q6k(b, o); break;
            default: dq_iq2s(b, grid, o); break;
        }
    }
    return 0;
}

/* fp32 -> bf16 bits, round to nearest even (what __float2bfloat16 does; the
 * reference's backward stores this: csrc/ck/mmq_backward.cuh:44). */
void tgo_ref_round_bf16(const float *in, int64_t n, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        uint32_t x;
        memcpy(&x, in + i, 4);
        if ((x & 0x7fffffffu) > 0x7f800000u) {
            out[i] = (uint16_t)((x >> 16) | 0x40u);
        } else {
            x += 0x7fffu + ((x >> 16) & 1u);
            out[i] = (uint16_t)(x >> 16);
        }
    }
}
