/* CPU restatement of the reference's host reading of the packed weight block types.
 * TEST INFRASTRUCTURE ONLY: the tests and the smoke check use it as the checker; nothing in the
 * product package reads this file.
 *
 * What it follows: the reference reads a weight of a packed tensor on the host, in double,
 * straight from the format definitions (tests/matrix_kref.h:110-181 for Q4_1, Q5_0, Q5_1 and
 * the K types; tests/matrix_test.cu:84-109 for Q8_0, Q4_0, F16 and F32, there with a rounding
 * to half that belongs to the dequantisation, not to the value).  This file restates the value
 * of weight j of a row, in double, type by type; tests/test_blocks.py pins it against the
 * reference's reading compiled from the reference tree (oracle/_ref/libkref_ref.so) and
 * against tests/golden/blocks.npz.
 *
 * The formats (bytes of one block; every d, dmin, m is a little-endian binary16):
 *   Q4_0 18: d | 16 bytes, byte i = weight i (low nibble) and weight i + 16 (high nibble)
 *   Q4_1 20: d m | 16 nibble bytes                      value = d q + m
 *   Q5_0 22: d | 32 fifth bits | 16 nibble bytes        value = d (q - 16)
 *   Q5_1 24: d m | 32 fifth bits | 16 nibble bytes      value = d q + m
 *   Q8_0 34: d | 32 signed bytes                        value = d q
 *   Q2_K  84 / 256: 16 bytes (scale low, minimum high) | 64 code bytes | d dmin
 *   Q3_K 110 / 256: 32 mask bytes | 64 code bytes | 12 scale bytes | d
 *   Q4_K 144 / 256: d dmin | 12 scale bytes | 128 nibble bytes
 *   Q5_K 176 / 256: d dmin | 12 scale bytes | 32 fifth-bit bytes | 128 nibble bytes
 *   Q6_K 210 / 256: 128 nibble bytes | 64 bytes of bit pairs | 16 signed scales | d
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static double half_value(const uint8_t *at)
{
    uint32_t bits = (uint32_t)at[0] | ((uint32_t)at[1] << 8);
    uint32_t exponent = (bits >> 10) & 31u;
    uint32_t fraction = bits & 1023u;
    double magnitude;
    if (exponent == 31u) {
        magnitude = fraction == 0u ? INFINITY : NAN;
    } else if (exponent == 0u) {
        magnitude = ldexp((double)fraction, -24);
    } else {
        magnitude = ldexp((double)(fraction + 1024u), (int)exponent - 25);
    }
    return (bits & 0x8000u) ? -magnitude : magnitude;
}

/* Bytes of a row of k weights; 0 for a type without a layout or a row that is not whole
 * blocks (tests/matrix_kref.h:92-107; disk/modelfile/modelfile.h:58-88). */
uint64_t q8o_block_row_bytes(uint32_t type, uint32_t k)
{
    uint32_t weights, bytes;
    switch (type) {
    case 0: weights = 1; bytes = 4; break;
    case 1: weights = 1; bytes = 2; break;
    case 2: weights = 32; bytes = 18; break;
    case 3: weights = 32; bytes = 20; break;
    case 6: weights = 32; bytes = 22; break;
    case 7: weights = 32; bytes = 24; break;
    case 8: weights = 32; bytes = 34; break;
    case 10: weights = 256; bytes = 84; break;
    case 11: weights = 256; bytes = 110; break;
    case 12: weights = 256; bytes = 144; break;
    case 13: weights = 256; bytes = 176; break;
    case 14: weights = 256; bytes = 210; break;
    default: return 0;
    }
    if (k % weights != 0u) {
        return 0;
    }
    return (uint64_t)(k / weights) * bytes;
}

/* scale and minimum (6 bits each) of sub block `sub` of a Q4_K / Q5_K super block
 * (tests/matrix_kref.h:78-89) */
static void six_bit_pair(const uint8_t *packed, uint32_t sub, uint32_t *scale, uint32_t *minimum)
{
    if (sub < 4u) {
        *scale = packed[sub] % 64u;
        *minimum = packed[sub + 4u] % 64u;
    } else {
        *scale = packed[sub + 4u] % 16u + 16u * (packed[sub - 4u] / 64u);
        *minimum = packed[sub + 4u] / 16u + 16u * (packed[sub] / 64u);
    }
}

/* Weight j of a row, in double; NAN for a type without a layout. */
double q8o_block_weight(uint32_t type, const uint8_t *row, uint32_t j)
{
    if (type == 0u) {
        float value;
        memcpy(&value, row + (size_t)j * 4u, sizeof value);
        return (double)value;
    }
    if (type == 1u) {
        return half_value(row + (size_t)j * 2u);
    }
    if (type == 2u || type == 3u || type == 6u || type == 7u || type == 8u) {
        const uint32_t size = (uint32_t)q8o_block_row_bytes(type, 32u);
        const uint8_t *block = row + (size_t)(j / 32u) * size;
        const uint32_t at = j % 32u;
        const double d = half_value(block);
        if (type == 8u) {
            return d * (double)(int8_t)block[2u + at];
        }
        const int affine = type == 3u || type == 7u;
        const int fifth = type == 6u || type == 7u;
        const uint32_t head = affine ? 4u : 2u;
        const uint8_t *nibbles = block + head + (fifth ? 4u : 0u);
        const uint32_t pair = nibbles[at % 16u];
        int code = (int)(at < 16u ? pair % 16u : pair / 16u);
        if (fifth) {
            /* bit `at` of the 32-bit little-endian word after the head */
            code += 16 * (int)((block[head + at / 8u] >> (at % 8u)) & 1u);
        }
        if (affine) {
            return d * (double)code + half_value(block + 2u);
        }
        return d * (double)(code - (fifth ? 16 : 8));
    }
    if (type < 10u || type > 14u) {
        return NAN;
    }
    const uint32_t size = (uint32_t)q8o_block_row_bytes(type, 256u);
    const uint8_t *block = row + (size_t)(j / 256u) * size;
    const uint32_t at = j % 256u;      /* position in the super block */
    const uint32_t sub = at / 32u;     /* sub block of 32 */
    const uint32_t lane = at % 32u;    /* weight of the sub block */
    if (type == 10u) {
        /* two bits per weight: byte (at / 128) * 32 + lane holds the weights lane, lane + 32,
         * lane + 64, lane + 96 of its half from the low bits up; one scale byte per 16 weights */
        const uint32_t code = (block[16u + (at / 128u) * 32u + lane] >> (2u * (sub % 4u))) & 3u;
        const uint32_t packed = block[at / 16u];
        return half_value(block + 80u) * (double)(packed % 16u) * (double)code
             - half_value(block + 82u) * (double)(packed / 16u);
    }
    if (type == 11u) {
        int code = (int)((block[32u + (at / 128u) * 32u + lane] >> (2u * (sub % 4u))) & 3u);
        if (((block[lane] >> sub) & 1u) == 0u) {
            code -= 4;                  /* a clear mask bit lowers the code by 4 */
        }
        const uint32_t s = at / 16u;    /* one 6-bit scale per 16 weights, stored split */
        const uint32_t low = (block[96u + s % 8u] >> (4u * (s / 8u))) & 15u;
        const uint32_t high = (block[104u + s % 4u] >> (2u * (s / 4u))) & 3u;
        return half_value(block + 108u) * (double)((int)(low + 16u * high) - 32) * (double)code;
    }
    if (type == 14u) {
        const uint32_t half_block = sub / 4u;   /* 128 weights */
        const uint32_t quarter = sub % 4u;
        const uint32_t byte = block[half_block * 64u + (quarter % 2u) * 32u + lane];
        const uint32_t low = quarter < 2u ? byte % 16u : byte / 16u;
        const uint32_t high = (block[128u + half_block * 32u + lane] >> (2u * quarter)) & 3u;
        const int scale = (int)(int8_t)block[192u + 2u * sub + lane / 16u];
        return half_value(block + 208u) * (double)scale * (double)((int)(low + 16u * high) - 32);
    }
    /* Q4_K and Q5_K */
    uint32_t scale = 0, minimum = 0;
    six_bit_pair(block + 4u, sub, &scale, &minimum);
    const uint8_t *nibbles = block + (type == 12u ? 16u : 48u);
    const uint32_t byte = nibbles[(sub / 2u) * 32u + lane];
    uint32_t code = sub % 2u == 0u ? byte % 16u : byte / 16u;
    if (type == 13u && ((block[16u + lane] >> sub) & 1u) != 0u) {
        code += 16u;
    }
    return half_value(block) * (double)scale * (double)code - half_value(block + 2u) * (double)minimum;
}

/* [rows][k] doubles of rows [first, first + rows) of a tensor. */
void q8o_block_rows(uint32_t type, const uint8_t *w, uint32_t k, uint32_t first, uint32_t rows, double *out)
{
    const uint64_t stride = q8o_block_row_bytes(type, k);
    for (uint32_t r = 0; r < rows; ++r) {
        const uint8_t *row = w + stride * (uint64_t)(first + r);
        for (uint32_t j = 0; j < k; ++j) {
            out[(size_t)r * k + j] = q8o_block_weight(type, row, j);
        }
    }
}
