// The block formats of a GGUF weight tensor other than Q8_0's fast path: one decoder that turns
// the 32 weights of one block (or of one 32-weight sub block of a 256-weight super block) into
// floats, written for host and device from the published definitions of the formats.
//
// Every value is the correctly rounded float of the format's real-number expression, formed
// with at most one rounding (one fused multiply-add after exact products of a binary16 scale
// with a small integer).  That is also what the reference's device readers produce
// (cuda/model/matrix.cuh:163-245, 255-340, 413-470), so the halves this library writes are the
// same bits; the host reading tests/matrix_kref.h:110-181 is the checker on the CPU.
//
// Layouts (bytes of one block; d, dmin, m are binary16, little-endian):
//   F32    4 per weight          F16    2 per weight
//   Q4_0  18: d, 16 nibble bytes               w[i] = d (lo(i) - 8), w[i+16] = d (hi(i) - 8)
//   Q4_1  20: d, m, 16 nibble bytes            w = d q + m
//   Q5_0  22: d, 4 bytes of fifth bits, 16 nibble bytes        w = d (q - 16)
//   Q5_1  24: d, m, 4 bytes of fifth bits, 16 nibble bytes     w = d q + m
//   Q8_0  34: d, 32 signed bytes               w = d q
//   Q2_K  84 per 256: 16 (scale | min << 4) bytes, 64 code bytes, d, dmin
//   Q3_K 110 per 256: 32 sign-mask bytes, 64 code bytes, 12 scale bytes, d
//   Q4_K 144 per 256: d, dmin, 12 scale bytes, 128 nibble bytes
//   Q5_K 176 per 256: d, dmin, 12 scale bytes, 32 fifth-bit bytes, 128 nibble bytes
//   Q6_K 210 per 256: 128 nibble bytes, 64 bytes of upper bit pairs, 16 signed scales, d
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace q8 {

enum BlockType : uint32_t {
    kTypeF32 = 0, kTypeF16 = 1, kTypeQ4_0 = 2, kTypeQ4_1 = 3, kTypeQ5_0 = 6, kTypeQ5_1 = 7, kTypeQ8_0 = 8,
    kTypeQ2_K = 10, kTypeQ3_K = 11, kTypeQ4_K = 12, kTypeQ5_K = 13, kTypeQ6_K = 14
};

// Weights and bytes of one block of the type; false for a type without a layout here.
__host__ __device__ inline bool block_shape(uint32_t type, uint32_t *weights, uint32_t *bytes)
{
    switch (type) {
    case kTypeF32: *weights = 1; *bytes = 4; return true;
    case kTypeF16: *weights = 1; *bytes = 2; return true;
    case kTypeQ4_0: *weights = 32; *bytes = 18; return true;
    case kTypeQ4_1: *weights = 32; *bytes = 20; return true;
    case kTypeQ5_0: *weights = 32; *bytes = 22; return true;
    case kTypeQ5_1: *weights = 32; *bytes = 24; return true;
    case kTypeQ8_0: *weights = 32; *bytes = 34; return true;
    case kTypeQ2_K: *weights = 256; *bytes = 84; return true;
    case kTypeQ3_K: *weights = 256; *bytes = 110; return true;
    case kTypeQ4_K: *weights = 256; *bytes = 144; return true;
    case kTypeQ5_K: *weights = 256; *bytes = 176; return true;
    case kTypeQ6_K: *weights = 256; *bytes = 210; return true;
    default: return false;
    }
}

// Bytes of a row of k weights; 0 when the type is unknown or k is not whole blocks.
__host__ __device__ inline unsigned long long block_row_bytes(uint32_t type, uint32_t k)
{
    uint32_t weights = 0, bytes = 0;
    if (!block_shape(type, &weights, &bytes) || (k % weights) != 0u) {
        return 0ull;
    }
    return (unsigned long long)(k / weights) * bytes;
}

// The step in which rows must be whole: 32 for everything that decodes in runs of 32.
__host__ __device__ inline uint32_t block_run(uint32_t type)
{
    uint32_t weights = 0, bytes = 0;
    if (!block_shape(type, &weights, &bytes)) {
        return 0u;
    }
    return weights < 32u ? 32u : weights;
}

__host__ __device__ inline float half_at(const unsigned char *at)
{
    // rows of some types start on odd multiples of 2: read the two bytes, not a half object
    unsigned short bits = (unsigned short)(at[0] | (at[1] << 8));
    return __half2float(__ushort_as_half(bits));
}

// The 6-bit scale and minimum of sub block j from the 12 packed bytes of Q4_K and Q5_K.
__host__ __device__ inline void k_scale_min(const unsigned char *packed, uint32_t j, uint32_t *scale, uint32_t *minimum)
{
    if (j < 4u) {
        *scale = packed[j] & 63u;
        *minimum = packed[j + 4u] & 63u;
    } else {
        *scale = (packed[j + 4u] & 15u) | ((packed[j - 4u] >> 6) << 4);
        *minimum = (packed[j + 4u] >> 4) | ((packed[j] >> 6) << 4);
    }
}

// Weights [32 run, 32 run + 32) of a row of the given type as floats.  `row` is the first byte
// of the row, `run` counts runs of 32 weights from the start of the row.
__host__ __device__ inline void decode_run(uint32_t type, const unsigned char *row, uint32_t run, float *out)
{
    switch (type) {
    case kTypeF32: {
        const unsigned char *at = row + (size_t)run * 128u;
        for (uint32_t i = 0; i < 32u; ++i) {
            uint32_t bits = (uint32_t)at[4u * i] | ((uint32_t)at[4u * i + 1u] << 8) | ((uint32_t)at[4u * i + 2u] << 16)
                          | ((uint32_t)at[4u * i + 3u] << 24);
            union { uint32_t u; float f; } cast;
            cast.u = bits;
            out[i] = cast.f;
        }
        return;
    }
    case kTypeF16: {
        const unsigned char *at = row + (size_t)run * 64u;
        for (uint32_t i = 0; i < 32u; ++i) {
            out[i] = half_at(at + 2u * i);
        }
        return;
    }
    case kTypeQ4_0: {
        const unsigned char *one = row + (size_t)run * 18u;
        const float d = half_at(one);
        for (uint32_t i = 0; i < 16u; ++i) {
            const uint32_t pair = one[2u + i];
            out[i] = d * (float)((int)(pair & 15u) - 8);
            out[i + 16u] = d * (float)((int)(pair >> 4) - 8);
        }
        return;
    }
    case kTypeQ4_1: {
        const unsigned char *one = row + (size_t)run * 20u;
        const float d = half_at(one);
        const float m = half_at(one + 2u);
        for (uint32_t i = 0; i < 16u; ++i) {
            const uint32_t pair = one[4u + i];
            out[i] = fmaf(d, (float)(pair & 15u), m);
            out[i + 16u] = fmaf(d, (float)(pair >> 4), m);
        }
        return;
    }
    case kTypeQ5_0:
    case kTypeQ5_1: {
        const bool affine = type == kTypeQ5_1;
        const unsigned char *one = row + (size_t)run * (affine ? 24u : 22u);
        const float d = half_at(one);
        const float m = affine ? half_at(one + 2u) : 0.0f;
        const unsigned char *fifth = one + (affine ? 4u : 2u);
        const uint32_t bits = (uint32_t)fifth[0] | ((uint32_t)fifth[1] << 8) | ((uint32_t)fifth[2] << 16)
                            | ((uint32_t)fifth[3] << 24);
        const unsigned char *nibbles = fifth + 4u;
        for (uint32_t i = 0; i < 16u; ++i) {
            const uint32_t pair = nibbles[i];
            const uint32_t low = (pair & 15u) | (((bits >> i) & 1u) << 4);
            const uint32_t high = (pair >> 4) | (((bits >> (i + 16u)) & 1u) << 4);
            if (affine) {
                out[i] = fmaf(d, (float)low, m);
                out[i + 16u] = fmaf(d, (float)high, m);
            } else {
                out[i] = d * (float)((int)low - 16);
                out[i + 16u] = d * (float)((int)high - 16);
            }
        }
        return;
    }
    case kTypeQ8_0: {
        const unsigned char *one = row + (size_t)run * 34u;
        const float d = half_at(one);
        for (uint32_t i = 0; i < 32u; ++i) {
            out[i] = d * (float)(int)(signed char)one[2u + i];
        }
        return;
    }
    case kTypeQ2_K: {
        const unsigned char *one = row + (size_t)(run >> 3) * 84u;
        const uint32_t j = run & 7u;                  // sub block of 32 in the super block
        const float d = half_at(one + 80u);
        const float dmin = half_at(one + 82u);
        const unsigned char *codes = one + 16u + (j >> 2) * 32u;
        const uint32_t shift = (j & 3u) * 2u;
        for (uint32_t half_run = 0; half_run < 2u; ++half_run) {
            const uint32_t packed = one[2u * j + half_run];   // one scale byte per 16 weights
            const float scale = d * (float)(packed & 15u);
            const float offset = dmin * (float)(packed >> 4);
            for (uint32_t i = 16u * half_run; i < 16u * half_run + 16u; ++i) {
                out[i] = fmaf(scale, (float)((codes[i] >> shift) & 3u), -offset);
            }
        }
        return;
    }
    case kTypeQ3_K: {
        const unsigned char *one = row + (size_t)(run >> 3) * 110u;
        const uint32_t j = run & 7u;
        const float d = half_at(one + 108u);
        const unsigned char *codes = one + 32u + (j >> 2) * 32u;
        const uint32_t shift = (j & 3u) * 2u;
        for (uint32_t half_run = 0; half_run < 2u; ++half_run) {
            const uint32_t s = 2u * j + half_run;     // one 6-bit scale per 16 weights
            const uint32_t low = (one[96u + (s & 7u)] >> ((s >> 3) * 4u)) & 15u;
            const uint32_t high = (one[104u + (s & 3u)] >> ((s >> 2) * 2u)) & 3u;
            const float scale = d * (float)((int)(low | (high << 4)) - 32);
            for (uint32_t i = 16u * half_run; i < 16u * half_run + 16u; ++i) {
                int code = (int)((codes[i] >> shift) & 3u);
                if (((one[i] >> j) & 1u) == 0u) {
                    code -= 4;
                }
                out[i] = scale * (float)code;
            }
        }
        return;
    }
    case kTypeQ4_K:
    case kTypeQ5_K: {
        const bool five = type == kTypeQ5_K;
        const unsigned char *one = row + (size_t)(run >> 3) * (five ? 176u : 144u);
        const uint32_t j = run & 7u;
        uint32_t s = 0, m = 0;
        k_scale_min(one + 4u, j, &s, &m);
        const float scale = half_at(one) * (float)s;
        const float offset = half_at(one + 2u) * (float)m;
        const unsigned char *nibbles = one + (five ? 48u : 16u) + (j >> 1) * 32u;
        const uint32_t shift = (j & 1u) * 4u;
        for (uint32_t i = 0; i < 32u; ++i) {
            uint32_t q = (nibbles[i] >> shift) & 15u;
            if (five) {
                q |= ((one[16u + i] >> j) & 1u) << 4;
            }
            out[i] = fmaf(scale, (float)q, -offset);
        }
        return;
    }
    case kTypeQ6_K: {
        const unsigned char *one = row + (size_t)(run >> 3) * 210u;
        const uint32_t j = run & 7u;
        const uint32_t half_block = j >> 2;           // 128 weights each
        const uint32_t quarter = j & 3u;
        const float d = half_at(one + 208u);
        const unsigned char *nibbles = one + half_block * 64u + (quarter & 1u) * 32u;
        const unsigned char *upper = one + 128u + half_block * 32u;
        const uint32_t shift = (quarter >> 1) * 4u;
        for (uint32_t i = 0; i < 32u; ++i) {
            const int scale_byte = (int)(signed char)one[192u + 2u * j + (i >> 4)];
            const float scale = d * (float)scale_byte;
            const uint32_t low = (nibbles[i] >> shift) & 15u;
            const uint32_t high = (upper[i] >> (quarter * 2u)) & 3u;
            out[i] = scale * (float)((int)(low | (high << 4)) - 32);
        }
        return;
    }
    default:
        for (uint32_t i = 0; i < 32u; ++i) {
            out[i] = 0.0f;
        }
        return;
    }
}

} // namespace q8
