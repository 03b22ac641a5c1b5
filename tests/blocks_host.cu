// Host build of the block decoder (aotx_b200/csrc/q_blocks.cuh), the same source the kernels
// compile, so that the tests can hold it against the reference's host reading on the CPU.
#include "q_blocks.cuh"

extern "C" void blocks_decode_run(uint32_t type, const unsigned char *row, uint32_t run, float *out)
{
    q8::decode_run(type, row, run, out);
}

extern "C" unsigned long long blocks_row_bytes(uint32_t type, uint32_t k)
{
    return q8::block_row_bytes(type, k);
}

// half(weight) as the dequantisation writes it
extern "C" void blocks_decode_run_half(uint32_t type, const unsigned char *row, uint32_t run, unsigned short *out)
{
    float values[32];
    q8::decode_run(type, row, run, values);
    for (int i = 0; i < 32; ++i) {
        out[i] = __half_as_ushort(__float2half_rn(values[i]));
    }
}
