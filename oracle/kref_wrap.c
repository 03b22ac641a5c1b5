/* Exposes the reference's host reading of packed weight blocks (tests/matrix_kref.h:110-181,
 * double precision, written by the reference from the format definitions) and its Q8_0 / Q4_0 /
 * F16 / F32 reading (tests/matrix_test.cu:84-109 restated in q8_oracle.c for Q8_0) to the tests.
 * TEST INFRASTRUCTURE ONLY.  The header is included from where it lies in the reference tree;
 * nothing of it is copied. */
#include <stddef.h>

#include "matrix_kref.h"

double kref_weight(const unsigned char *row, unsigned int type, unsigned int j)
{
    return aotx_kref_weight(row, type, j);
}

unsigned long long kref_row_bytes(unsigned int type, unsigned int k)
{
    return aotx_kref_row_bytes(type, k);
}
