/*
 * Test infrastructure only. The reference's delta-rule chunk kernel calls
 * tinytitan_sgemm_rowmajor (sources/TinyTitanKernelsC/include/
 * tinytitan_kernels.h:76-78), whose own definition forwards to Apple's BLAS and
 * is empty elsewhere (sources/TinyTitanKernelsC/dequant_affine.c:139-160).
 * This plain loop supplies the symbol when the reference's two delta-rule
 * sources are compiled, unmodified and in place, into oracle/_ref.
 */
#include <stddef.h>

void tinytitan_sgemm_rowmajor(int transposed_b, int rows, int columns, int inner,
                              const float *a, const float *b, float *out) {
    for (int i = 0; i < rows; ++i) {
        for (int j = 0; j < columns; ++j) {
            float acc = 0.0f;
            for (int l = 0; l < inner; ++l) {
                const float bv = transposed_b ? b[(size_t)j * inner + l] : b[(size_t)l * columns + j];
                acc += a[(size_t)i * inner + l] * bv;
            }
            out[(size_t)i * columns + j] = acc;
        }
    }
}
