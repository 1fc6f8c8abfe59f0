/*
 * ref_wrap.c -- exported shims around the reference's own CPU decode.
 *
 * TEST INFRASTRUCTURE ONLY.  build.py extracts the plain-C decode section of the
 * reference's inference/src/format.m (lines 17-174: format_fp16_to_f32,
 * format_bf16_to_f32, format_unpack_q4k_scale_min_pair and the four
 * format_decode_*_row functions) into _ref/format_core.inc at build time and
 * compiles this file around it.  The extracted text is never committed.  The
 * functions there are `static`, so they are reached through the shims below.
 */
#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>
#include <math.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "_ref/format_core.inc"

float ref_fp16_to_f32(uint16_t h) { return format_fp16_to_f32(h); }

void ref_unpack_scale_min_pair(const uint8_t *sc, uint32_t g, float *out4)
{
    format_unpack_q4k_scale_min_pair(sc, g, out4 + 0, out4 + 1, out4 + 2, out4 + 3);
}

/* fmt uses the QuantFormat numbering of inference/include/orome.h:227-235 */
static size_t ref_row_bytes(int fmt, uint32_t in_dim)
{
    switch (fmt) {
    case 3: return (size_t)(in_dim / 32) * 34;
    case 0: return (size_t)(in_dim / 256) * 144;
    case 1: return (size_t)(in_dim / 256) * 176;
    case 2: return (size_t)(in_dim / 256) * 210;
    }
    return 0;
}

int ref_decode_row(int fmt, const uint8_t *row, uint32_t in_dim, float *out)
{
    switch (fmt) {
    case 3: return format_decode_q8_0_row(row, in_dim, out) ? 0 : -1;
    case 0: return format_decode_q4_k_row(row, in_dim, out) ? 0 : -1;
    case 1: return format_decode_q5_k_row(row, in_dim, out) ? 0 : -1;
    case 2: return format_decode_q6_k_row(row, in_dim, out) ? 0 : -1;
    }
    return -1;
}

int ref_decode_rows(int fmt, const uint8_t *data, uint32_t row0, uint32_t nrows, uint32_t in_dim, float *out)
{
    size_t rb = ref_row_bytes(fmt, in_dim);
    int rc = 0;
#pragma omp parallel for schedule(static) reduction(|:rc)
    for (int64_t r = 0; r < (int64_t)nrows; ++r)
        rc |= ref_decode_row(fmt, data + (size_t)(row0 + r) * rb, in_dim, out + (size_t)r * in_dim);
    return rc ? -1 : 0;
}

/* The reference's CPU form of the path: its own row decode into an fp32 row
 * buffer followed by the fp32 dot product its tests write inline
 * (tests/test_q8_0.m:41,66).  Rows are spread over the host threads. */
int ref_matvec_f32(int fmt, const uint8_t *data, uint32_t out_dim, uint32_t in_dim,
                   const float *x, int batch, int ldx, float *y, int ldy)
{
    size_t rb = ref_row_bytes(fmt, in_dim);
    int rc = 0;
#pragma omp parallel reduction(|:rc)
    {
        float *w = (float *)malloc((size_t)in_dim * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)out_dim; ++r) {
            rc |= ref_decode_row(fmt, data + (size_t)r * rb, in_dim, w);
            for (int b = 0; b < batch; ++b) {
                const float *xb = x + (size_t)b * ldx;
                float acc = 0.0f;
                for (uint32_t c = 0; c < in_dim; ++c) acc += w[c] * xb[c];
                y[(size_t)b * ldy + r] = acc;
            }
        }
        free(w);
    }
    return rc ? -1 : 0;
}

int ref_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for its thread count explicitly. */
void ref_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
