/*
 * oracle.c -- CPU restatement of Orome's quantized dequant-matvec path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; only tests/, the smoke check and the CPU-baseline leg of the
 * benchmark may use it, and only as the checker.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the Orome source tree).  Compile with -ffp-contract=off: the reference's CPU
 * decode is written as separate multiply / subtract C expressions.  For the
 * decoders the contraction mode turns out not to matter (d*sc*q carries at most
 * 11+6+5 significant bits, so the product is exact and `a*q - m` rounds once
 * either way; the `fused` switch exists so a test can demonstrate it), but the
 * fp32 dot products would change with it.
 *
 * Parity pin: decode functions are checked bit-for-bit against the reference's
 * own format.m decode (compiled from the reference tree into oracle/_ref) and
 * against the closed-form vectors of tests/test_q8_0.m, tests/test_q4k.m and
 * tests/test_f32.m.  Layout-B scales, the routing kernel, the expert FFN and
 * MoE block, and the arg-max kernel's tie order have no reference test; they
 * follow the shader source only (parity unpinned beyond the source itself).
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* QuantFormat numbering: inference/include/orome.h:227-235 */
enum { OQ_Q4_K = 0, OQ_Q5_K = 1, OQ_Q6_K = 2, OQ_Q8_0 = 3, OQ_F16 = 4, OQ_BF16 = 5, OQ_F32 = 6 };
enum { LAYOUT_A = 0, LAYOUT_B = 1 };

/* ---------------------------------------------------------------------- */
/* scalar helpers                                                          */
/* ---------------------------------------------------------------------- */

/* IEEE binary16 -> binary32, exact.  Restates format.m:17-32 (subnormals are
 * mant * 2^-24, exp 31 is inf/NaN).  Written as a bit construction rather than
 * ldexpf so it has no libm dependency; the value is identical for every one of
 * the 65536 inputs (tests compare all of them against the reference build). */
float oracle_half_to_float(uint16_t h)
{
    uint32_t sgn = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 31u, m = h & 1023u, bits;
    if (e == 31u) {
        bits = m ? 0x7FC00000u : (sgn | 0x7F800000u);        /* NaN is the positive quiet NAN macro */
    } else if (e) {
        bits = sgn | ((e + 112u) << 23) | (m << 13);
    } else if (m == 0) {
        bits = sgn;
    } else {
        int sh = 0;
        while (!(m & 1024u)) { m <<= 1; ++sh; }
        bits = sgn | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
    }
    float f; memcpy(&f, &bits, 4); return f;
}

static float bf16_to_float(uint16_t h)   /* format.m:34-39 */
{
    uint32_t b = (uint32_t)h << 16; float f; memcpy(&f, &b, 4); return f;
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Six-bit scale / min tables of one K-quant superblock (12 packed bytes).
 *
 * Layout A restates format_unpack_q4k_scale_min_pair, format.m:41-64 (identical
 * to shaders.metal:1413-1436): sub-blocks 0..3 read the low six bits of bytes
 * 0..3 (scales) and 4..7 (mins); for the pair (4+2u, 5+2u), u in {0,1}, the low
 * and high nibble of byte 8+u (scales) or 10+u (mins) are extended by the top
 * two bits of bytes 2u, 2u+1 (scales) or 2u+4, 2u+5 (mins).
 *
 * Layout B restates the mask arithmetic of the llama-style kernels,
 * shaders.metal:1575-1578: for j >= 4 the scale is the low nibble of byte j+4
 * extended by the top bits of byte j-4, the min the high nibble of byte j+4
 * extended by the top bits of byte j.  The two layouts agree on sub-blocks
 * 0..3, on scale 4 and on min 7 only.
 */
void oracle_kquant_scales(const uint8_t *p, int layout, uint8_t sc[8], uint8_t mn[8])
{
    for (int j = 0; j < 4; ++j) { sc[j] = p[j] & 63; mn[j] = p[j + 4] & 63; }
    if (layout == LAYOUT_A) {
        for (int u = 0; u < 2; ++u) {
            uint8_t sp = p[8 + u], mp = p[10 + u];
            sc[4 + 2 * u] = (uint8_t)((sp & 15) | ((p[2 * u]     >> 6) << 4));
            sc[5 + 2 * u] = (uint8_t)((sp >> 4) | ((p[2 * u + 1] >> 6) << 4));
            mn[4 + 2 * u] = (uint8_t)((mp & 15) | ((p[2 * u + 4] >> 6) << 4));
            mn[5 + 2 * u] = (uint8_t)((mp >> 4) | ((p[2 * u + 5] >> 6) << 4));
        }
    } else {
        for (int j = 4; j < 8; ++j) {
            sc[j] = (uint8_t)((p[j + 4] & 15) | ((p[j - 4] >> 6) << 4));
            mn[j] = (uint8_t)((p[j + 4] >> 4) | ((p[j]     >> 6) << 4));
        }
    }
}

size_t oracle_row_bytes(int fmt, uint32_t in_dim)
{
    switch (fmt) {
    case OQ_Q8_0: return (size_t)(in_dim / 32) * 34;     /* format.m:198 */
    case OQ_Q4_K: return (size_t)(in_dim / 256) * 144;   /* format.m:203 */
    case OQ_Q5_K: return (size_t)(in_dim / 256) * 176;   /* format.m:208 */
    case OQ_Q6_K: return (size_t)(in_dim / 256) * 210;   /* format.m:213 */
    case OQ_F16: case OQ_BF16: return (size_t)in_dim * 2;
    case OQ_F32: return (size_t)in_dim * 4;
    }
    return 0;
}

/* ---------------------------------------------------------------------- */
/* row decoders (bit-exact contract)                                       */
/* ---------------------------------------------------------------------- */

/* format_decode_q8_0_row, format.m:66-79: w = d * (float)q, one fp32 multiply. */
static void dec_q8_0(const uint8_t *row, uint32_t n, float *out)
{
    for (uint32_t b = 0; b < n / 32; ++b, row += 34, out += 32) {
        float d = oracle_half_to_float(rd16(row));
        const int8_t *q = (const int8_t *)(row + 2);
        for (int j = 0; j < 32; ++j) out[j] = d * (float)q[j];
    }
}

/* format_decode_q4_k_row, format.m:81-108.  Order of operations: a = d*sc and
 * m = dmin*mn first (both exact: 11-bit half mantissa times a 6-bit integer),
 * then a*q (exact) minus m, one rounding; fmaf(a, q, -m) is the same number. */
static void dec_q4_k(const uint8_t *row, uint32_t n, float *out, int layout, int fused)
{
    for (uint32_t s = 0; s < n / 256; ++s, row += 144, out += 256) {
        float d = oracle_half_to_float(rd16(row)), dmin = oracle_half_to_float(rd16(row + 2));
        uint8_t sc[8], mn[8];
        oracle_kquant_scales(row + 4, layout, sc, mn);
        const uint8_t *qs = row + 16;
        for (int sub = 0; sub < 8; ++sub) {
            float a = d * (float)sc[sub], m = dmin * (float)mn[sub];
            const uint8_t *src = qs + 32 * (sub >> 1);
            int shift = (sub & 1) * 4;
            for (int l = 0; l < 32; ++l) {
                float q = (float)((src[l] >> shift) & 15);
                out[32 * sub + l] = fused ? fmaf(a, q, -m) : (a * q) - m;
            }
        }
    }
}

/* format_decode_q5_k_row, format.m:110-142: Q4_K plus one high bit per weight,
 * bit (sub) of qh[l] for sub-block sub (mask 1<<(2g) / 1<<(2g+1) with sub=2g,2g+1). */
static void dec_q5_k(const uint8_t *row, uint32_t n, float *out, int layout, int fused)
{
    for (uint32_t s = 0; s < n / 256; ++s, row += 176, out += 256) {
        float d = oracle_half_to_float(rd16(row)), dmin = oracle_half_to_float(rd16(row + 2));
        uint8_t sc[8], mn[8];
        oracle_kquant_scales(row + 4, layout, sc, mn);
        const uint8_t *qh = row + 16, *ql = row + 48;
        for (int sub = 0; sub < 8; ++sub) {
            float a = d * (float)sc[sub], m = dmin * (float)mn[sub];
            const uint8_t *src = ql + 32 * (sub >> 1);
            int shift = (sub & 1) * 4;
            for (int l = 0; l < 32; ++l) {
                int q5 = ((src[l] >> shift) & 15) | (((qh[l] >> sub) & 1) << 4);
                float q = (float)q5;
                out[32 * sub + l] = fused ? fmaf(a, q, -m) : (a * q) - m;
            }
        }
    }
}

/* format_decode_q6_k_row, format.m:144-174.  Superblock = ql[128] qh[64]
 * sc[16] (int8) d (fp16 at byte 208).  Within each 128-weight half, position
 * p = 32*t + l (t = 0..3, l = 0..31) takes its low nibble from
 * ql[64*half + 32*(t&1) + l] (high nibble when t >= 2), its top two bits from
 * bits 2t..2t+1 of qh[32*half + l], and its scale from sc[8*half + l/16 + 2t].
 * Value = (d * (float)sc) * (float)(q - 32), evaluated left to right. */
static void dec_q6_k(const uint8_t *row, uint32_t n, float *out)
{
    for (uint32_t s = 0; s < n / 256; ++s, row += 210, out += 256) {
        const int8_t *sc = (const int8_t *)(row + 192);
        float d = oracle_half_to_float(rd16(row + 208));
        for (int half = 0; half < 2; ++half) {
            const uint8_t *ql = row + 64 * half, *qh = row + 128 + 32 * half;
            for (int t = 0; t < 4; ++t) {
                for (int l = 0; l < 32; ++l) {
                    int lo = (ql[32 * (t & 1) + l] >> (4 * (t >> 1))) & 15;
                    int hi = (qh[l] >> (2 * t)) & 3;
                    int q = (lo | (hi << 4)) - 32;
                    float a = d * (float)sc[8 * half + (l >> 4) + 2 * t];
                    out[128 * half + 32 * t + l] = a * (float)q;
                }
            }
        }
    }
}

/* format_decode_row_f32, format.m:176-218.  `row` points at the first byte of
 * the row.  Returns 0 on success, -1 when in_dim is not a whole number of
 * blocks (the reference returns false). */
int oracle_decode_row(int fmt, int layout, int fused, const uint8_t *row, uint32_t in_dim, float *out)
{
    switch (fmt) {
    case OQ_F32: memcpy(out, row, (size_t)in_dim * 4); return 0;
    case OQ_F16: for (uint32_t j = 0; j < in_dim; ++j) out[j] = oracle_half_to_float(rd16(row + 2 * j)); return 0;
    case OQ_BF16: for (uint32_t j = 0; j < in_dim; ++j) out[j] = bf16_to_float(rd16(row + 2 * j)); return 0;
    case OQ_Q8_0: if (in_dim % 32) return -1; dec_q8_0(row, in_dim, out); return 0;
    case OQ_Q4_K: if (in_dim % 256) return -1; dec_q4_k(row, in_dim, out, layout, fused); return 0;
    case OQ_Q5_K: if (in_dim % 256) return -1; dec_q5_k(row, in_dim, out, layout, fused); return 0;
    case OQ_Q6_K: if (in_dim % 256) return -1; dec_q6_k(row, in_dim, out); return 0;
    }
    return -1;
}

/* Decode nrows consecutive rows into out[nrows][in_dim]. */
int oracle_decode_rows(int fmt, int layout, int fused, const uint8_t *data, uint32_t row0, uint32_t nrows,
                       uint32_t in_dim, float *out)
{
    size_t rb = oracle_row_bytes(fmt, in_dim);
    int rc = 0;
#pragma omp parallel for schedule(static) reduction(|:rc)
    for (int64_t r = 0; r < (int64_t)nrows; ++r)
        rc |= oracle_decode_row(fmt, layout, fused, data + (size_t)(row0 + r) * rb, in_dim, out + (size_t)r * in_dim);
    return rc ? -1 : 0;
}

/* ---------------------------------------------------------------------- */
/* matvec                                                                   */
/* ---------------------------------------------------------------------- */

/* y[b][r] = sum_c W[r][c] * x[b][c] with W the decoded fp32 weights and the sum
 * carried in double: the tolerance reference for every GPU matvec.  The
 * reference has no CPU matvec (kernels.m:21-23 is an empty section); its tests
 * form sum(d*q*x) inline (tests/test_q8_0.m:42-69, tests/verify_gguf.py:61-67). */
int oracle_matvec_f64(int fmt, int layout, const uint8_t *data, uint32_t out_dim, uint32_t in_dim,
                      const float *x, int batch, int ldx, double *y, int ldy)
{
    size_t rb = oracle_row_bytes(fmt, in_dim);
    int rc = 0;
#pragma omp parallel reduction(|:rc)
    {
        float *w = (float *)malloc((size_t)in_dim * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)out_dim; ++r) {
            rc |= oracle_decode_row(fmt, layout, 0, data + (size_t)r * rb, in_dim, w);
            for (int b = 0; b < batch; ++b) {
                const float *xb = x + (size_t)b * ldx;
                double acc = 0.0;
                for (uint32_t c = 0; c < in_dim; ++c) acc += (double)w[c] * (double)xb[c];
                y[(size_t)b * ldy + r] = acc;
            }
        }
        free(w);
    }
    return rc ? -1 : 0;
}

/* Same product with fp32 accumulation in column order, the way the
 * reference's own tests accumulate (tests/test_q8_0.m:41,66; test_f32.m:25-27).
 * This is the routine timed as the CPU baseline ("port" kind). */
int oracle_matvec_f32(int fmt, int layout, const uint8_t *data, uint32_t out_dim, uint32_t in_dim,
                      const float *x, int batch, int ldx, float *y, int ldy)
{
    size_t rb = oracle_row_bytes(fmt, in_dim);
    int rc = 0;
#pragma omp parallel reduction(|:rc)
    {
        float *w = (float *)malloc((size_t)in_dim * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)out_dim; ++r) {
            rc |= oracle_decode_row(fmt, layout, 0, data + (size_t)r * rb, in_dim, w);
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

/* silu(g) * u with silu(g) = g / (1 + exp(-g)): shaders.metal:1027-1029, 2307-2308, 2383-2384.
 * Carried in double so it serves as the tolerance reference for the fused kernels. */
void oracle_swiglu_f64(const double *gate, const double *up, size_t n, double *out)
{
    for (size_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0 + exp(-gate[i])) * up[i];
}

/* ---------------------------------------------------------------------- */
/* MoE routing and expert FFN                                              */
/* ---------------------------------------------------------------------- */

/* softmax_topk_route, shaders.metal:1141-1234.  K rounds of arg-max with the
 * strict `>` comparison, so the lowest index wins a tie (1173, 1194); the winner
 * is masked to -inf (1207-1209).  The weights are a softmax over the selected
 * logits only, w_k = exp(l_k - l_0) / sum (1213-1227), with 1/sum forced to 0
 * when the sum is not positive (1222).  K is capped at 8 (1164) and slots
 * K..7 are zero-filled (1228-1231).  fp32 throughout like the kernel; exp is
 * the host expf, so weights are compared with a small tolerance, indices exactly. */
void oracle_route(const float *logits, uint32_t n_experts, uint32_t K, uint32_t *idx8, float *w8)
{
    uint32_t lim = K < 8 ? K : 8;
    float *v = (float *)malloc(sizeof(float) * (n_experts ? n_experts : 1));
    memcpy(v, logits, sizeof(float) * n_experts);
    float found[8];
    for (uint32_t k = 0; k < lim; ++k) {
        /* The kernel's shuffle tree keeps the left operand unless the right is
         * strictly greater, which yields the first maximum in index order.  With
         * every remaining value at -inf (K > n_experts) the tree returns lane 0. */
        uint32_t bi = 0; float bv = -INFINITY;
        if (n_experts) { bv = v[0]; }
        for (uint32_t i = 1; i < n_experts; ++i) if (v[i] > bv) { bv = v[i]; bi = i; }
        found[k] = bv; idx8[k] = bi;
        if (bi < n_experts) v[bi] = -INFINITY;
    }
    float sum = 0.0f, w[8];
    for (uint32_t k = 0; k < lim; ++k) { w[k] = expf(found[k] - found[0]); sum += w[k]; }
    float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (uint32_t k = 0; k < lim; ++k) w8[k] = w[k] * inv;
    for (uint32_t k = lim; k < 8; ++k) { idx8[k] = 0; w8[k] = 0.0f; }
    free(v);
}

/* Routed-expert FFN of one token, in double on decoded fp32 weights:
 *   act[k][m] = silu(Wg[e_k] x)[m] * (Wu[e_k] x)[m]   (shaders.metal:2232-2310)
 *   out[h]    = sum_k w_k * (Wd[e_k] act[k])[h]        (shaders.metal:2590-2668 + combine 1049-1055)
 * Expert e of a projection starts at base + e * expert_stride (format.m:381-406).
 * The shared-expert term and the residual of the combine kernel are outside
 * this path (the benchmarked MoE configuration has no shared expert). */
int oracle_moe_ffn_f64(const uint8_t *gate, size_t gate_stride, int gate_fmt,
                       const uint8_t *up, size_t up_stride, int up_fmt,
                       const uint8_t *down, size_t down_stride, int down_fmt, int layout,
                       const float *x, uint32_t hidden, uint32_t inter,
                       const uint32_t *idx, const float *w, uint32_t K, double *out)
{
    double *g = (double *)malloc(sizeof(double) * inter), *u = (double *)malloc(sizeof(double) * inter);
    double *act = (double *)malloc(sizeof(double) * inter), *o = (double *)malloc(sizeof(double) * hidden);
    float *actf = (float *)malloc(sizeof(float) * inter);
    int rc = 0;
    for (uint32_t h = 0; h < hidden; ++h) out[h] = 0.0;
    for (uint32_t k = 0; k < K; ++k) {
        size_t e = idx[k];
        rc |= oracle_matvec_f64(gate_fmt, layout, gate + e * gate_stride, inter, hidden, x, 1, 0, g, 0);
        rc |= oracle_matvec_f64(up_fmt, layout, up + e * up_stride, inter, hidden, x, 1, 0, u, 0);
        oracle_swiglu_f64(g, u, inter, act);
        /* the activation handed to the down projection is an fp32 buffer in the reference (engine.m:204) */
        for (uint32_t m = 0; m < inter; ++m) actf[m] = (float)act[m];
        rc |= oracle_matvec_f64(down_fmt, layout, down + e * down_stride, hidden, inter, actf, 1, 0, o, 0);
        for (uint32_t h = 0; h < hidden; ++h) out[h] += (double)w[k] * o[h];
    }
    free(g); free(u); free(act); free(o); free(actf);
    return rc ? -1 : 0;
}

/* argmax_kernel, shaders.metal:1249-1305, as a simulation of its 1024 threads: each thread scans
 * i = lid, lid + 1024, ... keeping its first maximum (strict >, start at -inf / index 0: 1260-1268);
 * a shuffle-down tree inside every 32-lane simdgroup takes the other lane's pair only when its
 * value is strictly greater (1271-1278; lanes whose partner lies beyond the simdgroup keep their
 * own pair); lane 0 of every simdgroup stores its pair, and simdgroup 0 reduces the 32 pairs the
 * same way (1281-1304).  NaN never satisfies `>`, so it never wins. */
uint32_t oracle_argmax(const float *data, uint32_t count)
{
    enum { T = 1024 };
    float val[T]; uint32_t idx[T];
    for (uint32_t lid = 0; lid < T; ++lid) {
        float m = -INFINITY; uint32_t mi = 0;
        for (uint32_t i = lid; i < count; i += T) if (data[i] > m) { m = data[i]; mi = i; }
        val[lid] = m; idx[lid] = mi;
    }
    float tv[32]; uint32_t ti[32];
    for (uint32_t g = 0; g < T / 32; ++g) {
        float *v = val + 32 * g; uint32_t *ix = idx + 32 * g;
        for (uint32_t off = 16; off > 0; off >>= 1) {
            float nv[32]; uint32_t ni[32];
            for (uint32_t l = 0; l < 32; ++l) {
                nv[l] = v[l]; ni[l] = ix[l];
                if (l + off < 32 && v[l + off] > v[l]) { nv[l] = v[l + off]; ni[l] = ix[l + off]; }
            }
            memcpy(v, nv, sizeof nv); memcpy(ix, ni, sizeof ni);
        }
        tv[g] = v[0]; ti[g] = ix[0];
    }
    for (uint32_t off = 16; off > 0; off >>= 1) {
        float nv[32]; uint32_t ni[32];
        for (uint32_t l = 0; l < 32; ++l) {
            nv[l] = tv[l]; ni[l] = ti[l];
            if (l + off < 32 && tv[l + off] > tv[l]) { nv[l] = tv[l + off]; ni[l] = ti[l + off]; }
        }
        memcpy(tv, nv, sizeof nv); memcpy(ti, ni, sizeof ni);
    }
    return ti[0];
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU baseline asks for its thread count explicitly. */
void oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
