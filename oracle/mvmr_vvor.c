/*
 * TEST INFRASTRUCTURE: plain-C restatement of the reference's CPU operators
 * for the two sparse primitives of point convolution.  Built by
 * oracle/build_ref.py into oracle/_ref/liboracle_sparse.so and loaded through
 * ctypes by oracle/sparse_ops.py.  Never linked into the product library.
 *
 *   MVMR  o[oi[t], g, :] += b[bi[t], g, :] @ a[ai[t], g, :, :]
 *         follows extensions/sparse_engines_cuda/csrc/spare_mvmr.cpp:12-75
 *   VVOR  o[oi[t], g, m, c] += a[ai[t], g, m] * b[bi[t], g, c]
 *         follows extensions/sparse_engines_cuda/csrc/sparse_vvor.cpp:12-53
 *
 * Arithmetic is fp32 with fused multiply-add, round-to-nearest, single
 * thread, triplets visited in array order -- the properties that fix the
 * reference's rounding.  The MVMR dot product is not one long chain: the
 * channel axis is cut into blocks of 8 (C <= 8), 16 (C <= 16) or 32 channels,
 * every block is accumulated from zero, and the block sums (then the ragged
 * tail) are added to the running total in order.
 */
#include <math.h>
#include <stdint.h>

static int block_width(int C) {
    if (C <= 8) return 8;
    return C <= 16 ? 16 : 32;
}

/* sum_c w[c*ldw] * x[c], blocked as described above */
static float blocked_dot(const float *w, int ldw, const float *x, int C) {
    const int bw = block_width(C);
    const int nfull = C / bw;
    float total = 0.0f;
    int c = 0;
    for (int blk = 0; blk < nfull; ++blk) {
        float part = 0.0f;
        for (int e = 0; e < bw; ++e, ++c)
            part = fmaf(w[(int64_t)c * ldw], x[c], part);
        total += part;
    }
    float tail = 0.0f;
    for (; c < C; ++c)
        tail = fmaf(w[(int64_t)c * ldw], x[c], tail);
    total += tail;
    return total;
}

/* a: (K,G,C,M)  b: (Nb,G,C)  o: (No,G,M), o must be pre-zeroed by the caller */
void oracle_mvmr_f32(const float *a, const int32_t *ai, const float *b,
                     const int32_t *bi, const int32_t *oi, float *o,
                     int64_t T, int G, int C, int M) {
    for (int64_t t = 0; t < T; ++t) {
        for (int g = 0; g < G; ++g) {
            const float *w = a + ((int64_t)ai[t] * G + g) * C * M;
            const float *x = b + ((int64_t)bi[t] * G + g) * C;
            float *y = o + ((int64_t)oi[t] * G + g) * M;
            if (C == 1) {
                /* spare_mvmr.cpp:16-19 hands C == 1 to the outer-product
                 * loop, which fuses the add into the output element. */
                for (int m = 0; m < M; ++m) y[m] = fmaf(x[0], w[m], y[m]);
                continue;
            }
            for (int m = 0; m < M; ++m) y[m] += blocked_dot(w + m, M, x, C);
        }
    }
}

/* a: (Na,G,M)  b: (Nb,G,C)  o: (No,G,M,C), o must be pre-zeroed */
void oracle_vvor_f32(const float *a, const int32_t *ai, const float *b,
                     const int32_t *bi, const int32_t *oi, float *o,
                     int64_t T, int G, int M, int C) {
    for (int64_t t = 0; t < T; ++t) {
        for (int g = 0; g < G; ++g) {
            const float *u = a + ((int64_t)ai[t] * G + g) * M;
            const float *v = b + ((int64_t)bi[t] * G + g) * C;
            float *y = o + ((int64_t)oi[t] * G + g) * M * C;
            for (int m = 0; m < M; ++m) {
                const float um = u[m];
                float *row = y + (int64_t)m * C;
                for (int c = 0; c < C; ++c) row[c] = fmaf(um, v[c], row[c]);
            }
        }
    }
}
