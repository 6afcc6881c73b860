/*
 * CPU oracle for the packed-s4 x packed-s4 -> int32 linear layer.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library or its Python
 * package may call into this file; it exists so that tests, the smoke check and
 * the benchmark's CPU-baseline leg have an independent statement of the
 * reference's arithmetic to compare the CUDA path against.
 *
 * It is a restatement, in plain C, of three pieces of myeongs-song/Int4Linear:
 *   - pack      utils/packer.cpp:3-18
 *   - unpack    utils/packer.cpp:20-31
 *   - linear_ref / is_same   test/test_correctness.cu:12-27
 *
 * Parity pin: the reference ships no golden vectors (its own comparison is
 * commented out, test/test_correctness.cu:66-76), so this file is pinned by
 * running it against the reference's own pack / unpack / linear_ref compiled
 * from the reference tree (see build.py in this directory) and by the fixtures under
 * tests/golden/ that were produced by that compiled reference code.
 *
 * All arithmetic is integer; OpenMP parallelism over output rows cannot change
 * any result.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* utils/packer.cpp:3-18 -- eight signed nibbles per 32-bit word, element
 * j*8+t of a row goes to bits [4t, 4t+4); rows are padded to a multiple of 8
 * elements with zero nibbles. */
void oracle_pack(const int *src, int *dst, int m, int n)
{
    int n_dst = (n + 7) / 8;
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n_dst; ++j) {
            uint32_t word = 0;
            for (int t = 0; t < 8; ++t) {
                int col = j * 8 + t;
                if (col < n)
                    word |= ((uint32_t)src[(size_t)i * n + col] & 0xFu) << (4 * t);
            }
            dst[(size_t)i * n_dst + j] = (int)word;
        }
    }
}

/* utils/packer.cpp:20-31 -- inverse of oracle_pack with sign extension of
 * each nibble (0x8..0xF -> -8..-1). */
void oracle_unpack(const int *src, int *dst, int m, int n)
{
    int n_src = (n + 7) / 8;
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            uint32_t word = (uint32_t)src[(size_t)i * n_src + j / 8];
            int nib = (int)((word >> (4 * (j % 8))) & 0xFu);
            dst[(size_t)i * n + j] = (nib & 0x8) ? (nib - 16) : nib;
        }
    }
}

/* test/test_correctness.cu:12-19 -- y[i][j] = sum_l x[i][l] * w[j][l], int32
 * accumulate, operands one int per element. */
void oracle_linear_ref(const int *x, const int *w, int *y, int m, int n, int k)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < m; ++i) {
        const int *xr = x + (size_t)i * k;
        for (int j = 0; j < n; ++j) {
            const int *wr = w + (size_t)j * k;
            int acc = 0;
            for (int l = 0; l < k; ++l) acc += xr[l] * wr[l];
            y[(size_t)i * n + j] = acc;
        }
    }
}

/* Same arithmetic for a chosen subset of output rows: y_rows[r][j] is row
 * rows[r] of the full product.  Lets full-size shapes be spot-checked
 * exactly without computing all m rows on the CPU. */
void oracle_linear_ref_rows(const int *x, const int *w, int *y_rows,
                            const int *rows, int n_rows, int n, int k)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < n_rows; ++r) {
        const int *xr = x + (size_t)rows[r] * k;
        for (int j = 0; j < n; ++j) {
            const int *wr = w + (size_t)j * k;
            int acc = 0;
            for (int l = 0; l < k; ++l) acc += xr[l] * wr[l];
            y_rows[(size_t)r * n + j] = acc;
        }
    }
}

/* The operator exactly as the device sees it: packed operands in, int32 out.
 * Unpacks with oracle_unpack and then applies oracle_linear_ref. Returns 0 on
 * success, -1 if the scratch allocation fails. */
int oracle_linear_packed(const int *x_packed, const int *w_packed, int *y,
                         int m, int n, int k)
{
    int *x = (int *)malloc((size_t)m * k * sizeof(int));
    int *w = (int *)malloc((size_t)n * k * sizeof(int));
    if (!x || !w) { free(x); free(w); return -1; }
    oracle_unpack(x_packed, x, m, k);
    oracle_unpack(w_packed, w, n, k);
    oracle_linear_ref(x, w, y, m, n, k);
    free(x);
    free(w);
    return 0;
}

/* test/test_correctness.cu:22-27 -- exact equality over `count` ints.
 * Returns 1 when every element matches, else 0. */
int oracle_is_same(const int *a, const int *b, long long count)
{
    for (long long i = 0; i < count; ++i)
        if (a[i] != b[i]) return 0;
    return 1;
}

/* Single-threaded variant used when the CPU baseline is timed on one core,
 * which is how the reference itself would run it. */
void oracle_linear_ref_1t(const int *x, const int *w, int *y, int m, int n, int k)
{
    for (int i = 0; i < m; ++i) {
        for (int j = 0; j < n; ++j) {
            int acc = 0;
            for (int l = 0; l < k; ++l)
                acc += x[(size_t)i * k + l] * w[(size_t)j * k + l];
            y[(size_t)i * n + j] = acc;
        }
    }
}
