/*
 * Thin extern "C" shim around the UNMODIFIED reference sources, compiled where
 * they lie (the reference tree is passed with -I; nothing is copied).
 *
 * TEST INFRASTRUCTURE ONLY: the built library lands in oracle/_ref/ and is
 * used to pin the C restatement in linear_ref.c, to generate the fixtures in
 * tests/golden/, and as the "reference" CPU baseline.
 *
 * The reference keeps linear_ref / is_same inside test/test_correctness.cu
 * next to a main() that needs a GPU, so that translation unit is included
 * here with its main renamed; the functions themselves are untouched.
 */
#define main int4linear_reference_main_not_used
#include "test/test_correctness.cu"
#undef main

extern "C" {

/* utils/packer.cpp:3 */
void ref_pack(const int *src, int *dst, int m, int n) { pack(src, dst, m, n); }

/* utils/packer.cpp:20 */
void ref_unpack(const int *src, int *dst, int m, int n) { unpack(src, dst, m, n); }

/* test/test_correctness.cu:12 */
void ref_linear_ref(int *x, int *w, int *y, int m, int n, int k) { linear_ref(x, w, y, m, n, k); }

/* test/test_correctness.cu:22 */
int ref_is_same(int *a, int *b, int count) { return is_same(a, b, count) ? 1 : 0; }

/* kernels/linear_v21.cu:9 -- the reference's own GPU launcher (Ampere-style
 * mma.sync kernel recompiled for sm_100a); device pointers in, blocking. */
void ref_linear_v21_launch(void *x_packed_d, void *w_packed_d, void *y_d, int m, int n, int k)
{
    linear_v21_launch(x_packed_d, w_packed_d, y_d, m, n, k);
}

}  // extern "C"
