/*
 * Drop-in for the launcher declared by the reference's kernels/linear_v0.h:
 *     void linear_v0_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k);
 * Same operand format and contract as linear_v21_launch (device pointers, default stream, result
 * complete on return); the symbol is exported by libint4linear_b200.so and runs the sm_100a kernels.
 * Only the launcher is provided: the reference's harnesses instantiate a kernel template from
 * kernels/linear_v21.h alone, for which see the header of that name in this directory.
 */
#ifndef INT4LINEAR_B200_COMPAT_LINEAR_V0_H_
#define INT4LINEAR_B200_COMPAT_LINEAR_V0_H_

void linear_v0_launch(void* x_packed_d, void* w_packed_d, void* y_d, int m, int n, int k);

#endif
