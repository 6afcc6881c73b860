/*
 * Drop-in for the reference's utils/packer.h: the host packer, same signatures (utils/packer.h:5-6)
 * and bit layout (utils/packer.cpp:3-31).  The functions are exported by libint4linear_b200.so, so
 * a program written against the reference needs neither its header nor utils/packer.cpp.
 *   src of pack / dst of unpack: m x n ints, one signed 4-bit value per int;
 *   dst of pack / src of unpack: m x ceil(n / 8) ints, eight nibbles per word, low nibble = even index.
 */
#ifndef INT4LINEAR_B200_COMPAT_PACKER_H_
#define INT4LINEAR_B200_COMPAT_PACKER_H_

#include <stdint.h>

void pack(const int* src, int* dst, const int m, const int n);
void unpack(const int* src, int* dst, const int m, const int n);

#endif
