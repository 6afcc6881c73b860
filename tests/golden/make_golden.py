"""Generate tests/golden/*.npz from the reference's OWN code.

Runs only where oracle/_ref/libint4linear_ref.so exists (built by
oracle/build.py from the reference checkout: utils/packer.cpp and the
linear_ref of test/test_correctness.cu).  Inputs come from the seeded generator
of this repository plus hand-made extreme patterns; packed words come from the
reference's pack(), results from the reference's linear_ref().  The committed
.npz files are what travels; this script documents how they were made.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from int4linear_b200.data import uniform_s4  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, m, n, k, seed_x, seed_w)
RANDOM_CASES = [
    ("rand_8x16x32", 8, 16, 32, 0xA001, 0xB001),
    ("rand_17x24x96", 17, 24, 96, 0xA002, 0xB002),
    ("rand_33x10x160", 33, 10, 160, 0xA003, 0xB003),
    ("rand_1x8x32", 1, 8, 32, 0xA004, 0xB004),
    ("rand_130x66x256", 130, 66, 256, 0xA005, 0xB005),
    ("rand_16x72x512", 16, 72, 512, 0xA006, 0xB006),
    # pack() pads rows to a multiple of 8 elements; exercise that too
    ("rand_5x7x19", 5, 7, 19, 0xA007, 0xB007),
]


def pattern_cases():
    m, n, k = 24, 40, 128
    yield "all_min", np.full((m, k), -8, np.int32), np.full((n, k), -8, np.int32)
    yield "min_times_max", np.full((m, k), -8, np.int32), np.full((n, k), 7, np.int32)
    alt = np.where(np.arange(k) % 2 == 0, 7, -8).astype(np.int32)
    yield "alternating", np.tile(alt, (m, 1)), np.tile(-alt - 1, (n, 1))
    # one non-zero per row at a row-dependent K position: catches any K
    # permutation that differs between the operands
    x = np.zeros((m, k), np.int32)
    w = np.zeros((n, k), np.int32)
    for i in range(m):
        x[i, (5 * i + 3) % k] = (i % 15) - 7
    for j in range(n):
        w[j, (5 * j + 3) % k] = -8 if j % 2 else 7
    yield "single_nonzero", x, w


def main():
    if O.ref_lib() is None:
        raise SystemExit("oracle/_ref is not built (needs the reference checkout); nothing generated")
    for name, m, n, k, sx, sw in RANDOM_CASES:
        x = uniform_s4(sx, m, k).astype(np.int32)
        w = uniform_s4(sw, n, k).astype(np.int32)
        save(name, x, w)
    for name, x, w in pattern_cases():
        save("pattern_" + name, x, w)


def save(name, x, w):
    xp, wp = O.ref_pack(x), O.ref_pack(w)
    assert (O.ref_unpack(xp, x.shape[1]) == x).all()
    y = O.ref_linear_ref(x, w)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        x=x.astype(np.int8), w=w.astype(np.int8), x_packed=xp, w_packed=wp, y=y)
    print(name, x.shape, w.shape, "->", y.shape)


if __name__ == "__main__":
    main()
