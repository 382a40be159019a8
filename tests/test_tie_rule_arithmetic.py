"""The NVFP4 quantisers find the three values where the hardware's round-to-nearest-even e2m1 conversion differs
from the reference's rule (ties go to the smaller magnitude, examples/nvfp4_gemm.py:368-381) by arithmetic instead
of comparisons: with a = |v|, t = | |a - 1.25| - 1.375 | in fp32, one rounding per operation, and t == 0.875 is the
tie test (csrc/quant_nvfp4.cu, tie_bit).  This file restates the expression in numpy and walks every finite
non-negative fp32 value: the test is true at 0.75, 1.75 and 3.5 and nowhere else."""

from __future__ import annotations

import numpy as np


def test_the_tie_expression_singles_out_exactly_the_three_ties():
    mismatches, ties = 0, 0
    step = 1 << 21
    for start in range(0, 0x7F800000, step):
        a = np.arange(start, min(start + step, 0x7F800000), dtype=np.uint32).view(np.float32)
        t = np.abs(np.abs(a + np.float32(-1.25)) + np.float32(-1.375))
        tie = (a == np.float32(0.75)) | (a == np.float32(1.75)) | (a == np.float32(3.5))
        mismatches += int(((t == np.float32(0.875)) != tie).sum())
        ties += int(tie.sum())
    assert (mismatches, ties) == (0, 3)
