"""CPU oracle for the INT4 linear GEMM -- test infrastructure, not product code."""
