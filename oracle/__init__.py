"""CPU oracle for the dequant-matmul path: test infrastructure, never imported by the package."""
