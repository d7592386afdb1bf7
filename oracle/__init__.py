"""CPU oracle for the quantized-matmul path (test infrastructure, never the product)."""
