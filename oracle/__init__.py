"""CPU oracle for the quantize / dequantize path.  Test infrastructure only: nothing under
``cubek_b200`` imports this package."""
