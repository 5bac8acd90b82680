"""Per-kernel micro-benchmarks and roofline helpers."""
