"""Learned-table I/O for the packed KV cache: the FP16 table ABI and the per-layer quant
configuration file (mirror of the reference's ``beyond.quantization`` modules that feed the
encode and decode kernels)."""
