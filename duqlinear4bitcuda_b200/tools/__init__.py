from .quantization import pack_i4, unpack_i4, asym_quant_dequant, sym_quant_dequant  # noqa: F401
