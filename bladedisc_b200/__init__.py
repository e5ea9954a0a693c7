"""B200-native quantized-inference path of BladeDISC: int8 linear (tcgen05),
activation quantize and LayerNorm / softmax row kernels behind the RAL
custom-call C ABI (include/disc_b200_ral.h)."""

__all__ = ["lib", "ops", "ral", "quant", "host_api", "sharding", "build"]
__version__ = "0.1.0"
