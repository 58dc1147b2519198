from .linear import HadamardLinear, MMFP4Linear, QuantizedLinear, Sparse24Linear, TrellisLinear

__all__ = ["HadamardLinear", "MMFP4Linear", "QuantizedLinear", "Sparse24Linear", "TrellisLinear"]
