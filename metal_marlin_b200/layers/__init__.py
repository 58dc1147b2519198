from .linear import HadamardLinear, MMFP4Linear, QuantizedLinear, TrellisLinear

__all__ = ["HadamardLinear", "MMFP4Linear", "QuantizedLinear", "TrellisLinear"]
