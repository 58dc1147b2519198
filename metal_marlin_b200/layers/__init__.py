from .linear import HadamardLinear, MMFP4Linear, QuantizedLinear, Sparse24Linear, TrellisLinear
from .blocks import MMFP4FusedMoE, MMFP4MLA, MMFP4MoE, MixedPrecisionLinear, verify_kernel


def __getattr__(name: str):
    if name in ("MMFP4MTPHead", "GLMMTPHead"):          # the multi-token-prediction head lives with the draft models
        from ..spec.draft import MTPHead
        return MTPHead
    raise AttributeError(name)


__all__ = ["HadamardLinear", "MMFP4Linear", "QuantizedLinear", "Sparse24Linear", "TrellisLinear", "MMFP4FusedMoE", "MMFP4MLA", "MMFP4MoE",
           "MixedPrecisionLinear", "verify_kernel", "MMFP4MTPHead", "GLMMTPHead"]
