from .linear import HadamardLinear, MMFP4Linear, QuantizedLinear, Sparse24Linear, TrellisLinear
from .lora import LoRAMixin, apply_lora
from .blocks import MMFP4FusedMoE, MMFP4MLA, MMFP4MoE, MixedPrecisionLinear, verify_kernel


def __getattr__(name: str):
    if name in ("MMFP4MTPHead", "GLMMTPHead"):          # the multi-token-prediction head lives with the draft models
        from ..spec.draft import MTPHead
        return MTPHead
    if name == "MarlinLinear":                          # the reference's quantized linear module (an nn.Module there, a layer object here)
        from .. import compat_api
        return compat_api.MarlinLinear
    raise AttributeError(name)


__all__ = ["HadamardLinear", "MMFP4Linear", "QuantizedLinear", "Sparse24Linear", "TrellisLinear", "MMFP4FusedMoE", "MMFP4MLA", "MMFP4MoE",
           "MixedPrecisionLinear", "verify_kernel", "LoRAMixin", "apply_lora", "MMFP4MTPHead", "GLMMTPHead", "MarlinLinear"]
