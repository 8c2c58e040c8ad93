"""Precision names <-> torch dtypes (reference: axon/utils/torch/dtypes.py ``PrecisionType``)."""
import torch

_GROUPS = {
    torch.float16: (16, "16", "fp16", "float16", "half", torch.float16),
    torch.float32: (32, "32", "fp32", "float32", "float", torch.float32),
    torch.bfloat16: ("bf16", "bfloat16", torch.bfloat16),
    torch.float64: (64, "64", "fp64", "float64", "double", torch.float64),
}
HALF_LIST, FLOAT_LIST, BFLOAT_LIST = list(_GROUPS[torch.float16]), list(_GROUPS[torch.float32]), list(_GROUPS[torch.bfloat16])


class PrecisionType:
    HALF, FLOAT, FULL, BFLOAT, MIXED = "16", "32", "64", "bf16", "mixed"

    @staticmethod
    def supported_types() -> list[str]:
        return [PrecisionType.HALF, PrecisionType.FLOAT, PrecisionType.FULL, PrecisionType.BFLOAT, PrecisionType.MIXED]

    @staticmethod
    def supported_type(precision) -> bool:
        return str(precision) in PrecisionType.supported_types()

    @staticmethod
    def _is(precision, dtype) -> bool:
        return any(precision is x or (not isinstance(x, torch.dtype) and not isinstance(precision, torch.dtype) and precision == x)
                   for x in _GROUPS[dtype])

    @staticmethod
    def is_fp16(precision) -> bool:
        return PrecisionType._is(precision, torch.float16)

    @staticmethod
    def is_fp32(precision) -> bool:
        return PrecisionType._is(precision, torch.float32)

    @staticmethod
    def is_bf16(precision) -> bool:
        return PrecisionType._is(precision, torch.bfloat16)

    @staticmethod
    def to_dtype(precision) -> torch.dtype:
        for dtype in _GROUPS:
            if PrecisionType._is(precision, dtype):
                return dtype
        raise RuntimeError(f"unexpected precision: {precision}")

    @staticmethod
    def to_str(precision) -> str:
        names = {torch.float16: "fp16", torch.float32: "fp32", torch.bfloat16: "bf16", torch.float64: "fp64"}
        if precision in names:
            return names[precision]
        raise RuntimeError(f"unexpected precision: {precision}")
