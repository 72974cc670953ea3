"""Copy ops of upstream's ``nvgpu.cpasync`` namespace that the b200 backend lowers."""
from ..dsl import CopyReduceBulkTensorTileS2GOp, ReductionOp

__all__ = ["CopyReduceBulkTensorTileS2GOp", "ReductionOp"]
