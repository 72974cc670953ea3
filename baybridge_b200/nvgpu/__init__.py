"""``cute.nvgpu`` — the slice of upstream's NVIDIA namespace the b200 path traces (upstream ``nvgpu.py``):
``cpasync.CopyReduceBulkTensorTileS2GOp`` / ``cpasync.ReductionOp`` for reducing copies and ``tcgen05.CtaGroup``."""
from . import cpasync, tcgen05

__all__ = ["cpasync", "tcgen05"]
