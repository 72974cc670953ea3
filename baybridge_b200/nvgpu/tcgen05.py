"""``nvgpu.tcgen05.CtaGroup`` as upstream records it on copy ops."""
from ..dsl import CtaGroup

__all__ = ["CtaGroup"]
