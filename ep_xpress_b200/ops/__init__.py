"""Hand-written device operators exposed to users of a context."""

from .expert import scale_rows  # noqa: F401
from .moe import GroupedSwiGLU, swiglu_reference  # noqa: F401
