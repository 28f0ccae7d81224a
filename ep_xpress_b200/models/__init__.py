"""Model-level building blocks driven through the public context API."""

from .synthetic import IdentityMoELayer  # noqa: F401
from .moe_layer import SwiGLUMoELayer  # noqa: F401
