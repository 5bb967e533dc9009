"""B200-native MoE expert layer behind the C ABI of include/moe_layer.h."""
from .layer import MoEError, MoELayer  # noqa: F401
