"""B200-native fused linear + cross-entropy loss.

Same public names as ``linear_cross_entropy`` (the reference package, __init__.py:1):
``LinearCrossEntropyLoss``, ``linear_cross_entropy``, ``fwd_configs``, ``bwd_configs``.
"""
from .ops import (  # noqa: F401
    LinearCrossEntropyLoss,
    LinearXentImplementation,
    bwd_configs,
    fwd_configs,
    linear_cross_entropy,
    set_autocast_policy,
)

__all__ = ["LinearCrossEntropyLoss", "linear_cross_entropy", "fwd_configs", "bwd_configs", "set_autocast_policy"]
