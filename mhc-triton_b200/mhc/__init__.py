"""mhc: manifold-constrained hyper-connections on hand-written sm_100a CUDA kernels.

Same public surface as the reference package for the GPU path: the HyperConnection module
and the four ops.  The shared library is loaded on first use; there is no CPU path.
"""

from .module import HyperConnection
from .ops import (fused_add_residual, fused_dynamic_weights, fused_stream_mix, hyper_connection_mix,
                  sequence_mean_pool, sinkhorn_knopp)
from ._backward import get_abs_grad_at_zero, set_abs_grad_at_zero
from .host import HostStreamedStep
from .parallel import GradSync, shard_batch

__version__ = "0.1.0"
__all__ = [
    "HyperConnection",
    "sinkhorn_knopp",
    "fused_stream_mix",
    "fused_add_residual",
    "fused_dynamic_weights",
    "hyper_connection_mix",
    "sequence_mean_pool",
    "HostStreamedStep",
    "GradSync",
    "shard_batch",
    "set_abs_grad_at_zero",
    "get_abs_grad_at_zero",
]
