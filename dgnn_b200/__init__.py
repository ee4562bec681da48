"""dgnn_b200: B200 (sm_100a) kernels behind the dgNN operator / layer API.

    from dgnn_b200.layers import GATConv, GMMConv, EdgeConv
    from dgnn_b200.operators import GATConvFuse, GmmConvFuse, EdgeConvFuse

`import dgNN` (the alias package at the repository root) exposes the same
objects under the reference's package name.  The compiled library is loaded on
first use; there is no CPU fallback.
"""
from . import ext, kernels, layers, operators  # noqa: F401
from .layers import EdgeConv, GATConv, GMMConv  # noqa: F401
from .operators import EdgeConvFuse, GATConvFuse, GATConvFuse_inference, GmmConvFuse  # noqa: F401

__version__ = "0.1.0"
