"""nn.Module layers with the reference's names (dgNN/layers/__init__.py:2-4)."""
from .edgeconv_layer import EdgeConv
from .gatconv_layer import GATConv
from .gmmconv_layer import GMMConv

__all__ = ["EdgeConv", "GATConv", "GMMConv"]
