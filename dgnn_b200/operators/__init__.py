"""Autograd operators with the reference's names (dgNN/operators/__init__.py:2-4)."""
from .fused_edgeconv import EdgeConvFuse
from .fused_gatconv import GATConvFuse, GATConvFuse_inference, GATLayerFuse
from .fused_gmmconv import GmmConvFuse
from .projection import project
from .tile_balance_scheduler import TileBalanceScheduler

__all__ = ["EdgeConvFuse", "GATConvFuse", "GATConvFuse_inference", "GATLayerFuse", "GmmConvFuse", "TileBalanceScheduler", "project"]
