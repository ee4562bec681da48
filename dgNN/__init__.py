"""Alias package: `import dgNN`, `dgNN.layers`, `dgNN.operators` (and the
operator sub-modules such as dgNN.operators.fused_gatconv) resolve to dgnn_b200,
and the six extension-module names of the reference (fused_gatconv, mhsddmm, ...)
become importable."""
import sys

import dgnn_b200
from dgnn_b200 import ext as _ext
from dgnn_b200 import layers, operators  # noqa: F401
from dgnn_b200.layers import *  # noqa: F401,F403
from dgnn_b200.operators import *  # noqa: F401,F403

_ext.install()
for _name in ("layers", "operators", "layers.gatconv_layer", "layers.gmmconv_layer", "layers.edgeconv_layer",
              "operators.fused_gatconv", "operators.fused_gmmconv", "operators.fused_edgeconv",
              "operators.tile_balance_scheduler"):
    __import__("dgnn_b200." + _name)
    sys.modules["dgNN." + _name] = sys.modules["dgnn_b200." + _name]
