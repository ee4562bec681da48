"""Python modules with the names and call conventions of the reference's six
compiled extension modules (setup.py:28-35 of the reference) and of its unbuilt
single-head `sddmm` module, each a thin
wrapper over the C ABI.  `install()` registers them under their top-level
names so that `import fused_gatconv as fused_gat` (operators/fused_gatconv.py:4
of the reference) resolves to this package."""
import sys

from . import format_conversion, fused_edgeconv, fused_gatconv, fused_gmmconv, mhsddmm, mhtranspose, sddmm

_MODULES = {
    "fused_gatconv": fused_gatconv,
    "fused_gmmconv": fused_gmmconv,
    "fused_edgeconv": fused_edgeconv,
    "mhsddmm": mhsddmm,
    "mhtranspose": mhtranspose,
    "format_conversion": format_conversion,
    "sddmm": sddmm,
}


def install(overwrite: bool = False) -> None:
    """Make the six modules importable by their reference names."""
    for name, mod in _MODULES.items():
        if overwrite or name not in sys.modules:
            sys.modules[name] = mod
