"""Drop-in for the reference's ``import pcie_through``: importing it only loads the
operator library so that ``torch.ops.pcie_through.*`` exists
(pcieThrough/pcie_through/__init__.py:1-3, _load.py:8-11)."""
from heterofusedkernels_b200 import load_ops as _load_opextension_so

_load_opextension_so()
