"""eppgcn_b200 -- B200 (sm_100a) implementation of EPPGCN's GCN aggregation
hot path behind the reference's ``GNNAdvisor`` operator API.

``eppgcn_b200.GNNAdvisor``   the operator module (C++/CUDA, built in-tree)
``eppgcn_b200.gcn_conv``     GNNAFunction / GCNConv (autograd boundary)
``eppgcn_b200.param``        inputProperty / maskInputProperty / backInputProperty
``eppgcn_b200.capi``         ctypes view of the C-ABI library
``eppgcn_b200.graphs``       seeded synthetic workloads
"""
import importlib
import sys

__version__ = "0.1.0"


def load_gnnadvisor():
    """Imports the native operator module; raises if it has not been built
    (there is no Python or CPU fallback)."""
    try:
        return importlib.import_module("eppgcn_b200.GNNAdvisor")
    except ImportError as exc:
        raise ImportError(
            "eppgcn_b200.GNNAdvisor is not built: run `python -m eppgcn_b200.build`") from exc


def install_as_gnnadvisor():
    """Registers the native module under the top-level name ``GNNAdvisor`` so
    that code written against the reference (``import GNNAdvisor as GNNA``)
    runs unchanged."""
    mod = load_gnnadvisor()
    sys.modules.setdefault("GNNAdvisor", mod)
    return mod
