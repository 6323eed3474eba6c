"""Loads the reference's own extension from ``oracle/_ref`` when it has been
built there (``oracle/build_ref.py``).  TEST INFRASTRUCTURE ONLY."""
import glob
import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference():
    """The module ``eppgcn_reference`` (the reference's twelve operators), or
    None when it was never built on this machine."""
    hits = glob.glob(os.path.join(_HERE, "_ref", "eppgcn_reference*.so"))
    if not hits:
        return None
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location("eppgcn_reference", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
