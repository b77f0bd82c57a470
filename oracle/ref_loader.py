"""Load the unmodified reference extension modules built by oracle/build_ref.py.

TEST INFRASTRUCTURE ONLY (see chunk_attn_oracle.py).  Returns None when the build is absent.
"""
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = {}


def load_reference(kind="cpu"):
    """kind: 'cpu' (the reference's MKL path) or 'cuda' (its CUDA kernels built for sm_100a)."""
    if kind in _CACHE:
        return _CACHE[kind]
    import sysconfig
    import torch  # noqa: F401  (the extension links against libtorch)
    path = os.path.join(_HERE, "_ref", kind, "chunk_attn_c" + sysconfig.get_config_var("EXT_SUFFIX"))
    mod = None
    if os.path.exists(path):
        name = "ca_reference_%s.chunk_attn_c" % kind
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[name] = mod
    _CACHE[kind] = mod
    return mod
