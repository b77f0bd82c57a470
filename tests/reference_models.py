"""Loads the reference's OWN model layer (src/chunk_attn/models: llama_hf + ModelHost, installed unchanged into
oracle/_ref/py/models by oracle/build_ref.py) so that it runs on top of THIS repository's `chunk_attn` package:
its `import chunk_attn`, `from chunk_attn import ops`, `chunk_attn.nvtx`, `..logger` all resolve to the B200
engine.  Two things the reference's files import are not in this image and are stood in for here, in the test
only: `xformers.ops` (memory_efficient_attention with a lower-triangular mask -> torch's scaled_dot_product
attention) and, if the installed `transformers` lacks them, the handful of names the files import."""
import importlib
import importlib.util
import os
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODELS_DIR = os.path.join(ROOT, "oracle", "_ref", "py", "models")


def available():
    return os.path.isfile(os.path.join(MODELS_DIR, "llama_hf", "modeling_llama.py"))


def _xformers_stub():
    import torch
    xf = types.ModuleType("xformers")
    xops = types.ModuleType("xformers.ops")

    class LowerTriangularMask:
        pass

    def memory_efficient_attention(q, k, v, attn_bias=None):
        # q, k, v: [batch, tokens, heads, d]
        causal = isinstance(attn_bias, LowerTriangularMask)
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             dropout_p=0.0, is_causal=causal)
        return o.transpose(1, 2).contiguous()

    xops.LowerTriangularMask = LowerTriangularMask
    xops.memory_efficient_attention = memory_efficient_attention
    xf.ops = xops
    return xf, xops


def load():
    """Returns the reference's `chunk_attn.models` package, imported from its unmodified files with this
    repository's chunk_attn underneath.  Whatever cannot be imported raises ImportError naming the symbol."""
    if not available():
        raise ImportError("oracle/_ref/py/models is not installed (run oracle/build_ref.py where the reference tree is)")
    import chunk_attn  # this repository's package: Attention, ops, nvtx, logger
    if "xformers.ops" not in sys.modules:
        try:
            importlib.import_module("xformers.ops")
        except Exception:
            xf, xops = _xformers_stub()
            sys.modules["xformers"], sys.modules["xformers.ops"] = xf, xops
    for name in [m for m in sys.modules if m == "chunk_attn.models" or m.startswith("chunk_attn.models.")]:
        del sys.modules[name]      # this repository's own decoder steps aside
    spec = importlib.util.spec_from_file_location("chunk_attn.models", os.path.join(MODELS_DIR, "__init__.py"),
                                                  submodule_search_locations=[MODELS_DIR])
    pkg = importlib.util.module_from_spec(spec)
    sys.modules["chunk_attn.models"] = pkg
    try:
        spec.loader.exec_module(pkg)
    except Exception:
        for name in [m for m in sys.modules if m == "chunk_attn.models" or m.startswith("chunk_attn.models.")]:
            del sys.modules[name]
        raise
    chunk_attn.models = pkg
    return pkg


def unload():
    """Put this repository's own chunk_attn.models back."""
    import chunk_attn
    for name in [m for m in sys.modules if m == "chunk_attn.models" or m.startswith("chunk_attn.models.")]:
        del sys.modules[name]
    chunk_attn.models = importlib.import_module("chunk_attn.models")
