"""chunk_attn — B200-native drop-in for the reference package of the same name.

`from chunk_attn import Attention` gives the prefix-aware KV cache with two-phase decode
attention, same constructor and methods as the reference's (src/chunk_attn/__init__.py:15-16
re-exports its compiled module the same way).  The compiled module needs a CUDA device to
construct an `Attention`; there is no CPU implementation and no fallback.
"""
__version__ = "1.0.0b200"

import torch  # noqa: F401  (libtorch must be loaded before the extension)

from .lib.chunk_attn_c import *  # noqa: F401,F403
from .lib.chunk_attn_c import Attention, Chunk, PrefixTree, ops  # noqa: F401
