"""turboquant_pro_b200 — B200-native append/encode + decode-on-codes attention for
TurboQuant Pro's compressed KV cache, behind the reference's own Python API.

Public names mirror ``turboquant_pro`` for this path: :class:`TurboQuantKVCache`,
:class:`AutoConfig`; :class:`KVContext` is the batched / multi-layer extension.
Importing the package does not touch CUDA; constructing a cache does, and raises when
the in-tree shared library or a CUDA device is missing (there is no CPU fallback).
"""

from .autoconfig import AutoConfig
from .cache import TurboQuantKVCache
from .context import KVContext, rotation_matrix, value_codebook

__version__ = "0.1.0"
__all__ = ["AutoConfig", "TurboQuantKVCache", "KVContext", "rotation_matrix", "value_codebook"]
