"""mlops_b200.attention: the interface of `mlops.attention` (reference: attention/python/mlops/attention/__init__.py:6-9)."""
from .fbla import FBLACache, append, decode, empty, encode, prefill

__all__ = ["FBLACache", "append", "decode", "empty", "encode", "prefill"]
