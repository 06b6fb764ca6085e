"""Decoder entry points with the reference's names (sparsify/utils.py:81-103).

The reference picks between an eager `F.embedding_bag` and a Triton kernel at
import time. This package has a single backend, the CUDA embedding-bag kernel,
so every name resolves to it; there is no eager or CPU fallback.
"""

from __future__ import annotations

from torch import Tensor

from .embedding_bag import xformers_embedding_bag


def cuda_decode(top_indices: Tensor, top_acts: Tensor, W_dec: Tensor, weight_lp: Tensor | None = None):
    """`W_dec` is the [D, M] view the reference passes (`self.W_dec.mT`)."""
    return xformers_embedding_bag(top_indices, W_dec.mT, top_acts, weight_lp)


# Names the reference exports; all of them run the CUDA kernel.
triton_decode = cuda_decode
eager_decode = cuda_decode
decoder_impl = cuda_decode


def assert_type(typ, obj):
    """Assert that an object is of a given type at runtime and return it."""
    if not isinstance(obj, typ):
        raise TypeError(f"Expected {typ.__name__}, got {type(obj).__name__}")
    return obj
