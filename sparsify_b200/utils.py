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


def get_layer_list(model):
    """(name, ModuleList) of the model's layer stack (sparsify/utils.py:20-31)."""
    from torch import nn
    N = assert_type(int, model.config.num_hidden_layers)
    candidates = [
        (name, mod) for (name, mod) in model.base_model.named_modules()
        if isinstance(mod, nn.ModuleList) and len(mod) == N
    ]
    assert len(candidates) == 1, "Could not find the list of layers."
    return candidates[0]


def resolve_widths(model, module_names: list[str], dim: int = -1) -> dict[str, int]:
    """Output width of each named module, probed with the model's dummy inputs
    (sparsify/utils.py:34-61)."""
    import torch

    module_to_name = {model.base_model.get_submodule(name): name for name in module_names}
    shapes: dict[str, int] = {}

    def hook(module, _, output):
        if isinstance(output, tuple):
            output, *_ = output
        shapes[module_to_name[module]] = output.shape[dim]

    handles = [mod.register_forward_hook(hook) for mod in module_to_name]
    dummy = {k: (v.to(model.device) if hasattr(v, "to") else v) for k, v in model.dummy_inputs.items()}
    try:
        with torch.inference_mode():
            model(**dummy)
    finally:
        for handle in handles:
            handle.remove()
    return shapes
