"""ctypes binding of libsparsecoder.so (the C ABI declared in include/sparsecoder.h).

The library is mandatory: there is no CPU or eager fallback. ``lib()`` raises if
the shared object has not been built (``python -m sparsify_b200.build``).
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libsparsecoder.so"

SC_OK = 0
SC_ERR_TIMEOUT = 5
SC_F32, SC_BF16 = 0, 1
STATUS_NAMES = {
    0: "SC_OK",
    1: "SC_ERR_INVALID",
    2: "SC_ERR_UNSUPPORTED",
    3: "SC_ERR_WORKSPACE",
    4: "SC_ERR_CUDA",
    5: "SC_ERR_TIMEOUT",
    6: "SC_ERR_TOO_LARGE",
}

P = c_void_p
I64 = c_int64

# name -> (restype, argtypes); mirrors include/sparsecoder.h one to one.
SIGNATURES: dict[str, tuple] = {
    "sc_version": (c_int, []),
    "sc_set_reserved_sms": (c_int, [c_int]),
    "sc_set_cta_pairs": (c_int, [c_int]),
    "sc_last_error": (c_size_t, [c_char_p, c_size_t]),
    "sc_status_string": (c_char_p, [c_int]),
    "sc_selftest_wait_timeout": (c_int, [P, I64, P]),
    "sc_prep_input": (c_int, [P, c_int, P, I64, I64, P, c_int, P]),
    "sc_preacts_dense": (c_int, [P, c_int, P, c_int, P, I64, I64, I64, P, c_int, P]),
    "sc_topk_rows": (c_int, [P, I64, I64, c_int, P, P, P, P]),
    "sc_topk_mask_rows": (c_int, [P, I64, I64, c_int, P, P, P]),
    "sc_groupmax_rows": (c_int, [P, I64, I64, c_int, P, P, P]),
    "sc_encode_topk_workspace_bytes": (c_size_t, [I64, I64, I64, c_int]),
    "sc_encode_topk": (c_int, [P, P, P, I64, I64, I64, c_int, P, P, P, c_size_t, P, P]),
    "sc_encode_groupmax": (c_int, [P, P, P, I64, I64, I64, c_int, P, P, P, P]),
    "sc_embedding_bag_fwd": (c_int, [P, P, P, c_int, P, I64, I64, I64, c_int, P, P]),
    "sc_embedding_bag_bwd_acts": (c_int, [P, P, c_int, P, c_int, I64, I64, I64, c_int, P, P]),
    "sc_decode_residual_workspace_bytes": (c_size_t, [I64]),
    "sc_decode_residual": (
        c_int,
        [P, P, P, c_int, P, P, c_int, I64, I64, I64, c_int, P, P, P, P, P, c_size_t, P],
    ),
    "sc_decode_residual_dots": (
        c_int,
        [P, P, P, c_int, P, P, c_int, I64, I64, I64, c_int, P, P, P, P, P, P, c_size_t, P],
    ),
    "sc_csr_workspace_bytes": (c_size_t, [I64]),
    "sc_csr_build": (c_int, [P, I64, c_int, I64, P, P, P, c_size_t, P]),
    "sc_csr_build_noalloc": (c_int, [P, I64, c_int, I64, P, P, P]),
    "sc_rows_accumulate": (
        c_int,
        [P, P, c_int, P, P, c_int, P, P, P, P, c_int, P, P, I64, I64, I64, I64, P],
    ),
    "sc_loss_workspace_bytes": (c_size_t, [I64]),
    "sc_total_variance": (c_int, [P, c_int, I64, I64, P, P, c_size_t, P]),
    "sc_sq_err": (c_int, [P, P, I64, P, P, P, c_size_t, P]),
    "sc_weighted_colsum": (c_int, [P, c_int, P, I64, I64, P, P, c_size_t, P]),
    "sc_normalize_rows": (c_int, [P, I64, I64, c_float, P, P]),
    "sc_adam_rows": (
        c_int,
        [P, P, P, P, I64, I64, c_float, c_float, c_float, c_float, I64, c_int, P, P],
    ),
    "sc_cast_bf16": (c_int, [P, P, I64, P]),
    "sc_muon_workspace_bytes": (c_size_t, []),
    "sc_muon_momentum": (c_int, [P, P, I64, c_float, c_int, P, P, P, c_size_t, P]),
    "sc_scale_transpose_bf16": (c_int, [P, I64, I64, P, P, P, P]),
    "sc_muon_apply": (c_int, [P, P, I64, c_float, c_float, P, P]),
    "sc_project_rows": (c_int, [P, P, I64, I64, P]),
    "sc_signum_schedulefree": (c_int, [P, P, P, I64, c_float, c_float, c_float, P, P]),
    "sc_gemm_bf16_nt": (c_int, [P, P, I64, I64, I64, c_float, c_float, P, c_int, P, c_int, P, c_int, c_int, P, P, P]),
    "sc_transpose_bf16": (c_int, [P, I64, I64, P, P]),
    "sc_csr_segment_sum": (c_int, [P, P, P, I64, P, P]),
    "sc_rows_adam": (
        c_int,
        [P, P, c_int, P, P, c_int, P, P, c_int, I64, I64, P, P, P, P, c_int, c_int, c_float, P,
         P, P, P, P, P, P, P, c_int, c_int, P],
    ),
}

class AdamHparams(ctypes.Structure):
    """Mirror of sc_adam_hparams."""
    _fields_ = [("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float),
                ("step", c_int64)]


_lib = None


class SparseCoderLibError(RuntimeError):
    """A libsparsecoder entry point returned a non-zero status."""

    def __init__(self, fn: str, status: int, message: str):
        self.fn, self.status, self.message = fn, status, message
        super().__init__(f"{fn} -> {STATUS_NAMES.get(status, status)}: {message}")


def lib() -> ctypes.CDLL:
    """Loads the kernel library once and declares every prototype."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m sparsify_b200.build`. "
                "sparsify_b200 has no CPU or eager fallback."
            )
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    lib().sc_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def call(name: str, *args):
    """Calls an int-status entry point and raises SparseCoderLibError on failure."""
    status = getattr(lib(), name)(*args)
    if status != SC_OK:
        raise SparseCoderLibError(name, status, last_error())


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return SC_F32
    if t.dtype == torch.bfloat16:
        return SC_BF16
    raise TypeError(f"unsupported dtype {t.dtype}; expected float32 or bfloat16")


def ptr(t: torch.Tensor | None):
    """Device pointer of a contiguous CUDA tensor (None -> NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(
            "sparsify_b200 kernels need CUDA tensors; there is no CPU path "
            f"(got a tensor on {t.device})"
        )
    if not t.is_contiguous():
        raise RuntimeError("sparsify_b200 kernels need contiguous tensors")
    return t.data_ptr()


def stream_ptr(device: torch.device | None = None):
    return torch.cuda.current_stream(device).cuda_stream
