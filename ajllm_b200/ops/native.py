"""ctypes binding to the in-tree sm_100a kernel library.

The library is built by ``ajllm_b200.build`` into ``ajllm_b200/_native/libajllm_b200.so`` with
``nvcc -gencode arch=compute_100a,code=sm_100a``. Kernels take raw device pointers and a CUDA stream,
so nothing here depends on torch's C++ headers. A CUDA tensor handed to an op when the library is
absent raises: there is no silent eager fallback on a GPU.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "_native"
_LIB_NAME = "libajllm_b200.so"
_lib: ctypes.CDLL | None = None
_load_error: str | None = None

c_void = ctypes.c_void_p
c_int = ctypes.c_int
c_long = ctypes.c_longlong
c_float = ctypes.c_float

# name -> argument ctypes; every entry point returns int (0 = ok)
_SIGNATURES: dict[str, list] = {
    "ajb_gemm_bf16": [c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_long,
                      c_int, c_int, c_int, c_void],
    "ajb_gemm_bf16_pair": [c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_long,
                           c_int, c_int, c_int, c_int, c_void],
    "ajb_gemm_bf16_swiglu": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_long, c_long,
                             c_int, c_void],
    "ajb_gemm_bf16_batched_swiglu": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_long, c_long, c_long, c_long,
                                     c_long, c_long, c_long, c_long, c_int, c_void, c_int, c_void],
    "ajb_gemm_pair_capacity": [],
    "ajb_gemm_skinny_pair_split": [c_int, c_int, c_int],
    "ajb_gemm_bf16_skinny_pair": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_int, c_void],
    "ajb_set_sm_budget": [c_int],
    "ajb_sm_count": [],
    "ajb_gemm_decode_cluster_slices": [c_int, c_int],
    "ajb_gemm_bf16_decode_cluster": [c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_long, c_int, c_void],
    "ajb_gemm_bf16_batched": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_long, c_long, c_long, c_long, c_long,
                              c_long, c_int, c_int, c_int, c_void, c_int, c_void],
    "ajb_gemm_bf16_splitk": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_int, c_void],
    "ajb_gemm_bf16_decode": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_int, c_void],
    "ajb_rmsnorm_fwd": [c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_float, c_void],
    "ajb_rmsnorm_bwd": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_void],
    "ajb_colsum_f32": [c_void, c_void, c_int, c_int, c_int, c_void],
    "ajb_rope_qk": [c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_long, c_int, c_void],
    "ajb_swiglu_fwd": [c_void, c_void, c_long, c_int, c_void],
    "ajb_swiglu_bwd": [c_void, c_void, c_void, c_long, c_int, c_void],
    "ajb_repack_heads": [c_void, c_void, c_long, c_int, c_int, c_int, c_long, c_long, c_void],
    "ajb_silu": [c_void, c_void, c_void, c_long, c_void],
    "ajb_ce_fwd_bwd": [c_void, c_void, c_void, c_int, c_int, c_long, c_float, c_int, c_void],
    "ajb_embedding_fwd": [c_void, c_void, c_void, c_int, c_int, c_int, c_void],
    "ajb_embedding_bwd": [c_void, c_void, c_void, c_int, c_int, c_int, c_void],
    "ajb_sumsq_f32": [c_void, c_long, c_void, c_void, c_void],  # in, n, scratch, out, stream
    "ajb_adamw_flat": [c_void, c_void, c_void, c_void, c_void, c_long, c_float, c_float, c_float, c_float,
                       c_float, c_void, c_float, c_void],
    "ajb_add_bf16": [c_void, c_void, c_void, c_long, c_void],
    "ajb_flash_fwd": [c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int, c_long, c_int, c_float, c_void],
    "ajb_fp8_quantize_rows": [c_void, c_void, c_void, c_int, c_int, c_void],
    "ajb_fp8_block_gemm": [c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_long, c_long, c_long, c_int,
                           c_void, c_void],
    "ajb_fp8_block_gemm_splits": [c_int, c_int, c_int],
    "ajb_moe_route_fwd": [c_void, c_int, c_int, c_int, c_int, c_void, c_void, c_void, c_void],
    "ajb_moe_assign_slots": [c_void, c_long, c_int, c_int, c_int, c_void, c_void, c_void],
    "ajb_sample_rows": [c_void, c_long, c_int, c_int, c_void, c_void, c_void, c_void, c_void, c_int, c_void, c_void],
    "ajb_spec_verify": [c_void, c_void, c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_void],
    "ajb_paged_attention": [c_void] * 7 + [c_int] * 8 + [c_float, c_int, c_void, c_void, c_void],
    "ajb_flash_bwd": [c_void, c_void, c_void, c_void, c_void, c_void, c_void, c_int, c_int, c_int, c_int, c_int,
                      c_long, c_int, c_float, c_void],
}


def library_path() -> Path:
    return _LIB_DIR / _LIB_NAME


def _try_load() -> None:
    global _lib, _load_error
    if _lib is not None or _load_error is not None:
        return
    path = library_path()
    if not path.is_file():
        _load_error = f"{path} has not been built (run `python -m ajllm_b200.build`)"
        return
    try:
        lib = ctypes.CDLL(str(path), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else ctypes.DEFAULT_MODE)
    except OSError as error:
        _load_error = f"could not load {path}: {error}"
        return
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.ajb_last_error.restype = ctypes.c_char_p
    lib.ajb_last_error.argtypes = []
    _lib = lib


def available() -> bool:
    _try_load()
    return _lib is not None


def lib() -> ctypes.CDLL:
    """The loaded library; raises with the reason when it cannot be used."""
    _try_load()
    if _lib is None:
        raise RuntimeError(f"ajllm_b200 native kernels are required for CUDA tensors: {_load_error}")
    return _lib


def bind(name: str, argtypes: list, restype=c_int):
    """Declare an entry point that is not in the static table (used by optional subsystems)."""
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


class PeerTimeout(RuntimeError):
    """A kernel gave up a bounded wait (on a peer GPU's flag or on one of its own barriers) and returned early."""

    def __init__(self, code: int) -> None:
        self.code, self.kernel_id, self.stage = code, (code & 0xFF) - 1, code >> 8
        names = {0: "gemm", 1: "flash forward", 2: "flash backward (dK/dV)", 3: "flash backward (dQ)", 4: "tensor-parallel gemm",
                 5: "paged attention", 6: "fp8 gemm", 7: "expert exchange", 8: "flash backward (fused)", 9: "gradient reduce-scatter", 10: "gemm (CTA pairs)", 11: "decoding gemm (cluster)"}
        super().__init__(f"kernel '{names.get(self.kernel_id, self.kernel_id)}' stopped waiting at stage {self.stage} "
                         f"(status word {code:#x}); its outputs are incomplete")


def check_status(raise_on_timeout: bool = True) -> int:
    """Synchronise the device and read (and clear) the kernels' status words: 0 when every bounded wait completed."""
    code = int(lib().ajb_check_status())
    if code > 0 and raise_on_timeout:
        raise PeerTimeout(code)
    return code


@contextlib.contextmanager
def sm_budget(sms: int | None):
    """Kernels launched by this thread inside the block size their grids for at most ``sms`` SMs (``None`` or 0: no
    change), which leaves the rest of the device to kernels running on other streams."""
    if not sms:
        yield
        return
    fn = lib().ajb_set_sm_budget
    previous = fn(int(sms))
    try:
        yield
    finally:
        fn(int(previous))


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# kernels launched per entry point (everything else launches one)
_LAUNCHES_PER_CALL = {"ajb_flash_bwd": 3, "ajb_sumsq_f32": 2, "ajb_gemm_bf16_decode": 2, "ajb_gemm_bf16_skinny_pair": 2}
launch_count = 0


def call(name: str, *args) -> None:
    global launch_count
    launch_count += _LAUNCHES_PER_CALL.get(name, 1)
    fn = getattr(lib(), name)
    status = fn(*args)
    if status != 0:
        message = lib().ajb_last_error()
        detail = message.decode("utf-8", "replace") if message else ""
        raise RuntimeError(f"{name} failed with status {status}: {detail}")
