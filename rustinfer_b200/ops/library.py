"""Loading the compiled kernels through ctypes and calling them on torch tensors.

The libraries export plain C functions that take device pointers, sizes and a stream.
There is no other implementation behind these wrappers: a missing library is an error.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_SIGNATURES = {
    "ri_embed_gather": [_P, _P, _I, _P, _I, _I, _I, _P],
    "ri_add_rmsnorm": [_P, _P, _P, _I, _F, _P, _I, _P, _I, _I, _P],
    "ri_residual_add": [_P, _P, _I, _L, _P],
    "ri_rope_scatter": [_P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "ri_silu_mul": [_P, _P, _I, _I, _I, _P],
    "ri_gemm_f32": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P],
    "ri_argmax": [_P, _I, _I, _I, _P, _P, _P, _P],
    "ri_decode_feedback": [_P, _P, _I, _P, _P, _I, _P, _P, _P],
    "ri_sample": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "ri_sample_by_sorting": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P],
    "ri_attention_prefill_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "ri_attention_decode_bf16": [_P, _I, _P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _L, _P, _I, _P],
    "ri_attention_mma_tokens_per_tile": [_I],
    "ri_attention_prefill_tc": [_P, _I, _P, _I, _P, _L, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P],
    "ri_attention_tc_supports": [_I, _I, _I],
    "ri_gemm_tc": [_P, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P],
    "ri_gemm_tc_rope": [_P, _P, _I, _I, _I, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P],
    "ri_decode_chain": [_P, _I, _P, _I, _P, _P, _I, _P],
    "ri_decode_chain_fits": [_P, _I, _I, _I],
    "ri_attention_plain": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
}

_CORE_SOURCES = ["elementwise.cu", "gemm_f32.cu", "sampling.cu"]
_loaded: Dict[str, ctypes.CDLL] = {}


class KernelError(RuntimeError):
    pass


def _bind(lib: ctypes.CDLL) -> ctypes.CDLL:
    for name, args in _SIGNATURES.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _I
    return lib


_pdl = os.environ.get("RUSTINFER_B200_PDL", "1") != "0"


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of this package (default on; the
    environment variable RUSTINFER_B200_PDL=0 turns it off): a kernel may start its set-up
    while its predecessor on the stream drains."""
    global _pdl
    _pdl = bool(on)
    for lib in _loaded.values():
        if hasattr(lib, "ri_set_pdl"):
            lib.ri_set_pdl(1 if _pdl else 0)


def _load(name: str, sources, defines=()) -> ctypes.CDLL:
    lib = _loaded.get(name)
    if lib is None:
        path = build.build_library(name, sources, defines)
        lib = _bind(ctypes.CDLL(path))
        if hasattr(lib, "ri_set_pdl"):
            lib.ri_set_pdl.argtypes = [_I]
            lib.ri_set_pdl.restype = None
            lib.ri_set_pdl(1 if _pdl else 0)
        _loaded[name] = lib
    return lib


def core() -> ctypes.CDLL:
    return _load("ri_core", _CORE_SOURCES)


def attention_plain(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or not 16 <= head_dim <= 512:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 up to 512, "
                          f"got {head_dim}")
    return _load(f"ri_attention_plain_hd{head_dim}", ["attention_plain.cu"], [f"RI_HEAD_DIM={head_dim}"])


def gemm_tc() -> ctypes.CDLL:
    lib = _load("ri_gemm_tc", ["gemm_tc.cu", "decode_chain.cu", "decode_chain_wide.cu"])
    kb = os.environ.get("RUSTINFER_B200_STREAM_KB")
    if kb and not getattr(lib, "_budget_set", False):
        lib.ri_gemm_tc_set_stream_budget.argtypes = [_I]
        lib.ri_gemm_tc_set_stream_budget(int(kb) * 1024)
        lib._budget_set = True
    return lib


MMA_MAX_HEAD_DIM = 256


def attention_mma(head_dim: int) -> ctypes.CDLL:
    if head_dim % 16 != 0 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        raise KernelError(f"the tensor-core attention kernels take head sizes that are multiples of 16 "
                          f"up to {MMA_MAX_HEAD_DIM}, got {head_dim}")
    name, defines = f"ri_attention_mma_hd{head_dim}", [f"RI_HEAD_DIM={head_dim}"]
    tune = os.environ.get("RUSTINFER_B200_DECODE_TUNE")       # "warps,stages": for tuning runs only
    if tune:
        w, st = tune.split(",")
        name += f"_w{w}s{st}"
        defines += [f"RI_DEC_WARPS={int(w)}", f"RI_DEC_STAGES={int(st)}"]
    lib = _load(name, ["attention_mma.cu"], defines)
    lib.ri_attention_decode_ctas_per_sm.restype = _I
    lib.ri_attention_decode_tma_ctas_per_sm.restype = _I
    lib.ri_attention_decode_tma_ctas_per_sm.argtypes = [_I]
    lib.ri_attention_decode_tile_keys.restype = _I
    return lib


def attention_tc(head_dim: int) -> ctypes.CDLL:
    """The tcgen05 attention kernel for prompt portions (head sizes 64 and 128)."""
    if head_dim not in (64, 128):
        raise KernelError(f"the tcgen05 attention kernel takes head sizes 64 and 128, got {head_dim}")
    return _load(f"ri_attention_tc_hd{head_dim}", ["attention_tc.cu"], [f"RI_HEAD_DIM={head_dim}"])


def build_all(head_dims) -> None:
    """Compile every library for the given head sizes (the ahead-of-time build check)."""
    core()
    gemm_tc()
    for hd in head_dims:
        attention_plain(hd)
        if hd <= MMA_MAX_HEAD_DIM:
            attention_mma(hd)
        if hd in (64, 128):
            attention_tc(hd)


launch_count = 0        # kernels of this package launched (or captured into a graph) so far


def check(code: int, what: str, launches: int = 1) -> None:
    global launch_count
    launch_count += launches
    if code != 0:
        lib = core()
        lib.ri_error_string.restype = ctypes.c_char_p
        lib.ri_error_string.argtypes = [_I]
        raise KernelError(f"{what}: CUDA error {code} ({lib.ri_error_string(code).decode()})")


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the sm_100a kernels take CUDA tensors only; there is no CPU path")


_sms: Dict[int, int] = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of a CUDA device (the current one by default), asked of the device."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sms.get(index)
    if n is None:
        n = _sms[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")
