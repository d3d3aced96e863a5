"""Vinci-hit/RustInfer's own CUDA kernels, compiled unmodified and called through their C launchers.

RustInfer's serving path is a Rust workspace and cannot be built where there is no Rust
toolchain, but the kernels its Llama path runs are plain `.cu` files with `extern "C"`
launchers and the CuTe/CUTLASS headers vendored beside them.  `build()` compiles them with the
flags of the reference's own build script (crates/infer-backend-cuda/build.rs:148-153: `-O3 -w
-std=c++17 -arch=<detected>`, which on a B200 is `sm_100`) into `baseline/_ref/libref_kernels.so`;
nothing of the sources is changed or copied into this repository.  The wrappers below lay tensors
out the way those kernels want them and check every index on the host before a launch.

Used for two things: golden outputs that anchor the plain implementation under `tests/` on
executed reference code (`tests/golden/make_reference_goldens.py`), and the per-kernel timings
`bench.py` reports beside its own (the reference's attention kernels on the same GPU, same data).
This is not the reference arm of the benchmark: that would be RustInfer's stock serving path.

Sources (paths within the reference project):
  crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_paged_decode.cu   :479-498
  crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_paged_prefill.cu  :692-722
  crates/infer-backend-cuda/src/kernels/rmsnorm/rmsnorm.cu                          :169-181
  crates/infer-backend-cuda/src/kernels/fused_add_rmsnorm/fused_add_rmsnorm.cu
  crates/infer-backend-cuda/src/kernels/rope/rope.cu                                :135-160,288-310
  crates/infer-backend-cuda/src/kernels/swiglu/swiglu.cu                            (swiglu_packed_cu_bf16)
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
from typing import Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "libref_kernels.so")
KERNELS = "crates/infer-backend-cuda/src/kernels"
SOURCES = ["flash_attn_gqa/flash_attn_paged_decode.cu", "flash_attn_gqa/flash_attn_paged_prefill.cu",
           "rmsnorm/rmsnorm.cu", "fused_add_rmsnorm/fused_add_rmsnorm.cu", "rope/rope.cu", "swiglu/swiglu.cu"]
DECODE_MAX_SPLITS = 8           # kMaxSplits of flash_attn_paged_decode.cu:30 (sizes its workspace)
PREFILL_TILE = 128              # kBlockM of flash_attn_paged_prefill.cu:41

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def build(reference_root: str = "/root/reference", arch: str = "sm_100") -> str:
    """Compile the reference's kernels as they are.  Needs the reference tree and nvcc."""
    src = os.path.join(reference_root, KERNELS)
    if not os.path.isdir(src):
        raise FileNotFoundError(f"no reference tree at {src}")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [nvcc, "-O3", "-w", "-std=c++17", f"-arch={arch}", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(src, "third_party"), "-o", OUT] + [os.path.join(src, s) for s in SOURCES]
    print("[reference_kernels] " + " ".join(cmd), file=sys.stderr, flush=True)
    subprocess.run(cmd, check=True)
    return OUT


_lib: Optional[ctypes.CDLL] = None


def load() -> Optional[ctypes.CDLL]:
    """The compiled library, or None where it was never built."""
    global _lib
    if _lib is None and os.path.isfile(OUT):
        lib = ctypes.CDLL(OUT)
        lib.launch_flash_attn_paged_decode_bf16.argtypes = [_P, _L, _L, _P, _P, _P, _L, _L, _P, _I, _I, _P, _P,
                                                            _I, _I, _I, _I, _I, _F, _P]
        lib.launch_flash_attn_paged_decode_bf16.restype = _I
        lib.launch_flash_attn_paged_ragged_cute_bf16.argtypes = [_P, _L, _L, _P, _P, _P, _L, _L, _P, _I, _I, _P, _P,
                                                                 _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P]
        lib.launch_flash_attn_paged_ragged_cute_bf16.restype = _I
        for name in ("rustinfer_flash_attn_paged_decode_init_kernel_attributes",
                     "rustinfer_flash_attn_paged_prefill_init_kernel_attributes"):
            getattr(lib, name).argtypes = [_I]
            getattr(lib, name).restype = _I
        lib.rmsnorm_kernel_cu_bf16x8.argtypes = [_P, _P, _P, _I, _I, _I, _L, _L, _L, _L, _F, _P]
        lib.rmsnorm_kernel_cu_bf16x8.restype = None
        lib.fused_add_rmsnorm_kernel_cu_bf16.argtypes = [_P, _P, _P, _P, _I, _I, _F, _P]
        lib.fused_add_rmsnorm_kernel_cu_bf16.restype = None
        lib.rope_kernel_cu_bf16.argtypes = [_I, _I, _I, _P, _P, _P, _I, _I, _I, _P, _P, _P]
        lib.rope_kernel_cu_bf16.restype = None
        lib.sin_cos_cache_calc_cu_bf16.argtypes = [_I, _I, _F, _P, _P, _F, _F, _F, _F, _P]
        lib.sin_cos_cache_calc_cu_bf16.restype = None
        lib.swiglu_packed_cu_bf16.argtypes = [_P, _P, _I, _I, _P]
        lib.swiglu_packed_cu_bf16.restype = None
        _lib = lib
    return _lib


_configured = False


def _configure(lib) -> None:
    """The reference raises its kernels' shared-memory limits once per device, before any launch
    (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_gqa.h:33-38)."""
    global _configured
    if not _configured:
        import torch
        smem = torch.cuda.get_device_properties(0).shared_memory_per_block_optin
        for name in ("rustinfer_flash_attn_paged_decode_init_kernel_attributes",
                     "rustinfer_flash_attn_paged_prefill_init_kernel_attributes"):
            rc = getattr(lib, name)(int(smem))
            if rc != 0:
                raise RuntimeError(f"{name} returned {rc}")
        _configured = True


def _stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def _check_tables(block_tables, kv_lens: Sequence[int], block_size: int, n_blocks: int) -> None:
    """Nothing is launched with an index the kernels could not follow."""
    tables = block_tables.cpu()
    if tables.dim() != 2 or tables.shape[0] != len(kv_lens):
        raise ValueError("block_tables must be [batch, max_blocks_per_seq]")
    for b, n in enumerate(kv_lens):
        used = (int(n) + block_size - 1) // block_size
        if used > tables.shape[1]:
            raise ValueError(f"request {b}: {n} keys need {used} blocks, the table has {tables.shape[1]}")
        row = tables[b, :used]
        if used and (int(row.min()) < 0 or int(row.max()) >= n_blocks):
            raise ValueError(f"request {b}: a block id outside the pool of {n_blocks}")


def pools_from_pages(cache, block_size: int):
    """This engine's cache of one layer, [page][K|V][kv head][slot][head_dim], as the two pools the
    reference's kernels read: K and V, each [block, slot, kv head, head_dim]
    (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_paged_common.cuh:11,35)."""
    assert cache.dim() == 5 and cache.shape[1] == 2 and cache.shape[3] == block_size
    k = cache[:, 0].permute(0, 2, 1, 3).contiguous()
    v = cache[:, 1].permute(0, 2, 1, 3).contiguous()
    return k, v


def decode_workspace(batch: int, num_q_heads: int, head_dim: int):
    """fp32 partial outputs and log-sum-exps for kMaxSplits ranges, and a split count per request
    (flash_attn_paged_decode.cu:381-383)."""
    import torch
    n = batch * num_q_heads * DECODE_MAX_SPLITS * (head_dim + 1) + batch + 64
    return torch.zeros(n, dtype=torch.float32, device="cuda:0")


def paged_decode(q, k_pool, v_pool, out, block_tables, kv_lens, workspace, num_q_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, num_sm: int, kv_lens_host: Optional[Sequence[int]] = None) -> None:
    """One query token per request: q, out [batch, Hq*hd] bf16; block_tables int32 [batch, max_blocks];
    kv_lens int32 [batch].  `kv_lens_host` (the same numbers on the host) lets the index check
    run without a device read; leave it out and the check copies the tensor back."""
    lib = load()
    if lib is None:
        raise RuntimeError("the reference's kernels were not built (baseline/_ref/libref_kernels.so)")
    _configure(lib)
    import torch
    batch = q.shape[0]
    block_size = k_pool.shape[1]
    assert q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16
    assert block_tables.dtype == torch.int32 and kv_lens.dtype == torch.int32 and block_tables.is_contiguous()
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.shape == v_pool.shape
    assert tuple(k_pool.shape[2:]) == (num_kv_heads, head_dim) and q.shape[1] == num_q_heads * head_dim
    assert workspace.numel() >= batch * num_q_heads * DECODE_MAX_SPLITS * (head_dim + 1) + batch
    _check_tables(block_tables, kv_lens_host if kv_lens_host is not None else kv_lens.tolist(), block_size,
                  k_pool.shape[0])
    rc = lib.launch_flash_attn_paged_decode_bf16(
        q.data_ptr(), q.stride(0), head_dim, k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), out.stride(0),
        head_dim, block_tables.data_ptr(), block_tables.shape[1], block_size, kv_lens.data_ptr(),
        workspace.data_ptr(), batch, num_q_heads, num_kv_heads, num_sm, head_dim, float(scale), _stream())
    if rc != 0:
        raise RuntimeError(f"launch_flash_attn_paged_decode_bf16 returned {rc}")


def prefill_tiles(q_lens: Sequence[int]):
    """(block2req, block2tile, valid_q_tiles) for query tiles of 128 tokens
    (crates/infer-backend-cuda/src/kernels/flash_attn_gqa/flash_attn_gqa.h:73-80)."""
    import torch
    req, tile = [], []
    for b, n in enumerate(q_lens):
        for t in range((int(n) + PREFILL_TILE - 1) // PREFILL_TILE):
            req.append(b); tile.append(t)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda:0")
    return i32(req), i32(tile), i32([len(req)])


def paged_prefill(q, k_pool, v_pool, out, block_tables, kv_lens, cu_q_lens, tiles, q_lens_host: Sequence[int],
                  kv_lens_host: Sequence[int], num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float) -> None:
    """Ragged causal attention of prompt portions: q, out [tokens, Hq*hd] bf16, an entry's queries
    being the last q_len positions of its kv_len keys."""
    lib = load()
    if lib is None:
        raise RuntimeError("the reference's kernels were not built (baseline/_ref/libref_kernels.so)")
    _configure(lib)
    import torch
    block_size = k_pool.shape[1]
    assert q.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and block_tables.dtype == torch.int32
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and block_tables.is_contiguous()
    assert q.shape[0] == sum(int(n) for n in q_lens_host) and len(q_lens_host) == len(kv_lens_host)
    assert all(0 < int(a) <= int(b) for a, b in zip(q_lens_host, kv_lens_host))
    _check_tables(block_tables, kv_lens_host, block_size, k_pool.shape[0])
    block2req, block2tile, valid = tiles
    rc = lib.launch_flash_attn_paged_ragged_cute_bf16(
        q.data_ptr(), q.stride(0), head_dim, k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), out.stride(0),
        head_dim, block_tables.data_ptr(), block_tables.shape[1], block_size, kv_lens.data_ptr(),
        cu_q_lens.data_ptr(), block2req.data_ptr(), block2tile.data_ptr(), valid.data_ptr(), block2req.numel(),
        len(q_lens_host), q.shape[0], num_q_heads, num_kv_heads, head_dim, float(scale), 1, _stream())
    if rc != 0:
        raise RuntimeError(f"launch_flash_attn_paged_ragged_cute_bf16 returned {rc}")


def rmsnorm(x, weight, eps: float):
    """bf16 [rows, dim] -> bf16 (dim a multiple of 8)."""
    import torch
    lib = load()
    out = torch.empty_like(x)
    rows, dim = x.shape
    assert x.dtype == weight.dtype == torch.bfloat16 and dim % 8 == 0 and x.is_contiguous()
    lib.rmsnorm_kernel_cu_bf16x8(out.data_ptr(), x.data_ptr(), weight.data_ptr(), rows, 1, dim, dim, dim, dim, dim,
                                 float(eps), _stream())
    return out


def fused_add_rmsnorm(residual, delta, weight, eps: float):
    """residual += delta (kept in bf16, as the reference keeps its stream); returns the norm of the sum."""
    import torch
    lib = load()
    rows, dim = residual.shape
    assert residual.dtype == delta.dtype == weight.dtype == torch.bfloat16 and residual.is_contiguous()
    out = torch.empty_like(residual)
    lib.fused_add_rmsnorm_kernel_cu_bf16(out.data_ptr(), residual.data_ptr(), delta.data_ptr(), weight.data_ptr(),
                                         rows, dim, float(eps), _stream())
    return out


def rope_tables(head_dim: int, positions: int, theta: float, factor: float, low: float, high: float, orig: float):
    """(sin, cos) bf16 [positions, head_dim/2] from the reference's device table kernel, llama3
    scaling included (rope.cu:288-310; factor 1 with low == high leaves the frequencies alone)."""
    import torch
    lib = load()
    sin = torch.zeros(positions, head_dim // 2, dtype=torch.bfloat16, device="cuda:0")
    cos = torch.zeros_like(sin)
    lib.sin_cos_cache_calc_cu_bf16(head_dim, positions, float(theta), sin.data_ptr(), cos.data_ptr(), float(factor),
                                   float(low), float(high), float(orig), _stream())
    return sin, cos


def rope(q, k, positions, sin, cos, head_dim: int) -> None:
    """Rotate q [T, Hq*hd] and k [T, Hkv*hd] in place, pair (i, i + hd/2) (rope.cu:84-132)."""
    import torch
    lib = load()
    assert q.dtype == k.dtype == sin.dtype == torch.bfloat16 and positions.dtype == torch.int32
    assert int(positions.max()) < sin.shape[0] and int(positions.min()) >= 0
    lib.rope_kernel_cu_bf16(q.shape[1], k.shape[1], head_dim, q.data_ptr(), k.data_ptr(), positions.data_ptr(),
                            q.shape[0], q.stride(0), k.stride(0), sin.data_ptr(), cos.data_ptr(), _stream())


def swiglu_packed(gate_up):
    """[rows, 2*inter] bf16 with gate columns first -> silu(gate) * up, [rows, inter]."""
    import torch
    lib = load()
    rows, two = gate_up.shape
    assert gate_up.dtype == torch.bfloat16 and gate_up.is_contiguous() and (two // 2) % 8 == 0
    out = torch.empty(rows, two // 2, dtype=torch.bfloat16, device=gate_up.device)
    lib.swiglu_packed_cu_bf16(gate_up.data_ptr(), out.data_ptr(), rows, two // 2, _stream())
    return out


if __name__ == "__main__":
    print(build(*sys.argv[1:]))
