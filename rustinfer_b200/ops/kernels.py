"""Typed Python fronts of the CUDA kernels.  Each checks what the kernel assumes
(device, dtype, layout, sizes) and raises instead of computing something wrong."""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Sequence

import torch

from . import library as L
from .library import KernelError, check, dtype_code, require_cuda, stream_ptr


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t,:] (fp32) = table[ids[t],:]."""
    require_cuda(ids, table, out)
    _i32(ids, "ids"); _contig(table, "table"); _contig(out, "out")
    if out.dtype != torch.float32 or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"embed_gather: out must be fp32 [{ids.numel()}, {table.shape[1]}]")
    check(L.core().ri_embed_gather(_p(ids), _p(table), dtype_code(table.dtype), _p(out),
                                   ids.numel(), table.shape[1], table.shape[0], stream_ptr()),
          "embed_gather")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h (fp32 [T,d]) += delta; out = rmsnorm(h) * weight in out's dtype.  With `rows`
    (int32 [R]) only those rows are normed into out [R,d] and h is left as it is."""
    require_cuda(h, delta, weight, out, rows)
    d = h.shape[-1]
    _contig(h, "h"); _contig(out, "out"); _contig(weight, "weight"); _i32(rows, "rows")
    if h.dtype != torch.float32:
        raise KernelError("add_rmsnorm: the residual stream is fp32")
    if weight.numel() != d:
        raise KernelError(f"add_rmsnorm: weight has {weight.numel()} elements, rows have {d}")
    n_rows = h.shape[0] if rows is None else rows.numel()
    if out.shape != (n_rows, d):
        raise KernelError(f"add_rmsnorm: out must be [{n_rows}, {d}], got {tuple(out.shape)}")
    if delta is not None:
        _contig(delta, "delta")
        if delta.shape != h.shape or delta.dtype != out.dtype:
            raise KernelError("add_rmsnorm: delta must match h's shape and out's dtype")
    check(L.core().ri_add_rmsnorm(_p(h), _p(delta), _p(weight), dtype_code(weight.dtype), float(eps),
                                  _p(out), dtype_code(out.dtype), _p(rows), n_rows, d, stream_ptr()),
          "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(h, delta)
    _contig(h, "h"); _contig(delta, "delta")
    if h.dtype != torch.float32 or h.shape != delta.shape:
        raise KernelError("residual_add: h is fp32 and delta has its shape")
    check(L.core().ri_residual_add(_p(h), _p(delta), dtype_code(delta.dtype), h.numel(), stream_ptr()),
          "residual_add")


def rope_scatter(qkv: torch.Tensor, positions: torch.Tensor, cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], slot_of_token: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                 num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int) -> None:
    """Rotate q (in place) and k of qkv [T, (Hq+2Hkv)*hd]; write k,v of token t into the
    cache [pages, 2, Hkv, page, hd] at slot_of_token[t] (page*page_size + offset; <0 skips).
    With rotary_dim 0 (cos and sin None) nothing is rotated: k and v are only written."""
    require_cuda(qkv, positions, cos, sin, slot_of_token, cache)
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token")
    T = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("rope_scatter: qkv must be [T, (Hq+2Hkv)*head_dim] with unit column stride")
    if rotary_dim % 2 or not 0 <= rotary_dim <= head_dim:
        raise KernelError(f"rope_scatter: rotary_dim {rotary_dim} must be even and at most head_dim")
    if rotary_dim and (cos is None or sin is None or cos.dtype != torch.float32 or sin.dtype != torch.float32
                       or cos.shape[1] != rotary_dim // 2):
        raise KernelError("rope_scatter: cos/sin are fp32 [positions, rotary_dim/2]")
    page = 0
    if cache is not None:
        _contig(cache, "cache")
        if cache.dtype != qkv.dtype or cache.dim() != 5 or cache.shape[1] != 2 or \
                cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
            raise KernelError("rope_scatter: cache must be [pages, 2, Hkv, page, head_dim] of qkv's dtype")
        page = cache.shape[3]
    check(L.core().ri_rope_scatter(_p(qkv), dtype_code(qkv.dtype), qkv.stride(0), _p(positions),
                                   _p(cos), _p(sin), _p(slot_of_token), _p(cache), T, num_heads,
                                   num_kv_heads if cache is not None else 0, head_dim, rotary_dim,
                                   max(page, 1), stream_ptr()), "rope_scatter")


def silu_mul(gu: torch.Tensor, out: torch.Tensor) -> None:
    require_cuda(gu, out)
    _contig(gu, "gu"); _contig(out, "out")
    T, two_i = gu.shape
    if two_i % 2 or out.shape != (T, two_i // 2) or out.dtype != gu.dtype:
        raise KernelError("silu_mul: gu is [T, 2I], out [T, I] of the same dtype")
    check(L.core().ri_silu_mul(_p(gu), _p(out), dtype_code(gu.dtype), T, two_i // 2, stream_ptr()),
          "silu_mul")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T, exact fp32."""
    require_cuda(a, w, out)
    for t, n in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_f32: {n} must be a 2-d fp32 tensor with unit column stride")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    check(L.core().ri_gemm_f32(_p(a), a.stride(0), _p(w), w.stride(0), _p(out), out.stride(0),
                               M, N, K, stream_ptr()), "gemm_f32")


# ------------------------------------------------------------ tcgen05 bf16 matrix product
EPI_BF16, EPI_F32, EPI_SILU, EPI_RESIDUAL = 0, 1, 2, 3
_tc_state = {}
_TC_WORKSPACE_FLOATS = 8 << 20
_TC_COUNTERS = 1 << 14


def gemm_tc_state(device: torch.device):
    """(workspace fp32, tile counters int32, error flag int32, meeting buffer fp32) of the
    tensor-core GEMM on a device; made once, so that captured graphs keep valid addresses.
    The meeting buffer (two 256 x 256 fp32 tiles per pair of SMs) is where CTA pairs that
    share a tile's sum over K leave their parts."""
    st = _tc_state.get(device)
    if st is None:
        st = (torch.empty(_TC_WORKSPACE_FLOATS, dtype=torch.float32, device=device),
              torch.zeros(_TC_COUNTERS, dtype=torch.int32, device=device),
              torch.zeros(1, dtype=torch.int32, device=device),
              torch.zeros(L.num_sms() * 65536, dtype=torch.float32, device=device))
        _tc_state[device] = st
    return st


def gemm_tc_error(device: torch.device) -> int:
    """The code a timed-out wait inside the tensor-core GEMM left (0: none); clears it."""
    st = _tc_state.get(device)
    if st is None:
        return 0
    code = int(st[2].item())
    if code:
        st[2].zero_()
        st[1].zero_()
    return code


def gemm_tc_plan(M: int, N: int, K: int, num_sms: Optional[int] = None, epilogue: int = EPI_BF16):
    """(swap, bn, splits, a_box): which operand sits on the 128-row side of the MMA, the
    tile of the other one, how many K slices, and how many rows of the 128 a tile really
    covers, so that about one even wave of CTAs covers the GPU."""
    num_sms = num_sms or L.num_sms()
    if M <= 64:
        swap, bn = 1, (16 if M <= 16 else 32 if M <= 32 else 64)
        tiles = -(-N // 128)
    else:
        swap, bn = 0, (256 if N >= 256 else 128 if N > 64 else 64 if N > 32 else 32 if N > 16 else 16)
        tiles = -(-M // 128) * -(-N // bn)
    kblocks = -(-K // 64)
    splits, a_box = 1, 128
    if tiles * 2 <= num_sms:
        splits = max(1, min(num_sms // tiles, kblocks // 4, 32))
        if epilogue != EPI_RESIDUAL:                       # slices meet in the workspace
            while splits > 1 and tiles * splits * bn * 128 > _TC_WORKSPACE_FLOATS:
                splits -= 1
    elif swap:
        # few tokens, no K slices: shrink the tiles until the last wave is as full as the others
        waves = -(-tiles // num_sms)
        a_box = min(128, max(64, 8 * -(-N // (8 * waves * num_sms))))
    return swap, bn, splits, a_box


def gemm_tc_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_BF16,
            plan=None, num_sms: Optional[int] = None) -> None:
    """out = x[M,K] @ w[N,K]^T on the tcgen05 tensor cores, bf16 inputs, fp32 accumulation.
    epilogue: EPI_BF16 / EPI_F32 store into out [M,N]; EPI_SILU stores silu(gate)*up into
    out [M,N/2] for a weight whose rows alternate gate_j, up_j; EPI_RESIDUAL adds into the
    fp32 out [M,N]."""
    require_cuda(x, w, out)
    if not gemm_tc_supports(x, w):
        raise KernelError("gemm_tc: contiguous, 16-byte aligned bfloat16 x [M,K] and w [N,K] with K a multiple of 8")
    M, Kd = x.shape
    N = w.shape[0]
    if w.shape[1] != Kd or out.stride(1) != 1:
        raise KernelError(f"gemm_tc: shapes x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    cols = N // 2 if epilogue == EPI_SILU else N
    want = torch.bfloat16 if epilogue in (EPI_BF16, EPI_SILU) else torch.float32
    if out.dtype != want or out.shape != (M, cols) or (epilogue == EPI_SILU and N % 2):
        raise KernelError(f"gemm_tc: out must be {want} [{M}, {cols}] for epilogue {epilogue}")
    plan = plan or gemm_tc_plan(M, N, Kd, num_sms, epilogue)
    swap, bn, splits = plan[:3]
    a_box = plan[3] if len(plan) > 3 else 128
    ws, counters, err, meeting = gemm_tc_state(x.device)
    tiles = (-(-N // a_box)) * (-(-M // bn)) if swap else (-(-M // a_box)) * (-(-N // bn))
    meets = splits > 1 and epilogue != EPI_RESIDUAL
    if tiles > counters.numel() or (meets and tiles * splits * bn * 128 > ws.numel()):
        raise KernelError("gemm_tc: the split-K workspace is too small for this plan")
    check(L.gemm_tc().ri_gemm_tc(_p(x), _p(w), M, N, Kd, _p(out), out.stride(0), epilogue, swap, bn, splits,
                                 a_box, _p(ws), _p(counters), _p(err), _p(meeting), stream_ptr()), "gemm_tc")


def gemm_tc_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                 cos: torch.Tensor, sin: torch.Tensor, slot_of_token: Optional[torch.Tensor],
                 cache: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """q, k, v = x[M,K] @ w[N,K]^T with the rotary encoding and the write of keys and values into
    their pages in the product's epilogue: q_out [M, num_heads * head_dim] bf16 gets the rotated
    queries.  `num_kv_heads` 0 (no slots, no cache) for a layer that keeps no keys.  False when the
    kernel does not take the product (fewer than 512 tokens, another head size): nothing was
    launched, and the caller runs the product and `rope_scatter` one after the other."""
    require_cuda(x, w, q_out, positions, cos, sin)
    M, Kd = x.shape
    N = w.shape[0]
    if (M < 512 or head_dim not in (64, 128) or not gemm_tc_supports(x, w) or cos.dtype != torch.float32
            or cos.shape[-1] * 2 != head_dim or q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1
            or N != (num_heads + 2 * num_kv_heads) * head_dim or N < 256):
        return False
    page = 0
    if num_kv_heads > 0:
        if slot_of_token is None or cache is None:
            raise KernelError("gemm_tc_rope: a layer with keys needs the tokens' slots and the cache")
        require_cuda(slot_of_token, cache)
        page = cache.shape[3]
    _ws, counters, err, _meet = gemm_tc_state(x.device)
    st = L.gemm_tc().ri_gemm_tc_rope(_p(x), _p(w), M, N, Kd, _p(q_out), q_out.stride(0), _p(positions), _p(cos), _p(sin),
                                     _p(slot_of_token) if num_kv_heads > 0 else None,
                                     _p(cache) if num_kv_heads > 0 else None, num_heads, num_kv_heads, head_dim,
                                     page, _p(counters), _p(err), stream_ptr())
    if st == 801:                                           # not supported for this product: nothing was launched
        return False
    check(st, "gemm_tc_rope")
    return True


class _ChainPhase(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("N", ctypes.c_int), ("K", ctypes.c_int), ("x_kind", ctypes.c_int),
                ("ld_x", ctypes.c_int), ("x_rows", ctypes.c_int), ("x", ctypes.c_void_p), ("norm_w", ctypes.c_void_p),
                ("norm_w_dtype", ctypes.c_int), ("eps", ctypes.c_float), ("out_kind", ctypes.c_int),
                ("ld_out", ctypes.c_int), ("out", ctypes.c_void_p), ("xn", ctypes.c_void_p),
                ("rowsq", ctypes.c_void_p), ("part_lse", ctypes.c_void_p), ("part_splits", ctypes.c_int),
                ("part_heads", ctypes.c_int), ("part_head_dim", ctypes.c_int)]


class _ChainRope(ctypes.Structure):
    _fields_ = [("qkv", ctypes.c_void_p), ("ld", ctypes.c_int), ("positions", ctypes.c_void_p),
                ("cos_t", ctypes.c_void_p), ("sin_t", ctypes.c_void_p), ("slot_of_token", ctypes.c_void_p),
                ("q_out", ctypes.c_void_p), ("ld_q", ctypes.c_int), ("cache", ctypes.c_void_p),
                ("Hq", ctypes.c_int), ("Hkv", ctypes.c_int), ("hd", ctypes.c_int), ("rot", ctypes.c_int),
                ("page_size", ctypes.c_int)]


CHAIN_ADD_F32, CHAIN_SILU_BF16, CHAIN_BF16 = 0, 1, 2
CHAIN_MAX_TOKENS, CHAIN_MAX_PRODUCTS = 64, 6


class ChainProduct:
    """One product of a `decode_chain`: out (+)= f(x) w^T.  `x` is a bf16 matrix [M, K], or,
    with `norm=(weight, eps)`, the fp32 stream [M, K] whose RMS norm times `weight` is the
    operand.  `out_kind`: CHAIN_ADD_F32 adds into an fp32 matrix; CHAIN_SILU_BF16 stores
    silu(gate) * up of a weight whose rows alternate gate_j, up_j into bf16 [M, N/2];
    CHAIN_BF16 stores bf16 [M, N]."""

    def __init__(self, w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, out_kind: int, norm=None,
                 x_rows: Optional[int] = None, xn: Optional[torch.Tensor] = None,
                 rowsq: Optional[torch.Tensor] = None, partials=None):
        self.w, self.x, self.out, self.out_kind, self.norm = w, x, out, out_kind, norm
        # partials = (part_o, part_lse, splits, heads, head_dim): instead of reading `x`, the product
        # merges the key ranges a split decode attention left (steps of up to 16 tokens, one token an entry)
        self.partials = partials
        if partials is not None:
            po, pl, splits, heads, hd = partials
            M = x.shape[0]
            if (norm is not None or po.dtype != torch.float32 or pl.dtype != torch.float32 or heads * hd != w.shape[1]
                    or hd % 8 or po.numel() < M * heads * splits * hd or pl.numel() < M * heads * splits
                    or po.data_ptr() % 16 or M > 16):
                raise KernelError("decode_chain: the partial attention results do not fit this product")
        # steps of more than 16 tokens with a norm: room for the normed operand, bf16 [64, K], and
        # for the rows' sums of squares, fp32 [64], zero before the first use (the kernel leaves it zero)
        self.xn, self.rowsq = xn, rowsq
        if norm is not None and xn is not None and (xn.dtype != torch.bfloat16 or tuple(xn.shape) != (CHAIN_MAX_TOKENS, w.shape[1])
                                                  or not xn.is_contiguous() or rowsq is None or rowsq.dtype != torch.float32
                                                  or rowsq.numel() != CHAIN_MAX_TOKENS):
            raise KernelError("decode_chain: the room for the normed operand does not fit")
        # rows behind x that may be read (not used): a bf16 x is fetched in boxes of 8, 16 or 32 rows
        self.x_rows = x.shape[0] if x_rows is None else x_rows
        N, Kd = w.shape
        want_x = torch.float32 if norm is not None else torch.bfloat16
        cols = N // 2 if out_kind == CHAIN_SILU_BF16 else N
        want_o = torch.float32 if out_kind == CHAIN_ADD_F32 else torch.bfloat16
        if (w.dtype != torch.bfloat16 or not w.is_contiguous() or x.dtype != want_x or x.shape[1] != Kd
                or x.stride(1) != 1 or out.dtype != want_o or out.shape[1] != cols or out.stride(1) != 1
                or x.shape[0] != out.shape[0] or (norm is not None and norm[0].numel() != Kd)):
            raise KernelError(f"decode_chain: product w{tuple(w.shape)} x{tuple(x.shape)} {x.dtype} "
                              f"out{tuple(out.shape)} {out.dtype} does not fit together")

    def fill(self, c: "_ChainPhase") -> None:
        c.w, c.N, c.K = self.w.data_ptr(), self.w.shape[0], self.w.shape[1]
        c.x, c.ld_x, c.x_kind = self.x.data_ptr(), self.x.stride(0), 1 if self.norm is not None else 0
        c.x_rows = self.x_rows
        if self.norm is not None:
            c.norm_w, c.norm_w_dtype, c.eps = self.norm[0].data_ptr(), dtype_code(self.norm[0].dtype), float(self.norm[1])
        else:
            c.norm_w, c.norm_w_dtype, c.eps = None, 0, 0.0
        c.out, c.ld_out, c.out_kind = self.out.data_ptr(), self.out.stride(0), self.out_kind
        c.xn = self.xn.data_ptr() if self.xn is not None else None
        c.rowsq = self.rowsq.data_ptr() if self.rowsq is not None else None
        if self.partials is not None:
            po, pl, splits, heads, hd = self.partials
            c.x_kind, c.x, c.part_lse = 2, po.data_ptr(), pl.data_ptr()
            c.part_splits, c.part_heads, c.part_head_dim = int(splits), int(heads), int(hd)
        else:
            c.part_lse, c.part_splits, c.part_heads, c.part_head_dim = None, 0, 0, 0


class ChainRope:
    """The tail of a chain whose last product added q, k, v rows into the fp32 matrix `qkv`
    [M, (Hq + 2 Hkv) * hd]: rotate q and k, write q (bf16) into `q_out`, k and v into the pages
    of `cache` at `slot_of_token` (-1: not written), and put `qkv` back to zero."""

    def __init__(self, qkv, positions, cos_t, sin_t, slot_of_token, q_out, cache, Hq, Hkv, hd, rot):
        self.__dict__.update(locals())
        if qkv.dtype != torch.float32 or q_out.dtype != torch.bfloat16 or qkv.shape[1] != (Hq + 2 * Hkv) * hd \
                or q_out.shape[1] != Hq * hd or (cache is not None and (cache.dtype != torch.bfloat16 or cache.dim() != 5
                                                                      or cache.shape[2] != Hkv or cache.shape[4] != hd)):
            raise KernelError("decode_chain: the rotary tail's buffers do not fit together")

    def fill(self, c: "_ChainRope") -> None:
        c.qkv, c.ld = self.qkv.data_ptr(), self.qkv.stride(0)
        c.positions, c.cos_t, c.sin_t = self.positions.data_ptr(), self.cos_t.data_ptr(), self.sin_t.data_ptr()
        c.slot_of_token = self.slot_of_token.data_ptr() if self.slot_of_token is not None else None
        c.q_out, c.ld_q = self.q_out.data_ptr(), self.q_out.stride(0)
        c.cache = self.cache.data_ptr() if self.cache is not None else None
        c.Hq, c.Hkv, c.hd, c.rot = self.Hq, self.Hkv, self.hd, self.rot
        c.page_size = self.cache.shape[3] if self.cache is not None else 1


_chain_state: Dict[torch.device, torch.Tensor] = {}


def _chain_barrier(device: torch.device) -> torch.Tensor:
    bar = _chain_state.get(device)
    if bar is None:
        bar = torch.zeros(2, dtype=torch.int32, device=device)
        _chain_state[device] = bar
    return bar


def _chain_array(products: Sequence[ChainProduct]):
    arr = (_ChainPhase * len(products))()
    for c, pr in zip(arr, products):
        pr.fill(c)
    return arr


def decode_chain_fits(products: Sequence[ChainProduct], tokens: int, num_sms: int) -> bool:
    """Whether `decode_chain` can run these products for this many tokens."""
    if not 1 <= len(products) <= CHAIN_MAX_PRODUCTS or not 1 <= tokens <= CHAIN_MAX_TOKENS:
        return False
    lib = L.gemm_tc()
    lib.ri_decode_chain_fits.restype = ctypes.c_int
    return lib.ri_decode_chain_fits(ctypes.cast(_chain_array(products), ctypes.c_void_p), len(products),
                                    tokens, num_sms) > 0


def decode_chain(products: Sequence[ChainProduct], rope: Optional[ChainRope], tokens: int, num_sms: int) -> None:
    """Run the products one after the other for the first `tokens` rows of their matrices in
    one cooperative kernel (see csrc/decode_chain.cu), then the rotary tail if given."""
    dev = products[0].w.device
    arr = _chain_array(products)
    rp = None
    if rope is not None:
        rs = _ChainRope()
        rope.fill(rs)
        rp = ctypes.cast(ctypes.pointer(rs), ctypes.c_void_p)
    err = gemm_tc_state(dev)[2]
    check(L.gemm_tc().ri_decode_chain(ctypes.cast(arr, ctypes.c_void_p), len(products), rp, tokens,
                                      _p(_chain_barrier(dev)), _p(err), num_sms, stream_ptr()), "decode_chain")


def attention_plain(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                    cu_q: torch.Tensor, kv_len: torch.Tensor, tile_entry: torch.Tensor,
                    tile_q0: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: Optional[int]) -> None:
    """q [T, >=Hq*hd] (may be a column view of the qkv buffer), out [T, Hq*hd]."""
    require_cuda(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_q0)
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len"),
                 (tile_entry, "tile_entry"), (tile_q0, "tile_q0")):
        _i32(t, n)
    if q.stride(1) != 1 or out.stride(1) != 1 or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("attention: q, out and cache share a dtype; q and out have unit column stride")
    _contig(cache, "cache")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2, Hkv, page, head_dim]")
    if num_heads % num_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")
    lib = L.attention_plain(head_dim)
    check(lib.ri_attention_plain(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache),
                                 dtype_code(cache.dtype), _p(block_table), block_table.stride(0),
                                 _p(cu_q), _p(kv_len), _p(tile_entry), _p(tile_q0), tile_entry.numel(),
                                 num_heads, num_kv_heads, cache.shape[3], float(scale),
                                 int(window) if window else 0, stream_ptr()), "attention_plain")


def _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim):
    require_cuda(q, out, cache, block_table, cu_q, kv_len)
    for t, n in ((block_table, "block_table"), (cu_q, "cu_q"), (kv_len, "kv_len")):
        _i32(t, n)
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        raise KernelError("tensor-core attention takes bfloat16 q, out and cache")
    if q.stride(1) != 1 or out.stride(1) != 1 or q.stride(0) % 8 or q.data_ptr() % 16 or out.stride(0) % 2:
        raise KernelError("tensor-core attention: q rows must be 16-byte aligned with unit column stride")
    _contig(cache, "cache")
    if cache.dim() != 5 or cache.shape[1] != 2 or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2, Hkv, page, head_dim]")
    if num_heads % num_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")


def mma_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    """Query tokens one prefill CTA of the tensor-core kernel covers for this grouping."""
    return 64 // min(num_heads // num_kv_heads, 64)


def attention_prefill_bf16(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_tok0,
                           num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           window: Optional[int]) -> None:
    """Tiles are (entry, first token) pairs of `mma_tokens_per_tile` tokens each."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(tile_entry, tile_tok0)
    _i32(tile_entry, "tile_entry"); _i32(tile_tok0, "tile_tok0")
    lib = L.attention_mma(head_dim)
    check(lib.ri_attention_prefill_bf16(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), _p(block_table),
                                        block_table.stride(0), _p(cu_q), _p(kv_len), _p(tile_entry),
                                        _p(tile_tok0), tile_entry.numel(), num_heads, num_kv_heads,
                                        cache.shape[3], float(scale), int(window) if window else 0,
                                        stream_ptr()), "attention_prefill_bf16")


def tc_attention_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this geometry."""
    if head_dim not in (64, 128):
        return False
    return bool(L.attention_tc(head_dim).ri_attention_tc_supports(num_heads, num_kv_heads, page_size))


def tc_tokens_per_tile(num_heads: int, num_kv_heads: int) -> int:
    return 128 // (num_heads // num_kv_heads)


def attention_prefill_tc(q, out, cache, block_table, cu_q, kv_len, tile_entry, tile_tok0,
                         num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int]) -> None:
    """Prompt attention on tcgen05 tensor cores with TMA page fetches.  Tiles are (entry,
    first token) pairs of `tc_tokens_per_tile` tokens each."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(tile_entry, tile_tok0)
    _i32(tile_entry, "tile_entry"); _i32(tile_tok0, "tile_tok0")
    if out.stride(0) % 8 or out.data_ptr() % 16 or cache.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: out rows and the cache must be 16-byte aligned")
    err = gemm_tc_state(q.device)[2]
    lib = L.attention_tc(head_dim)
    check(lib.ri_attention_prefill_tc(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), cache.shape[0],
                                      _p(block_table), block_table.stride(0), _p(cu_q), _p(kv_len),
                                      _p(tile_entry), _p(tile_tok0), tile_entry.numel(), num_heads,
                                      num_kv_heads, cache.shape[3], float(scale), int(window) if window else 0,
                                      _p(err), stream_ptr()), "attention_prefill_tc")


def decode_scratch_floats(entries: int, num_heads: int, head_dim: int, splits: int):
    return entries * num_heads * splits * head_dim, entries * num_heads * splits


def attention_decode_bf16(q, out, cache, block_table, cu_q, kv_len, entry_list: Optional[torch.Tensor],
                          n_entries: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                          window: Optional[int], splits: int, part_o: Optional[torch.Tensor],
                          part_lse: Optional[torch.Tensor], by_tma: bool = True, merge: bool = True) -> None:
    """Entries of one token each (entry_list: their indices, None = 0..n-1); `splits` > 1
    cuts each entry's keys into that many ranges whose partial results go through
    part_o / part_lse (fp32 scratch).  Head sizes 64 and 128 with pages of 8, 16, 32 or a
    multiple of 64 keys fetch keys and values by TMA unless `by_tma` is False.  With `merge`
    False (and several ranges) the ranges are not merged: `out` stays unwritten and the caller
    reads part_o [entries, Hq, splits, hd] and part_lse [entries, Hq, splits] itself."""
    _attention_args(q, out, cache, block_table, cu_q, kv_len, num_heads, num_kv_heads, head_dim)
    require_cuda(entry_list, part_o, part_lse)
    _i32(entry_list, "entry_list")
    if splits > 1:
        need_o, need_l = decode_scratch_floats(n_entries, num_heads, head_dim, splits)
        if part_o is None or part_lse is None or part_o.dtype != torch.float32 or \
                part_lse.dtype != torch.float32 or part_o.numel() < need_o or part_lse.numel() < need_l:
            raise KernelError(f"attention_decode: scratch must hold {need_o} and {need_l} fp32")
    lib = L.attention_mma(head_dim)
    check(lib.ri_attention_decode_bf16(_p(q), q.stride(0), _p(out), out.stride(0), _p(cache), _p(block_table),
                                       block_table.stride(0), _p(cu_q), _p(kv_len), _p(entry_list), n_entries,
                                       num_heads, num_kv_heads, cache.shape[3], float(scale),
                                       int(window) if window else 0, int(splits), _p(part_o), _p(part_lse),
                                       cache.shape[0] if by_tma else 0, _p(gemm_tc_state(q.device)[2]),
                                       1 if merge else 0, stream_ptr()), "attention_decode_bf16",
          2 if splits > 1 and merge else 1)


_argmax_state = {}


def argmax_state(device: torch.device, rows: int) -> torch.Tensor:
    """Zeroed scratch of the argmax kernel for up to `rows` rows: int64 [2 * rows], the
    merged keys followed by the arrival counters.  The kernel leaves it zero."""
    return torch.zeros(2 * rows, dtype=torch.int64, device=device)


def argmax(logits: torch.Tensor, out: torch.Tensor, state: Optional[torch.Tensor] = None) -> None:
    """out[r] = index of the largest logit of row r, the lowest index among equals."""
    require_cuda(logits, out, state)
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32:
        raise KernelError("argmax: logits fp32 [R,V], out int32 [R]")
    R = logits.shape[0]
    if state is None:
        key = (logits.device, torch.cuda.current_stream().cuda_stream)
        state = _argmax_state.get(key)
        if state is None or state.numel() < 2 * R:
            state = argmax_state(logits.device, max(R, 64))
            _argmax_state[key] = state
    if state.dtype != torch.int64 or state.numel() < 2 * R:
        raise KernelError(f"argmax: state must be int64 [{2 * R}]")
    check(L.core().ri_argmax(_p(logits), logits.stride(0), R, logits.shape[1], _p(out),
                             state.data_ptr(), state.data_ptr() + 8 * (state.numel() // 2),
                             stream_ptr()), "argmax")


def decode_feedback(sampled: torch.Tensor, state_slots: torch.Tensor, slot_state: torch.Tensor,
                    eos_ids: Optional[torch.Tensor], result: torch.Tensor,
                    token_feed: Optional[torch.Tensor]) -> None:
    """Per row of a decode step: count the chosen token in slot_state[slot] = {generated,
    max_tokens, ignore_eos, last_token}, write result = [tokens | stop flags] (int32
    [2 * rows]) and copy the token to `token_feed`, the next step's input ids."""
    require_cuda(sampled, state_slots, slot_state, eos_ids, result, token_feed)
    rows = sampled.numel()
    for t, n in ((sampled, "sampled"), (state_slots, "state_slots"), (slot_state, "slot_state"),
                 (eos_ids, "eos_ids"), (result, "result"), (token_feed, "token_feed")):
        _i32(t, n)
    if state_slots.numel() < rows or result.numel() < 2 * rows or slot_state.dim() != 2 or slot_state.shape[1] != 4 \
            or not slot_state.is_contiguous() or (token_feed is not None and token_feed.numel() < rows):
        raise KernelError("decode_feedback: sizes")
    check(L.core().ri_decode_feedback(_p(sampled), _p(state_slots), rows, _p(slot_state), _p(eos_ids),
                                      0 if eos_ids is None else eos_ids.numel(), _p(result), _p(token_feed),
                                      stream_ptr()), "decode_feedback")


def sample(logits: torch.Tensor, scratch: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, draw: torch.Tensor, out: torch.Tensor,
           by_sorting: bool = False) -> None:
    """out[r] = the token drawn for row r: logit / temperature, top-k, min-p, top-p, then the token at
    which the running weight passes draw[r] * (kept weight).  `by_sorting` runs the kernel that sorts
    every row whole (the slow statement the bucketed kernel falls back to)."""
    require_cuda(logits, scratch, temperature, top_k, top_p, min_p, draw, out)
    R, V = logits.shape
    vpad = 1 << max(1, (V - 1).bit_length())
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits fp32 [R,V]")
    if scratch.dtype != torch.int64 or scratch.numel() < R * vpad + R:
        raise KernelError(f"sample: scratch must hold {R * vpad + R} int64")
    if (temperature.dtype, top_k.dtype, top_p.dtype, min_p.dtype, draw.dtype, out.dtype) != \
            (torch.float32, torch.int32, torch.float32, torch.float32, torch.float64, torch.int32):
        raise KernelError("sample: parameter dtypes")
    fn = L.core().ri_sample_by_sorting if by_sorting else L.core().ri_sample
    check(fn(_p(logits), logits.stride(0), R, V, vpad, _p(scratch), _p(temperature),
             _p(top_k), _p(top_p), _p(min_p), _p(draw), _p(out), stream_ptr()), "sample", 1 if by_sorting else 2)


def sample_scratch_elems(rows: int, vocab: int) -> int:
    """int64 words of scratch for `rows` rows: room for the rows that are sorted whole, and a flag a row."""
    return rows * (1 << max(1, (vocab - 1).bit_length())) + rows
