"""The decode-attention entry point for callers that cannot allocate device memory.

Some users of the library may not call cudaMalloc when they call it: code that lives
inside another framework's fixed memory plan, callers in a latency-critical or
stream-ordered section where an allocation would stall the device, and embedders that reach
the library through its C symbols and have no allocator to lend.  For them
`ri_attention_decode_bf16_static` keeps the split-KV scratch in a 4 MiB array inside the
library.  This test calls it through its exported C symbol, twice in a row on different
data (the second call finds the first call's leftovers in the shared array), and holds its
output to the existing entry point's, and to a float64 statement of the same attention
from the plain implementation, within the tolerance of the kernel tests; it also checks
that a request beyond the array's size is refused with a message.

It is collected last, so that a run that stops at the first failure has run every other
test before it.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
SCRATCH_FLOATS = 1 << 20


def _case(seed, entries, Hq, Hkv, hd, page, kv_lens):
    """Single-token entries over a paged cache filled by hand (pages in shuffled order)."""
    g = torch.Generator().manual_seed(seed)
    dev = torch.device("cuda:0")
    blocks = [(n + page - 1) // page for n in kv_lens]
    n_pages = sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.full((n_pages, 2, Hkv, page, hd), float("nan"), dtype=torch.bfloat16)
    table = torch.zeros(entries, max(blocks), dtype=torch.int32)
    at = 0
    keys, values = [], []
    for b, n in enumerate(kv_lens):
        k = torch.randn(n, Hkv, hd, generator=g).bfloat16()
        v = torch.randn(n, Hkv, hd, generator=g).bfloat16()
        keys.append(k); values.append(v)
        for j in range(blocks[b]):
            pg = perm[at]; at += 1
            table[b, j] = pg
            lo, hi = j * page, min((j + 1) * page, n)
            cache[pg, 0, :, : hi - lo] = k[lo:hi].transpose(0, 1)
            cache[pg, 1, :, : hi - lo] = v[lo:hi].transpose(0, 1)
    q = torch.randn(entries, Hq * hd, generator=g).bfloat16()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    return dict(q=q.to(dev), cache=cache.to(dev), table=table.to(dev), cu_q=i32(list(range(entries + 1))),
                kv_len=i32(kv_lens), q_host=q, keys=keys, values=values)


def _float64_statement(c, Hq, hd, scale):
    """The entry's one query sees all of its keys: the last row of whole-sequence attention."""
    import plain_llama
    rows = []
    for b, (k, v) in enumerate(zip(c["keys"], c["values"])):
        qfull = torch.zeros(k.shape[0], Hq, hd, dtype=torch.float64)
        qfull[-1] = c["q_host"][b].double().view(Hq, hd)
        rows.append(plain_llama.causal_gqa_attention(qfull, k.double(), v.double(), scale)[-1].reshape(-1))
    return torch.stack(rows)


def test_static_scratch_entry_point_matches_the_allocating_one():
    from rustinfer_b200.ops import kernels as K
    from rustinfer_b200.ops import library
    Hq, Hkv, hd, page, splits = 8, 2, 64, 16, 4
    lib = ctypes.CDLL(library.attention_mma(hd)._name)
    fn = lib.ri_attention_decode_bf16_static
    fn.argtypes = [P, I, P, I, P, P, I, P, P, P, I, I, I, I, F, I, I, P]
    fn.restype = I
    err = lib.ri_attention_decode_static_error
    err.restype = ctypes.c_char_p
    scale = 1 / math.sqrt(hd)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, kv_lens) in enumerate([(1, [300, 64, 1, 129, 17]), (2, [5, 500, 63, 200, 90])]):
        c = _case(seed, len(kv_lens), Hq, Hkv, hd, page, kv_lens)
        want = torch.full_like(c["q"], float("nan"))
        no, nl = K.decode_scratch_floats(len(kv_lens), Hq, hd, splits)
        K.attention_decode_bf16(c["q"], want, c["cache"], c["table"], c["cu_q"], c["kv_len"], None, len(kv_lens),
                                Hq, Hkv, hd, scale, None, splits, torch.empty(no, device="cuda:0"),
                                torch.empty(nl, device="cuda:0"))
        got = torch.full_like(c["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        rc = fn(c["q"].data_ptr(), c["q"].stride(0), got.data_ptr(), got.stride(0), c["cache"].data_ptr(),
                c["table"].data_ptr(), c["table"].stride(0), c["cu_q"].data_ptr(), c["kv_len"].data_ptr(), None,
                len(kv_lens), Hq, Hkv, page, scale, 0, splits, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert not torch.isnan(got).any()
        scale_ref = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 2 ** -8 * scale_ref, f"call {call}"
        # and against the plain statement, by the bound the attention kernels' own tests use:
        # one rounding of the output and one of each probability, 2^-9 (max|out| + max|v|)
        ref = _float64_statement(c, Hq, hd, scale)
        vmax = max(float(v.double().abs().max()) for v in c["values"])
        bound = 2 ** -9 * (float(ref.abs().max()) + vmax)
        assert float((got.double().cpu() - ref).abs().max()) <= bound, f"call {call}"
    # beyond the array: refused, nothing launched, the reason is told
    too_many = SCRATCH_FLOATS // (Hq * 16 * (hd + 1)) + 1
    rc = fn(None, 0, None, 0, None, None, 0, None, None, None, too_many, Hq, Hkv, page, scale, 0, 16, stream)
    assert rc != 0 and b"exceed the static scratch" in err()
    torch.cuda.synchronize()
