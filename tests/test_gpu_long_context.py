"""The bfloat16 attention kernels at the context lengths the benchmarks run: 4,096 and 32,768
keys, block tables of 256 to 2,048 pages, the numbers of key ranges the engine really picks
there, prompt portions that start deep inside a long sequence, and windows of thousands of
keys.  The float64 statement is computed row by row for sampled rows (a whole 32,768 x
32,768 score matrix per head is not needed to know one row of it)."""
import math

import pytest
import torch

from test_gpu_kernels import BF, K, PagedCase, _mma_tiles, dev

pytestmark = pytest.mark.gpu


def reference_rows(case, entry, rows, scale, window=None):
    """Attention output of the given query rows (indices among the entry's q tokens) in
    float64: the row at position p sees keys max(0, p - window + 1) .. p of its own request,
    q head h reads kv head h * Hkv // Hq, softmax of (q . k) * scale with the maximum
    subtracted (crates/infer-core/src/ports/fused_ops.rs:484-523)."""
    n_kv, n_q = case.kv_lens[entry], case.q_lens[entry]
    k, v, q = case.k[entry].double(), case.v[entry].double(), case.q[entry].double()
    G = case.Hq // case.Hkv
    out = torch.zeros(len(rows), case.Hq, case.hd, dtype=torch.float64)
    for i, r in enumerate(rows):
        p = n_kv - n_q + r
        lo = max(0, p - window + 1) if window else 0
        for g in range(case.Hkv):
            s = torch.einsum("hd,kd->hk", q[r, g * G:(g + 1) * G], k[lo: p + 1, g]) * scale
            s = s - s.max(dim=1, keepdim=True).values
            w = torch.exp(s)
            out[i, g * G:(g + 1) * G] = (w / w.sum(dim=1, keepdim=True)) @ v[lo: p + 1, g]
    return out.reshape(len(rows), case.Hq * case.hd)


def check_rows(out, case, entry, rows, scale, window=None):
    first = sum(case.q_lens[:entry])
    ref = reference_rows(case, entry, rows, scale, window)
    got = out[torch.tensor([first + r for r in rows], device=out.device)].double().cpu()
    assert not torch.isnan(got).any()
    # one rounding of the output and one of each probability (see close_attention)
    vmax = float(case.v[entry].double().abs().max())
    bound = 2 ** -9 * (float(ref.abs().max()) + vmax)
    err = float((got - ref).abs().max())
    assert err <= bound, f"entry {entry}: max err {err:.3e} vs bound {bound:.3e}"


def _mixer(Hq, Hkv, hd, page, window=None, seqs=64):
    """The attention part as the engine builds it, for the number of key ranges it picks."""
    from rustinfer_b200.parts.base import MIXERS, BuildContext
    from rustinfer_b200.parts.spec import PartSpec
    part = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": 64, "num_heads": Hq, "num_kv_heads": Hkv,
                                                   "head_dim": hd, "scale": 1 / math.sqrt(hd), "window": window,
                                                   "position": None}))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    part.prepare(BuildContext(dev(), BF, 32768, page, max_batch_seqs=seqs, num_sms=sms))
    return part


@pytest.mark.parametrize("Hq,Hkv,hd,kv_lens,window", [
    (32, 8, 64, [4096] * 8, None),                           # the headline decode step: batch 8 at 4,096
    (32, 8, 128, [4096, 4095, 4033, 3000, 4096, 1, 64, 65], None),
    (8, 2, 64, [32768, 20000, 32767], None),                 # block tables of 2,048 pages
    (8, 2, 128, [32768, 4096], None),
    (8, 2, 64, [32768, 9000, 4096], 4096),                   # windows of thousands of keys
    (8, 2, 128, [32768, 5000], 1000),
])
@pytest.mark.parametrize("by_tma", [True, False])
def test_decode_attention_at_long_contexts_with_the_engines_ranges(Hq, Hkv, hd, kv_lens, window, by_tma):
    k = K()
    page = 16
    case = PagedCase(BF, Hq, Hkv, hd, page, kv_lens, [1] * len(kv_lens), seed=hd + len(kv_lens), poison=True)
    part = _mixer(Hq, Hkv, hd, page, window)
    splits = part._splits(len(kv_lens), max(kv_lens))
    if kv_lens == [4096] * 8:
        assert 9 <= splits <= 16                             # what the benchmark's step runs with
    assert case.table.shape[1] == (max(kv_lens) + page - 1) // page
    scale = 1 / math.sqrt(hd)
    for s in sorted({splits, 16, 1}):
        out = torch.full_like(case.q_all, float("nan"))
        no, nl = k.decode_scratch_floats(len(kv_lens), Hq, hd, s)
        k.attention_decode_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, None, len(kv_lens),
                                Hq, Hkv, hd, scale, window, s, torch.full((no,), float("nan"), device=dev()),
                                torch.full((nl,), float("nan"), device=dev()), by_tma=by_tma)
        torch.cuda.synchronize()
        assert k.gemm_tc_error(dev()) == 0
        for b in range(len(kv_lens)):
            check_rows(out, case, b, [0], scale, window)


def _sampled_rows(n_q, tile):
    rows = {0, 1, n_q - 1, n_q - 2, n_q // 2}
    for edge in range(tile, n_q, max(tile, n_q // 24 // tile * tile or tile)):
        rows.update({edge - 1, edge})
    g = torch.Generator().manual_seed(n_q)
    rows.update(torch.randint(0, n_q, (40,), generator=g).tolist())
    return sorted(r for r in rows if 0 <= r < n_q)


@pytest.mark.parametrize("Hq,Hkv,hd,kv_len,q_len,window", [
    (8, 2, 64, 4096, 512, None),                             # a portion of 512 that starts at 3,584
    (8, 2, 128, 4096, 512, None),
    (4, 1, 64, 32768, 8192, None),                           # a portion of 8,192 that starts at 24,576
    (4, 1, 128, 32768, 8192, None),
    (8, 2, 64, 32768, 2048, 4096),
    (4, 1, 128, 8192, 1024, 1000),
    (6, 2, 128, 4096, 512, None),                            # groups of three
])
@pytest.mark.parametrize("kernel", ["tc", "mma"])
def test_prompt_attention_deep_inside_a_long_sequence(kernel, Hq, Hkv, hd, kv_len, q_len, window):
    k = K()
    page = 16
    if kernel == "tc" and not k.tc_attention_supports(Hq, Hkv, hd, page):
        pytest.skip("geometry not taken by the tcgen05 kernel")
    # a short neighbour in the batch, so that the long entry is not entry 0 of everything
    case = PagedCase(BF, Hq, Hkv, hd, page, [70, kv_len], [33, q_len], seed=hd + q_len, poison=True)
    out = torch.full_like(case.q_all, float("nan"))
    scale = 1 / math.sqrt(hd)
    if kernel == "tc":
        tpt = k.tc_tokens_per_tile(Hq, Hkv)
        te, tq = _mma_tiles(case, tpt, skip_decode=False)
        k.attention_prefill_tc(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                               Hq, Hkv, hd, scale, window)
    else:
        tpt = k.mma_tokens_per_tile(Hq, Hkv)
        te, tq = _mma_tiles(case, tpt, skip_decode=False)
        k.attention_prefill_bf16(case.q_all, out, case.cache, case.table, case.cu_q, case.kv_len, te, tq,
                                 Hq, Hkv, hd, scale, window)
    torch.cuda.synchronize()
    assert k.gemm_tc_error(dev()) == 0
    assert not torch.isnan(out).any()
    check_rows(out, case, 0, list(range(33)), scale, window)
    check_rows(out, case, 1, _sampled_rows(q_len, tpt), scale, window)
