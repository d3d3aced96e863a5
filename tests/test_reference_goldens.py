"""The plain implementation against what Vinci-hit/RustInfer's own CUDA kernels computed.

`tests/golden/reference_kernels.safetensors` holds small inputs and the outputs of the
reference's kernels, compiled unmodified and run on a B200 by
`tests/golden/make_reference_goldens.py`.  Every function of `plain_llama` that has such a
kernel behind it is held to those outputs here, on the CPU: how the reference pairs the
elements it rotates, which band of the llama3 scaling a frequency falls in, that the norm
weight multiplies directly, which kv head a query head reads, and how the causal mask is
aligned when a portion ends its sequence are then facts of executed reference code, not of
a reading of it.  Tolerances are the reference's own roundings (its kernels keep bf16
between steps, the plain implementation float64 throughout), stated at each comparison.
"""
import math
import os

import pytest
import torch

import plain_llama as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.safetensors")
BF_EPS = 2.0 ** -8          # one bf16 rounding: half an ulp, relative


@pytest.fixture(scope="module")
def gold():
    from safetensors import safe_open
    out = {}
    with safe_open(GOLDEN, framework="pt") as f:
        for name in f.keys():
            out[name] = f.get_tensor(name)
    return out


def maxerr(got, ref):
    return float((got.double() - ref.double()).abs().max())


@pytest.mark.parametrize("tag", ["rope_plain", "rope_llama3_a", "rope_llama3_b"])
def test_rotary_tables_and_llama3_bands(gold, tag):
    hd, theta, factor, low, high, orig = gold[tag + ".params"].tolist()
    hd = int(hd)
    scaling = None if factor == 1.0 else dict(rope_type="llama3", factor=factor, low_freq_factor=low,
                                              high_freq_factor=high, original_max_position_embeddings=orig)
    f = P.rope_inv_freq(hd, theta, scaling)
    if scaling is not None:
        plain = P.rope_inv_freq(hd, theta, None)
        changed = (f != plain)
        assert changed.any() and not changed.all()            # some frequencies kept, some scaled
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    # the reference forms pos * f in fp32 (up to 300 * 2^-24 * 300 in the angle) and stores bf16
    tol = BF_EPS + 300 * 300 * 2.0 ** -24
    assert maxerr(gold[tag + ".sin"], torch.sin(ang)) <= tol
    assert maxerr(gold[tag + ".cos"], torch.cos(ang)) <= tol


def test_rotation_pairs_i_with_i_plus_half(gold):
    q, k, pos = gold["rotate.q"], gold["rotate.k"], gold["rotate.positions"]
    T, hd = q.shape[0], 64
    f = P.rope_inv_freq(hd, 10000.0, None)
    for name, x in (("q", q), ("k", k)):
        heads = x.shape[1] // hd
        want = P.rope_rotate(x.double().view(T, heads, hd), pos.long(), f).reshape(T, -1)
        got = gold[f"rotate.{name}_out"]
        # its tables are bf16 (2^-8 on each of two products) and its output is rounded once more
        assert maxerr(got, want) <= 3 * BF_EPS * float(x.double().abs().max()) * math.sqrt(2)
    # the pairing of the reference's CPU back end (adjacent elements 2i, 2i+1) is another function
    x = q.double().view(T, -1, hd)
    ang = pos.double()[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    adjacent = torch.stack([x[..., 0::2] * c - x[..., 1::2] * s, x[..., 0::2] * s + x[..., 1::2] * c], dim=-1)
    assert maxerr(gold["rotate.q_out"], adjacent.reshape(T, -1)) > 0.5


@pytest.mark.parametrize("dim", [80, 2048])
def test_rmsnorm_alone_and_fused_with_the_residual_add(gold, dim):
    x, w, d = gold[f"rmsnorm{dim}.x"], gold[f"rmsnorm{dim}.w"], gold[f"rmsnorm{dim}.delta"]
    want = P.rmsnorm(x.double(), w.double(), 1e-5)
    scale = float(want.abs().max())
    # the kernel rounds the scale factor, x * scale, and the product with the weight to bf16
    assert maxerr(gold[f"rmsnorm{dim}.out"], want) <= 3 * BF_EPS * scale
    # fused: the sum is rounded to bf16 (that is the reference's residual stream), then normed
    summed = (x.double() + d.double()).to(torch.bfloat16)
    assert torch.equal(gold[f"rmsnorm{dim}.fused_residual"], summed)
    want = P.rmsnorm(summed.double(), w.double(), 1e-5)
    assert maxerr(gold[f"rmsnorm{dim}.fused_out"], want) <= 3 * BF_EPS * float(want.abs().max())


def test_swiglu_gate_columns_first(gold):
    gu = gold["swiglu.gate_up"].double()
    inter = gu.shape[1] // 2
    want = P.swiglu(gu[:, :inter], gu[:, inter:])
    assert maxerr(gold["swiglu.out"], want) <= 2 * BF_EPS * float(want.abs().max())


@pytest.mark.parametrize("tag,Hq,Hkv,hd", [("attn_g4_hd64", 8, 2, 64), ("attn_g3_hd128", 3, 1, 128)])
@pytest.mark.parametrize("kind", ["decode", "prefill"])
def test_paged_grouped_query_attention(gold, tag, Hq, Hkv, hd, kind):
    """An entry's queries are the last q_len positions of its kv_len keys; row t sees keys 0..t."""
    p = f"{tag}.{kind}."
    kv_lens, q_lens = gold[p + "lens"].tolist()
    q, got = gold[p + "q"].double(), gold[p + "out"].double()
    assert not torch.isnan(got).any()
    scale = 1.0 / math.sqrt(hd)
    row = 0
    for b, (n_kv, n_q) in enumerate(zip(kv_lens, q_lens)):
        k, v = gold[f"{tag}.k{b}"].double(), gold[f"{tag}.v{b}"].double()
        qfull = torch.zeros(n_kv, Hq, hd, dtype=torch.float64)
        qfull[n_kv - n_q:] = q[row: row + n_q].view(n_q, Hq, hd)
        want = P.causal_gqa_attention(qfull, k, v, scale)[n_kv - n_q:].reshape(n_q, Hq * hd)
        # probabilities rounded to bf16 before they meet the values, the output rounded once
        bound = 2.0 ** -8 * (float(want.abs().max()) + float(v.abs().max()))
        assert maxerr(got[row: row + n_q], want) <= bound, (b, n_kv, n_q)
        row += n_q
