"""The plain implementation checked against closed forms and element-by-element loops,
and the framework's host-side tables checked against it (no GPU)."""
import math

import pytest
import torch

import plain_llama as P
from helpers import TINY_A, TINY_B, TINY_C, sharp_weights
from rustinfer_b200.parts.rope import RotaryEncoding, rope_inv_freq
from rustinfer_b200.sampling.sampler import uniform_draw


def test_rope_bands_of_llama3_scaling():
    rs = TINY_B["rope_scaling"]
    f = P.rope_inv_freq(32, 500000.0, rs)
    base = [500000.0 ** (-2 * i / 32) for i in range(16)]
    orig, low, high, factor = 64.0, 1.0, 4.0, 8.0
    kinds = set()
    for i, b in enumerate(base):
        lam = 2 * math.pi / b
        if lam < orig / high:
            want, kind = b, "kept"
        elif lam > orig / low:
            want, kind = b / factor, "stretched"
        else:
            s = (orig / lam - low) / (high - low)
            want, kind = (1 - s) * b / factor + s * b, "blended"
        kinds.add(kind)
        assert f[i].item() == pytest.approx(want, rel=1e-14)
    assert kinds == {"kept", "stretched", "blended"}          # the tiny config hits all three
    assert torch.allclose(P.rope_inv_freq(16, 10000.0, None),
                          torch.tensor([10000.0 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64),
                          rtol=1e-14, atol=0)
    # incomplete or foreign scaling is ignored
    assert torch.equal(P.rope_inv_freq(32, 5e5, {"rope_type": "llama3", "factor": 8.0}),
                       P.rope_inv_freq(32, 5e5, None))


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C])
def test_framework_rope_tables_match_plain(cfg):
    hd = cfg["head_dim"]
    mine = rope_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"])
    ref = P.rope_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"])
    assert torch.allclose(torch.tensor(mine, dtype=torch.float64), ref, rtol=1e-14, atol=0)
    enc = RotaryEncoding({"head_dim": hd, "rotary_dim": hd, "theta": cfg["rope_theta"],
                          "scaling": cfg["rope_scaling"]})
    c, s = enc.tables(50)
    ang = torch.arange(50, dtype=torch.float64)[:, None] * ref[None, :]
    assert torch.allclose(c, torch.cos(ang), atol=1e-15) and torch.allclose(s, torch.sin(ang), atol=1e-15)


def test_rotation_pairs_i_with_i_plus_half():
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[0, 0, 1] = 1.0
    f = torch.tensor([0.0, 0.5, 0.0, 0.0], dtype=torch.float64)
    y = P.rope_rotate(x, torch.tensor([3]), f)
    want = torch.zeros(8, dtype=torch.float64)
    want[1], want[5] = math.cos(1.5), math.sin(1.5)
    assert torch.allclose(y[0, 0], want, atol=1e-15)
    z = torch.randn(5, 3, 16, dtype=torch.float64)
    r = P.rope_rotate(z, torch.arange(5), P.rope_inv_freq(16, 10000.0, None))
    assert torch.allclose(r.norm(dim=-1), z.norm(dim=-1)) and torch.equal(r[0], z[0])


def test_rmsnorm_and_swiglu_closed_forms():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rmsnorm(x, w, 0.5)
    inv = 1 / math.sqrt(12.5 + 0.5)
    assert torch.allclose(y, torch.tensor([[3 * 2 * inv, 4 * 0.5 * inv]], dtype=torch.float64))
    g, u = torch.tensor([1.5], dtype=torch.float64), torch.tensor([-2.0], dtype=torch.float64)
    assert P.swiglu(g, u).item() == pytest.approx(1.5 / (1 + math.exp(-1.5)) * -2.0)


def test_attention_against_loops():
    torch.manual_seed(0)
    T, Hq, Hkv, hd = 7, 6, 3, 4
    q, k, v = (torch.randn(T, h, hd, dtype=torch.float64) for h in (Hq, Hkv, Hkv))
    for window in (None, 3):
        out = P.causal_gqa_attention(q, k, v, 0.37, window)
        for t in range(T):
            for h in range(Hq):
                g = h * Hkv // Hq
                lo = 0 if window is None else max(0, t - window + 1)
                sc = [float(q[t, h] @ k[j, g]) * 0.37 for j in range(lo, t + 1)]
                m = max(sc)
                e = [math.exp(s - m) for s in sc]
                want = sum(ei / sum(e) * v[lo + j, g] for j, ei in enumerate(e))
                assert torch.allclose(out[t, h], want, atol=1e-12)


def test_logits_are_causal_and_tied_head_is_the_embedding():
    w = {k: v.double() for k, v in sharp_weights(TINY_A, 3).items()}
    ids = [5, 9, 200, 31, 7, 7]
    a = P.forward_logits(TINY_A, w, ids)
    b = P.forward_logits(TINY_A, w, ids[:4] + [100, 3])
    assert torch.equal(a[:4], b[:4]) and not torch.allclose(a[4:], b[4:])
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    assert torch.equal(P.forward_logits(TINY_A, w2, ids), a)
    with pytest.raises(ValueError):
        P.forward_logits(TINY_A, w, [256])


def test_sampler_filters_in_the_reference_order():
    row = torch.tensor([1.0, 3.0, 3.0, 2.0, -1.0])
    assert P.argmax_lowest(row) == 1
    for greedy in (dict(temperature=0.0, top_k=0, top_p=1.0), dict(temperature=1.0, top_k=1, top_p=1.0),
                   dict(temperature=1.0, top_k=0, top_p=0.0)):
        assert P.sample_filtered(row, min_p=0.0, draw=0.99, **greedy) == 1
    # order: ids 1, 2 (tie by id), 3, 0, 4; weights 1, 1, e^-1, e^-2, e^-4
    w = [1.0, 1.0, math.exp(-1), math.exp(-2), math.exp(-4)]
    order = [1, 2, 3, 0, 4]
    tot = sum(w)
    cum = 0.0
    for tok, wi in zip(order, w):
        mid = (cum + wi / 2) / tot
        assert P.sample_filtered(row, 1.0, 0, 1.0, 0.0, mid) == tok
        cum += wi
    assert P.sample_filtered(row, 1.0, 2, 1.0, 0.0, 0.999) == 2              # top-k 2
    assert P.sample_filtered(row, 1.0, 0, 1.0, 0.3, 0.999) == 3              # min-p drops e^-2, e^-4
    assert P.sample_filtered(row, 1.0, 0, 0.5, 0.0, 0.999) == 2              # top-p: 1/tot<0.5<=2/tot
    assert P.sample_filtered(row, 1.0, 0, 1e-9, 0.0, 0.999) == 1             # keeps at least one
    assert P.sample_filtered(row, 0.5, 0, 1.0, 0.0, (2 + math.exp(-2) / 2) / (2 + math.exp(-2) + math.exp(-4) + math.exp(-8))) == 3


def test_uniform_draw_depends_on_seed_and_position_only():
    a = [uniform_draw(3, p) for p in range(200)]
    assert a == [uniform_draw(3, p) for p in range(200)]
    assert all(0.0 <= u < 1.0 for u in a) and len(set(a)) == 200
    assert a != [uniform_draw(4, p) for p in range(200)]
    assert 0.35 < sum(a) / len(a) < 0.65
