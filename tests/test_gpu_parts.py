"""Each part of the decoder alone against the plain implementation, and a toy mixer with
state of its own that is registered, built and stepped from this file alone."""
import json
import math
import os

import pytest
import torch

import plain_llama as P
from helpers import rel_err

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over logits.  fp32: sums of a few hundred fp32 products
# against float64.  bf16: the same bound as the replay tests use (see the measured spread there);
# on these toy models with weights of 0.2 one cut lands at 3.5e-2 and another at 4.0e-2 depending
# only on which kernels round q and k (the chain rounds them once, from fp32).
LOGITS_TOL = {"float32": 2e-5, "bfloat16": 6e-2}


DT = [torch.float32, torch.bfloat16]
TOLP = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def dev():
    return torch.device("cuda:0")


def ctx(dtype, max_len=256, page=8):
    from rustinfer_b200.parts.base import BuildContext
    return BuildContext(dev(), dtype, max_len, page)


def one_sequence_step(T, page, n_groups=1, needs=()):
    """A StepContext for one whole sequence of T tokens laid out in pages 3, 4, 5, ..., with
    the index arrays the part under test declares (`needs`: its step_indices())."""
    import numpy as np
    from rustinfer_b200.parts.base import GroupStep, HostEntry, StepContext, StepShape
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    blocks = (T + page - 1) // page
    table = i32([[3 + b for b in range(blocks)]])
    slot = i32([(3 + t // page) * page + t % page for t in range(T)])
    a64 = lambda x: np.asarray(x, dtype=np.int64)
    shape = StepShape(a64([T]), a64([0]), a64([0, T]), a64([T]), a64([0]))
    indices = {n.key: tuple(i32(arr.tolist()) for arr in n.build(shape)) for n in needs}
    return StepContext(num_tokens=T, num_entries=1, token_ids=i32([0] * T), positions=i32(list(range(T))),
                       cu_q=i32([0, T]), kv_len=i32([T]), state_slots=i32([0]),
                       groups=[GroupStep(table, slot) for _ in range(n_groups)],
                       entries=[HostEntry("x", 0, T, 0)], max_q_len=T, max_kv_len=T, decode_only=False,
                       indices=indices)


@pytest.mark.parametrize("dt", DT)
def test_rmsnorm_part(dt):
    from rustinfer_b200.parts.base import NORMS
    from rustinfer_b200.parts.spec import PartSpec
    torch.manual_seed(0)
    part = NORMS.build(PartSpec("rmsnorm", {"size": 104, "eps": 2e-6}))
    assert {n: d.shape for n, d in part.param_decls().items()} == {"weight": (104,)}
    part.prepare(ctx(dt))
    w = (1 + 0.2 * torch.randn(104)).to(dt)
    part.load({"weight": w.to(dev())})
    h = torch.randn(9, 104, device=dev())
    delta = torch.randn(9, 104).to(dt).to(dev())
    want_h = h.double().cpu() + delta.double().cpu()
    out = part.add_norm(h, delta)
    assert out.dtype == dt
    assert rel_err(out, P.rmsnorm(want_h, w.double(), 2e-6)) <= TOLP[dt]
    assert rel_err(h, want_h) <= 1e-6


@pytest.mark.parametrize("dt", DT)
def test_swiglu_part(dt):
    from rustinfer_b200.parts.base import FEED_FORWARDS
    from rustinfer_b200.parts.spec import PartSpec
    torch.manual_seed(1)
    d, inter = 80, 104
    part = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": d, "intermediate_size": inter}))
    assert {n: v.shape for n, v in part.param_decls().items()} == {
        "gate_proj.weight": (inter, d), "up_proj.weight": (inter, d), "down_proj.weight": (d, inter)}
    part.prepare(ctx(dt))
    w = {n: (torch.randn(v.shape) / math.sqrt(v.shape[1])).to(dt) for n, v in part.param_decls().items()}
    part.load({n: t.to(dev()) for n, t in w.items()})
    x = torch.randn(13, d).to(dt)
    y = part.forward(x.to(dev()), None)
    xd = x.double()
    m = P.swiglu(xd @ w["gate_proj.weight"].double().T, xd @ w["up_proj.weight"].double().T)
    assert rel_err(y, m @ w["down_proj.weight"].double().T) <= TOLP[dt]


def test_linear_keeps_32_bit_weights_in_a_bfloat16_engine():
    from rustinfer_b200.parts.linear import Linear
    torch.manual_seed(2)
    w = torch.randn(37, 96)
    x = torch.randn(5, 96).bfloat16()
    ref = x.double() @ w.double().T
    y32 = Linear(w.to(dev()))(x.to(dev()), out_dtype=torch.float32)
    # exact in the weight: only x was rounded (it is the same x), so the error is fp32-sized
    assert rel_err(y32, ref) <= 1e-6
    ybf = Linear(w.bfloat16().to(dev()))(x.to(dev()), out_dtype=torch.float32)
    assert 1e-4 < rel_err(ybf, ref) <= 2e-2               # rounding the weight shows
    assert Linear(w.to(dev()))(x.to(dev())).dtype == torch.bfloat16


def test_rotary_part_tables_on_the_device():
    from rustinfer_b200.parts.base import POSITIONS
    from rustinfer_b200.parts.spec import PartSpec
    scaling = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                   original_max_position_embeddings=64)
    part = POSITIONS.build(PartSpec("rope", {"head_dim": 32, "rotary_dim": 32, "theta": 5e5, "scaling": scaling}))
    part.prepare(ctx(torch.bfloat16, max_len=300))
    assert part.cos.dtype == torch.float32 and part.cos.shape == (300, 16)      # fp32 whatever the engine
    f = P.rope_inv_freq(32, 5e5, scaling)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert float((part.cos.double().cpu() - torch.cos(ang)).abs().max()) <= 2 ** -24
    assert float((part.sin.double().cpu() - torch.sin(ang)).abs().max()) <= 2 ** -24


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("Hq,Hkv,hd,window", [(6, 3, 48, None), (4, 1, 32, None), (4, 2, 16, 11)])
def test_attention_part(dt, Hq, Hkv, hd, window):
    from rustinfer_b200.parts.base import MIXERS, PagedKV, PagedLayerCache
    from rustinfer_b200.parts.spec import PartSpec
    torch.manual_seed(3)
    d, T, page = 72, 45, 8
    rope = PartSpec("rope", {"head_dim": hd, "rotary_dim": hd, "theta": 10000.0, "scaling": None})
    part = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": d, "num_heads": Hq, "num_kv_heads": Hkv,
                                                   "head_dim": hd, "scale": 0.21, "window": window,
                                                   "position": rope}))
    assert part.cache_need() == PagedKV(Hkv, hd, window)
    part.prepare(ctx(dt, page=page))
    w = {n: (torch.randn(v.shape) * (2.0 if n[0] in "qk" else 1.0) / math.sqrt(v.shape[1])).to(dt)
         for n, v in part.param_decls().items()}
    part.load({n: t.to(dev()) for n, t in w.items()})
    x = torch.randn(T, d).to(dt)
    cache = torch.full((12, 2, Hkv, page, hd), float("nan"), dtype=dt, device=dev())
    y = part.forward(x.to(dev()), one_sequence_step(T, page, needs=part.step_indices()),
                     PagedLayerCache(cache, 0, True))
    xd, wd = x.double(), {n: t.double() for n, t in w.items()}
    f = P.rope_inv_freq(hd, 10000.0, None)
    pos = torch.arange(T)
    q = P.rope_rotate((xd @ wd["q_proj.weight"].T).view(T, Hq, hd), pos, f)
    k = P.rope_rotate((xd @ wd["k_proj.weight"].T).view(T, Hkv, hd), pos, f)
    v = (xd @ wd["v_proj.weight"].T).view(T, Hkv, hd)
    a = P.causal_gqa_attention(q, k, v, 0.21, window).reshape(T, Hq * hd)
    assert rel_err(y, a @ wd["o_proj.weight"].T) <= TOLP[dt]
    # what it left in the cache: rotated keys and plain values at the slots of the table
    got_k = cache[3: 3 + (T + page - 1) // page, 0].permute(0, 2, 1, 3).reshape(-1, Hkv, hd)[:T]
    assert rel_err(got_k, k) <= TOLP[dt]


# ------------------------------------------------------------------ a toy architecture
# A mixer with fixed-size state of its own (an exponential moving sum of its inputs), put
# into a model beside ordinary attention layers.  Everything it needs is in this file: the
# mixer class, the configuration, the registry entry, and the plain statement of what it
# computes.  No file of the framework knows it.

def _register_toy():
    from rustinfer_b200.config.registry import ArchitectureFamily, register_architecture
    from rustinfer_b200.parts.base import FixedState, Mixer, ParamDecl, register_mixer
    from rustinfer_b200.parts.linear import Linear
    from rustinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    @register_mixer("toy_moving_sum")
    class MovingSum(Mixer):
        """s_t = decay * s_{t-1} + x_t (fp32, per request); y_t = W s_t."""
        graph_safe = False                    # it walks the entries on the host

        def __init__(self, params):
            super().__init__(params)
            self.d, self.decay = int(params["hidden_size"]), float(params["decay"])

        def param_decls(self):
            return {"mix.weight": ParamDecl((self.d, self.d))}

        def cache_need(self):
            return FixedState((self.d,), "float32")

        def load(self, tensors):
            self.mix = Linear(tensors["mix.weight"])

        def forward(self, x, step, cache):
            states = torch.empty((x.shape[0], self.d), dtype=torch.float32, device=x.device)
            row = 0
            for e in step.entries:
                s = cache.state[e.slot]
                for j in range(e.q_len):
                    s = self.decay * s + x[row + j].float()
                    states[row + j] = s
                cache.state[e.slot] = s
                row += e.q_len
            return self.mix(states.to(x.dtype), out_dtype=x.dtype)

    def spec_of(cfg):
        d = cfg["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": d, "eps": cfg["eps"]})
        ffn = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": cfg["intermediate_size"]})
        rope = PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 10000.0, "scaling": None})
        att = PartSpec("gqa_attention", {"hidden_size": d, "num_heads": d // 16, "num_kv_heads": 1, "head_dim": 16,
                                         "scale": 0.25, "window": None, "position": rope})
        toy = PartSpec("toy_moving_sum", {"hidden_size": d, "decay": cfg["decay"]})
        layers = []
        for i, kind in enumerate(cfg["mixers"]):
            p = f"layers.{i}."
            layers.append(LayerSpec(mixer=toy if kind == "toy" else att, mixer_norm=norm, ffn=ffn, ffn_norm=norm,
                                    names={"mixer": p + "mixer.", "mixer_norm": p + "norm1.", "ffn": p + "mlp.",
                                           "ffn_norm": p + "norm2."}))
        return ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], layers=tuple(layers),
                         run_order=tuple(RunEntry(i) for i in range(len(layers))), final_norm=norm,
                         embed_name="embed.", final_norm_name="norm.", head_name="head.", tie_head=True)

    register_architecture(["ToyMovingSumLM"], ArchitectureFamily("toy", lambda c, g: dict(c), spec_of))


def _toy_plain(cfg, w, ids):
    """Whole sequence, float64, from the definitions above and the plain Llama parts."""
    d = cfg["hidden_size"]
    T = len(ids)
    h = P.embedding(w["embed.weight"], ids)
    f = P.rope_inv_freq(16, 10000.0, None)
    pos = torch.arange(T)
    for i, kind in enumerate(cfg["mixers"]):
        p = f"layers.{i}."
        x = P.rmsnorm(h, w[p + "norm1.weight"], cfg["eps"])
        if kind == "toy":
            s = torch.zeros(d, dtype=torch.float64)
            rows = []
            for t in range(T):
                s = cfg["decay"] * s + x[t]
                rows.append(s)
            h = h + torch.stack(rows) @ w[p + "mixer.mix.weight"].T
        else:
            Hq = d // 16
            q = P.rope_rotate((x @ w[p + "mixer.q_proj.weight"].T).view(T, Hq, 16), pos, f)
            k = P.rope_rotate((x @ w[p + "mixer.k_proj.weight"].T).view(T, 1, 16), pos, f)
            v = (x @ w[p + "mixer.v_proj.weight"].T).view(T, 1, 16)
            a = P.causal_gqa_attention(q, k, v, 0.25).reshape(T, d)
            h = h + a @ w[p + "mixer.o_proj.weight"].T
        x = P.rmsnorm(h, w[p + "norm2.weight"], cfg["eps"])
        m = P.swiglu(x @ w[p + "mlp.gate_proj.weight"].T, x @ w[p + "mlp.up_proj.weight"].T)
        h = h + m @ w[p + "mlp.down_proj.weight"].T
    return P.rmsnorm(h, w["norm.weight"], cfg["eps"]) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    from rustinfer_b200.weights.random_init import write_random_model
    _register_toy()
    cfg = {"architectures": ["ToyMovingSumLM"], "hidden_size": 48, "intermediate_size": 72, "vocab_size": 97,
           "eps": 1e-5, "decay": 0.8, "mixers": ["toy", "attention", "toy"]}
    folder = write_random_model(str(tmp_path / "toy"), cfg, seed=5, std=0.15, norm_std=0.2)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    r = ModelRunner(folder, dtype=dtype, max_model_len=128, page_size=8, num_pages=16, max_batch_seqs=3,
                    max_batch_tokens=128)
    from rustinfer_b200.parts.base import FixedState, PagedKV
    assert [type(g.need) for g in r.layout.groups] == [FixedState, PagedKV]
    assert r.layout.groups[0].entries == [0, 2] and not r.model.graph_safe
    _, w = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(0)
    a, b = (torch.randint(0, 97, (n,), generator=g).tolist() for n in (40, 23))
    tol = LOGITS_TOL[dtype]
    # two requests, cut differently and mixed in the same steps; state must carry across cuts
    r.open("a"), r.open("b")
    got_a, got_b = [], []
    plan = [([0, 10], [0, 1]), ([10, 11], [1, 20]), ([11, 30], [20, 21]), ([30, 40], [21, 23])]
    for (a0, a1), (b0, b1) in plan:
        lg = r.step([StepEntry("a", a[a0:a1], list(range(a1 - a0))), StepEntry("b", b[b0:b1], list(range(b1 - b0)))])
        got_a.append(lg[: a1 - a0]); got_b.append(lg[a1 - a0:])
    assert rel_err(torch.cat(got_a), _toy_plain(cfg, w, a)) <= tol
    assert rel_err(torch.cat(got_b), _toy_plain(cfg, w, b)) <= tol
    # a slot that is used again starts from zero state
    r.close("a")
    r.open("c")
    assert r.cache.slot("c") == 0
    lg = r.step([StepEntry("c", b, list(range(len(b))))])
    assert rel_err(lg, _toy_plain(cfg, w, b)) <= tol


# ------------------------------------------- run order as data, shared caches, windows
# A toy architecture out of the framework's own parts, arranged in ways Llama never is:
# a layer with a sliding window (its pages form a cache group of their own and are given
# back as the window passes), a layer that runs twice (each visit has its own cache), and
# a layer without key/value projections that reads the cache another visit wrote.

def _register_arranged():
    from rustinfer_b200.config.registry import ArchitectureFamily, register_architecture
    from rustinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    def spec_of(cfg):
        d, hd, Hq, Hkv = cfg["hidden_size"], 16, cfg["hidden_size"] // 16, 2
        norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
        ffn = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": cfg["intermediate_size"]})
        rope = PartSpec("rope", {"head_dim": hd, "rotary_dim": hd, "theta": 10000.0, "scaling": None})
        att = lambda window, own: PartSpec("gqa_attention", {
            "hidden_size": d, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd, "scale": 0.25,
            "window": window, "position": rope, "own_kv": own})
        kinds = [att(None, True), att(cfg["window"], True), att(None, False)]
        layers = tuple(LayerSpec(mixer=m, mixer_norm=norm, ffn=ffn, ffn_norm=norm,
                                 names={"mixer": f"l{i}.att.", "mixer_norm": f"l{i}.n1.", "ffn": f"l{i}.mlp.",
                                        "ffn_norm": f"l{i}.n2."}) for i, m in enumerate(kinds))
        # layer 0 (full), layer 1 (window), layer 0 again, layer 2 reading the cache of the first visit
        order = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(2, cache_of=0))
        return ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], layers=layers, run_order=order,
                         final_norm=norm, embed_name="embed.", final_norm_name="norm.", head_name="head.",
                         tie_head=False)

    register_architecture(["ArrangedToyLM"], ArchitectureFamily("arranged", lambda c, g: dict(c), spec_of))


def _arranged_plain(cfg, w, ids):
    d, hd, Hkv = cfg["hidden_size"], 16, 2
    Hq, T = d // hd, len(ids)
    f = P.rope_inv_freq(hd, 10000.0, None)
    pos = torch.arange(T)
    h = P.embedding(w["embed.weight"], ids)
    kv_of_visit = {}
    for visit, (layer, cache_of) in enumerate([(0, None), (1, None), (0, None), (2, 0)]):
        p = f"l{layer}."
        x = P.rmsnorm(h, w[p + "n1.weight"], 1e-5)
        q = P.rope_rotate((x @ w[p + "att.q_proj.weight"].T).view(T, Hq, hd), pos, f)
        if cache_of is None:
            k = P.rope_rotate((x @ w[p + "att.k_proj.weight"].T).view(T, Hkv, hd), pos, f)
            v = (x @ w[p + "att.v_proj.weight"].T).view(T, Hkv, hd)
            kv_of_visit[visit] = (k, v)
        else:
            k, v = kv_of_visit[cache_of]
        a = P.causal_gqa_attention(q, k, v, 0.25, cfg["window"] if layer == 1 else None).reshape(T, d)
        h = h + a @ w[p + "att.o_proj.weight"].T
        x = P.rmsnorm(h, w[p + "n2.weight"], 1e-5)
        m = P.swiglu(x @ w[p + "mlp.gate_proj.weight"].T, x @ w[p + "mlp.up_proj.weight"].T)
        h = h + m @ w[p + "mlp.down_proj.weight"].T
    return P.rmsnorm(h, w["norm.weight"], 1e-5) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_shared_cache_and_window_group(tmp_path, dtype):
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    from rustinfer_b200.parts.base import PagedKV
    from rustinfer_b200.weights.random_init import write_random_model
    _register_arranged()
    cfg = {"architectures": ["ArrangedToyLM"], "hidden_size": 64, "intermediate_size": 96, "vocab_size": 113,
           "window": 11}
    folder = write_random_model(str(tmp_path / "arranged"), cfg, seed=3, std=0.2, norm_std=0.2)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    _, w = P.read_model_folder(folder)
    assert "l2.att.k_proj.weight" not in w                    # the reading layer projects no keys
    r = ModelRunner(folder, dtype=dtype, max_model_len=128, page_size=4, num_pages=40, max_batch_seqs=2,
                    max_batch_tokens=128)
    # two cache groups: full attention (visits 0 and 2 of the run order) and the window layer
    assert [g.need for g in r.layout.groups] == [PagedKV(2, 16, None), PagedKV(2, 16, 11)]
    assert r.layout.groups[0].entries == [0, 2] and r.layout.groups[1].entries == [1]
    assert r.layout.entry_cache == [(0, 0), (1, 0), (0, 1), (0, 0)] and r.layout.entry_writes[3] is False
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 113, (60,), generator=g).tolist()
    ref = _arranged_plain(cfg, w, ids)
    tol = LOGITS_TOL[dtype]
    for cuts in ([60], [7, 20, 1, 1, 1, 2, 28], [1] * 60):
        r.open("a")
        outs, at = [], 0
        for c in cuts:
            outs.append(r.step([StepEntry("a", ids[at: at + c], list(range(c)))]))
            at += c
            held = r.cache.pages_held("a")
            assert held[0] == (at + 3) // 4                        # every key is kept
            assert held[1] <= (11 + 4 + 3) // 4 + 1                # the window group holds a window's worth
        assert rel_err(torch.cat(outs), ref) <= tol, cuts
        r.close("a")
        r.cache.check_invariants()
    assert r.cache.free_pages() == {0: 40, 1: 40}


# ------------------------------------------------ other shapes of a block, from this file alone
# A layer needs only a mixer: here one block runs attention and feed-forward side by side off
# one norm, one has a single sublayer, and one norms what its sublayers return (norms under
# roles of their own) before it is added.  The arrangements are registered below; the
# framework's files know none of them.
def _register_shapes():
    from rustinfer_b200.config.registry import ArchitectureFamily, register_architecture
    from rustinfer_b200.parts.block import register_arrangement
    from rustinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    def settle(hidden):
        """the stream with everything pending added (fp32)"""
        if hidden.pending is not None:
            hidden.stream += hidden.pending.float()
            hidden.pending = None
        return hidden.stream

    def parallel(block, hidden, step, cache):
        x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
        a = block.mixer.forward(x, step, cache)
        hidden.stream += a.float()
        hidden.pending = block.ffn.forward(x, step)

    def mixer_only(block, hidden, step, cache):
        x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
        hidden.pending = block.mixer.forward(x, step, cache)

    def sandwich(block, hidden, step, cache):
        x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
        a = block.mixer.forward(x, step, cache)
        zeros = torch.zeros_like(hidden.stream)
        hidden.pending = block.extra_norms["after_mixer"].add_norm(zeros, a)
        x = block.ffn_norm.add_norm(hidden.stream, hidden.pending)
        m = block.ffn.forward(x, step)
        hidden.pending = block.extra_norms["after_ffn"].add_norm(torch.zeros_like(hidden.stream), m)

    register_arrangement("toy_parallel", parallel)
    register_arrangement("toy_mixer_only", mixer_only)
    register_arrangement("toy_sandwich", sandwich)

    def spec_of(cfg):
        d, hd, Hq, Hkv = cfg["hidden_size"], 16, cfg["hidden_size"] // 16, 2
        norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
        ffn = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": cfg["intermediate_size"]})
        rope = PartSpec("rope", {"head_dim": hd, "rotary_dim": hd, "theta": 10000.0, "scaling": None})
        att = PartSpec("gqa_attention", {"hidden_size": d, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd,
                                         "scale": 0.25, "window": None, "position": rope})
        layers = (
            LayerSpec(mixer=att, mixer_norm=norm, ffn=ffn, arrangement="toy_parallel",
                      names={"mixer": "l0.att.", "mixer_norm": "l0.n.", "ffn": "l0.mlp."}),
            LayerSpec(mixer=att, mixer_norm=norm, arrangement="toy_mixer_only",
                      names={"mixer": "l1.att.", "mixer_norm": "l1.n."}),
            LayerSpec(mixer=att, mixer_norm=norm, ffn=ffn, ffn_norm=norm, arrangement="toy_sandwich",
                      extra_norms={"after_mixer": norm, "after_ffn": norm},
                      names={"mixer": "l2.att.", "mixer_norm": "l2.n1.", "ffn": "l2.mlp.", "ffn_norm": "l2.n2.",
                             "after_mixer": "l2.p1.", "after_ffn": "l2.p2."}),
        )
        return ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], layers=layers,
                         run_order=tuple(RunEntry(i) for i in range(3)), final_norm=norm, embed_name="embed.",
                         final_norm_name="norm.", head_name="head.", tie_head=False)

    register_architecture(["ShapesToyLM"], ArchitectureFamily("shapes", lambda c, g: dict(c), spec_of))


def _shapes_plain(cfg, w, ids):
    d, hd, Hkv = cfg["hidden_size"], 16, 2
    Hq, T = d // hd, len(ids)
    f = P.rope_inv_freq(hd, 10000.0, None)
    pos = torch.arange(T)

    def attention(x, p):
        q = P.rope_rotate((x @ w[p + "q_proj.weight"].T).view(T, Hq, hd), pos, f)
        k = P.rope_rotate((x @ w[p + "k_proj.weight"].T).view(T, Hkv, hd), pos, f)
        v = (x @ w[p + "v_proj.weight"].T).view(T, Hkv, hd)
        return P.causal_gqa_attention(q, k, v, 0.25, None).reshape(T, d) @ w[p + "o_proj.weight"].T

    def mlp(x, p):
        return P.swiglu(x @ w[p + "gate_proj.weight"].T, x @ w[p + "up_proj.weight"].T) @ w[p + "down_proj.weight"].T

    h = P.embedding(w["embed.weight"], ids)
    x = P.rmsnorm(h, w["l0.n.weight"], 1e-5)
    h = h + attention(x, "l0.att.") + mlp(x, "l0.mlp.")
    h = h + attention(P.rmsnorm(h, w["l1.n.weight"], 1e-5), "l1.att.")
    h = h + P.rmsnorm(attention(P.rmsnorm(h, w["l2.n1.weight"], 1e-5), "l2.att."), w["l2.p1.weight"], 1e-5)
    h = h + P.rmsnorm(mlp(P.rmsnorm(h, w["l2.n2.weight"], 1e-5), "l2.mlp."), w["l2.p2.weight"], 1e-5)
    return P.rmsnorm(h, w["norm.weight"], 1e-5) @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_blocks_of_other_shapes(tmp_path, dtype):
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    from rustinfer_b200.weights.random_init import write_random_model
    _register_shapes()
    cfg = {"architectures": ["ShapesToyLM"], "hidden_size": 64, "intermediate_size": 96, "vocab_size": 113}
    folder = write_random_model(str(tmp_path / "shapes"), cfg, seed=5, std=0.2, norm_std=0.2)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    _, w = P.read_model_folder(folder)
    assert "l1.mlp.gate_proj.weight" not in w and "l0.n2.weight" not in w and "l2.p2.weight" in w
    r = ModelRunner(folder, dtype=dtype, max_model_len=128, page_size=8, num_pages=24, max_batch_seqs=2,
                    max_batch_tokens=128, capture_sizes=[1, 2])
    assert r.model.chained is None                             # not the shape the chained products know
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 113, (50,), generator=g).tolist()
    ref = _shapes_plain(cfg, w, ids)
    tol = LOGITS_TOL[dtype]
    for cuts in ([50], [9, 30, 2] + [1] * 9):
        r.open("a")
        outs, at = [], 0
        for c in cuts:
            outs.append(r.step([StepEntry("a", ids[at: at + c], list(range(c)))]))
            at += c
        assert rel_err(torch.cat(outs), ref) <= tol, cuts
        r.close("a")
    assert r.graph_replays > 0                                 # single tokens were captured and replayed


# ------------------------------------------------ toy parts of every kind, from this file alone
# A stem with a multiplier and learned positions, a head with a soft cap, another rotary law, a
# feed-forward that routes each token to one of three experts, attention without any position
# encoding, and a mixer with fixed-size state that is safe to capture: it declares an index
# array of its own, which the step builder makes for every step and every replay.  None of
# them is a part of any real model; they show what the interfaces carry.

def _register_zoo():
    import numpy as np
    from rustinfer_b200.config.registry import ArchitectureFamily, register_architecture
    from rustinfer_b200.parts.base import (Embedding, FeedForward, FixedState, Head, Mixer, ParamDecl,
                                           PositionEncoding, StepIndex, register_embedding,
                                           register_feed_forward, register_head, register_mixer,
                                           register_position)
    from rustinfer_b200.parts.linear import Linear
    from rustinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    @register_embedding("zoo_scaled_positions")
    class ScaledWithPositions(Embedding):
        def __init__(self, params):
            super().__init__(params)
            self.V, self.d = int(params["vocab_size"]), int(params["hidden_size"])
            self.mult, self.max_pos = float(params["multiplier"]), int(params["max_positions"])

        def param_decls(self):
            return {"weight": ParamDecl((self.V, self.d)), "positions.weight": ParamDecl((self.max_pos, self.d))}

        def load(self, tensors):
            self.table, self.pos = tensors["weight"], tensors["positions.weight"]

        def shared_table(self):
            return self.table

        def forward(self, step, h):
            T = step.num_tokens
            ids, pos = step.token_ids[:T].long(), step.positions[:T].long()
            h.copy_(self.table[ids].float() * self.mult + self.pos[pos].float())

    @register_head("zoo_capped")
    class CappedHead(Head):
        def __init__(self, params):
            super().__init__(params)
            self.V, self.d, self.cap = int(params["vocab_size"]), int(params["hidden_size"]), float(params["cap"])

        def param_decls(self):
            return {"weight": ParamDecl((self.V, self.d), optional=True)}

        def load(self, tensors):
            self.linear = Linear(tensors.get("weight", self.shared))

        def forward(self, normed):
            return self.cap * torch.tanh(self.linear(normed, out_dtype=torch.float32) / self.cap)

    @register_position("zoo_stretched_rope")
    class StretchedRope(PositionEncoding):
        """angle = (position / stretch) * theta^(-2i/d): another frequency law behind the same tables."""
        def __init__(self, params):
            super().__init__(params)
            self.rotary_dim, self.theta, self.stretch = int(params["head_dim"]), float(params["theta"]), float(params["stretch"])

        def prepare(self, ctx):
            super().prepare(ctx)
            f = torch.tensor([self.theta ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)],
                             dtype=torch.float64)
            ang = (torch.arange(ctx.max_model_len, dtype=torch.float64) / self.stretch)[:, None] * f[None, :]
            self.cos, self.sin = torch.cos(ang).float().to(ctx.device), torch.sin(ang).float().to(ctx.device)

    phase = StepIndex(("zoo_phase",), lambda sh: (sh.pos0 % 3,), lambda max_tokens, max_entries: max_entries + 4,
                      depends_on_positions=True)

    @register_mixer("zoo_moving_sum")
    class MovingSumOnDevice(Mixer):
        """s_t = decay * s_{t-1} + (1 + 0.25 * (position mod 3)) * x_t; y_t = W s_t.  Steps of single
        tokens read only device tensors (the state rows by slot, the phase from the index array it
        declared), so they can be captured."""
        graph_safe = True

        def __init__(self, params):
            super().__init__(params)
            self.d, self.decay = int(params["hidden_size"]), float(params["decay"])

        def param_decls(self):
            return {"mix.weight": ParamDecl((self.d, self.d))}

        def cache_need(self):
            return FixedState((self.d,), "float32")

        def step_indices(self):
            return [phase]

        def load(self, tensors):
            self.mix = Linear(tensors["mix.weight"])

        def forward(self, x, step, cache):
            if step.decode_only:
                n = step.num_entries
                slots = step.state_slots[:n].long()
                (ph,) = step.index(phase)
                s = self.decay * cache.state[slots] + (1 + 0.25 * ph[:n].float())[:, None] * x.float()
                cache.state.index_copy_(0, slots, s)
                return self.mix(s.to(x.dtype), out_dtype=x.dtype)
            states = torch.empty((x.shape[0], self.d), dtype=torch.float32, device=x.device)
            row = 0
            for e in step.entries:
                s = cache.state[e.slot]
                for j in range(e.q_len):
                    s = self.decay * s + (1 + 0.25 * ((e.pos0 + j) % 3)) * x[row + j].float()
                    states[row + j] = s
                cache.state[e.slot] = s
                row += e.q_len
            return self.mix(states.to(x.dtype), out_dtype=x.dtype)

    @register_feed_forward("zoo_routed")
    class RoutedToy(FeedForward):
        """Each token goes to the expert with the largest router logit (fp32): down_e(relu(up_e(x)))."""
        def __init__(self, params):
            super().__init__(params)
            self.d, self.inter, self.E = int(params["hidden_size"]), int(params["intermediate_size"]), int(params["experts"])

        def param_decls(self):
            d = {"router.weight": ParamDecl((self.E, self.d))}
            for e in range(self.E):
                d[f"experts.{e}.up.weight"] = ParamDecl((self.inter, self.d))
                d[f"experts.{e}.down.weight"] = ParamDecl((self.d, self.inter))
            return d

        def load(self, tensors):
            self.router = Linear(tensors["router.weight"])
            self.up = [Linear(tensors[f"experts.{e}.up.weight"]) for e in range(self.E)]
            self.down = [Linear(tensors[f"experts.{e}.down.weight"]) for e in range(self.E)]

        def forward(self, x, step):
            pick = self.router(x, out_dtype=torch.float32).argmax(dim=1)
            out = torch.zeros_like(x)
            for e in range(self.E):
                y = self.down[e](torch.relu(self.up[e](x)), out_dtype=x.dtype)
                out += y * (pick == e)[:, None].to(x.dtype)
            return out

    def spec_of(cfg):
        d, hd = cfg["hidden_size"], 16
        norm = PartSpec("rmsnorm", {"size": d, "eps": 1e-5})
        swiglu = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": cfg["intermediate_size"]})
        routed = PartSpec("zoo_routed", {"hidden_size": d, "intermediate_size": cfg["intermediate_size"], "experts": 3})
        att = lambda pos: PartSpec("gqa_attention", {"hidden_size": d, "num_heads": d // hd, "num_kv_heads": 2,
                                                     "head_dim": hd, "scale": 0.25, "window": None, "position": pos})
        stretched = PartSpec("zoo_stretched_rope", {"head_dim": hd, "theta": 1000.0, "stretch": 2.5})
        mixers = [att(None), PartSpec("zoo_moving_sum", {"hidden_size": d, "decay": 0.7}), att(stretched)]
        ffns = [swiglu, routed if cfg["routed"] else swiglu, swiglu]
        layers = tuple(LayerSpec(mixer=m, mixer_norm=norm, ffn=f, ffn_norm=norm,
                                 names={"mixer": f"l{i}.mix.", "mixer_norm": f"l{i}.n1.", "ffn": f"l{i}.ffn.",
                                        "ffn_norm": f"l{i}.n2."}) for i, (m, f) in enumerate(zip(mixers, ffns)))
        return ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], layers=layers,
                         run_order=tuple(RunEntry(i) for i in range(3)), final_norm=norm, embed_name="embed.",
                         final_norm_name="norm.", head_name="head.", tie_head=True,
                         embed=PartSpec("zoo_scaled_positions", {"vocab_size": cfg["vocab_size"], "hidden_size": d,
                                                                 "multiplier": 1.5, "max_positions": 128}),
                         head=PartSpec("zoo_capped", {"vocab_size": cfg["vocab_size"], "hidden_size": d, "cap": 3.0}))

    register_architecture(["ZooLM"], ArchitectureFamily("zoo", lambda c, g: dict(c), spec_of))


def _zoo_plain(cfg, w, ids):
    d, hd, Hkv = cfg["hidden_size"], 16, 2
    Hq, T = d // hd, len(ids)
    pos = torch.arange(T)
    h = P.embedding(w["embed.weight"], ids) * 1.5 + w["embed.positions.weight"][:T]
    for i in range(3):
        p = f"l{i}."
        x = P.rmsnorm(h, w[p + "n1.weight"], 1e-5)
        if i == 1:
            s, rows = torch.zeros(d, dtype=torch.float64), []
            for t in range(T):
                s = 0.7 * s + (1 + 0.25 * (t % 3)) * x[t]
                rows.append(s)
            h = h + torch.stack(rows) @ w[p + "mix.mix.weight"].T
        else:
            q = (x @ w[p + "mix.q_proj.weight"].T).view(T, Hq, hd)
            k = (x @ w[p + "mix.k_proj.weight"].T).view(T, Hkv, hd)
            v = (x @ w[p + "mix.v_proj.weight"].T).view(T, Hkv, hd)
            if i == 2:
                f = torch.tensor([1000.0 ** (-2.0 * j / hd) for j in range(hd // 2)], dtype=torch.float64)
                q, k = P.rope_rotate(q, pos / 2.5, f), P.rope_rotate(k, pos / 2.5, f)
            h = h + P.causal_gqa_attention(q, k, v, 0.25).reshape(T, d) @ w[p + "mix.o_proj.weight"].T
        x = P.rmsnorm(h, w[p + "n2.weight"], 1e-5)
        if i == 1 and cfg["routed"]:
            pick = (x @ w[p + "ffn.router.weight"].T).argmax(dim=1)
            y = torch.zeros_like(x)
            for t in range(T):
                e = int(pick[t])
                y[t] = torch.relu(x[t] @ w[p + f"ffn.experts.{e}.up.weight"].T) @ w[p + f"ffn.experts.{e}.down.weight"].T
            h = h + y
        else:
            m = P.swiglu(x @ w[p + "ffn.gate_proj.weight"].T, x @ w[p + "ffn.up_proj.weight"].T)
            h = h + m @ w[p + "ffn.down_proj.weight"].T
    z = P.rmsnorm(h, w["norm.weight"], 1e-5) @ w["embed.weight"].T
    return 3.0 * torch.tanh(z / 3.0)


@pytest.mark.parametrize("dtype,routed", [("float32", True), ("float32", False), ("bfloat16", False)])
def test_toy_parts_of_every_kind_are_registered_built_stepped_and_captured(tmp_path, dtype, routed):
    """Stem, head, position law, routed feed-forward, attention without positions and a stateful
    mixer with an index array of its own, all defined above; stepped eagerly and from captured
    graphs whose bucket is larger than the batch (padding rows must not touch a live request's
    state), against the float64 statement."""
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    from rustinfer_b200.weights.random_init import write_random_model
    _register_zoo()
    cfg = {"architectures": ["ZooLM"], "hidden_size": 64, "intermediate_size": 80, "vocab_size": 101, "routed": routed}
    folder = write_random_model(str(tmp_path / "zoo"), cfg, seed=9, std=0.15, norm_std=0.2)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    _, w = P.read_model_folder(folder)
    assert "head.weight" not in w and "embed.positions.weight" in w
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (37, 50, 44)]
    refs = [_zoo_plain(cfg, w, s) for s in seqs]
    tol = LOGITS_TOL[dtype]
    for sizes in (None, [1, 2, 4]):
        r = ModelRunner(folder, dtype=dtype, max_model_len=96, page_size=8, num_pages=40, max_batch_seqs=4,
                        max_batch_tokens=96, capture_sizes=sizes)
        assert r.model.graph_safe and r.use_graphs == (sizes is not None)
        assert ("zoo_phase",) in [n.key for n in r.index_needs]
        got = [[] for _ in seqs]
        first = [9, 20, 3]
        for i, s in enumerate(seqs):
            r.open(i)
            got[i].append(r.step([StepEntry(i, s[: first[i]], list(range(first[i])))]))
        at = list(first)
        turn = 0
        while any(a < len(s) for a, s in zip(at, seqs)):
            live = [i for i in range(3) if at[i] < len(seqs[i]) and (turn + i) % 5 != 4]
            turn += 1
            if not live:
                continue
            lg = r.step([StepEntry(i, [seqs[i][at[i]]], [0]) for i in live])   # 1 to 3 rows: buckets 1, 2, 4
            for k_, i in enumerate(live):
                got[i].append(lg[k_: k_ + 1])
                at[i] += 1
        if sizes is not None:
            assert r.graph_replays > 30 and 4 in r._graphs
        for i in range(3):
            assert rel_err(torch.cat(got[i]), refs[i]) <= tol, (dtype, sizes, i)
