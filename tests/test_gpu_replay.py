"""The engine against the plain implementation under every way of cutting the work:
whole prompts, a decoded tail, portions of changing size, and mixed batches with so few
pages that they are used again.  In true 32-bit and in bfloat16, on tiny configurations
that differ in every size and option."""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import TINY, Plain, make_sharp_model, random_ids, rel_err

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# max |engine - plain| / max |plain| over the compared logits.  fp32: measured 0.6e-6 to
# 2e-6 on these models (sums of a few hundred fp32 products against float64).  bf16: the
# engine rounds activations, keys and values to 8 bits of mantissa, and these models are made
# sharp (one score stands out by design), so a rounding of q or k moves a whole softmax row.
# Measured over 24 sequences a model, cut into portions, with the products run one by one and
# chained alike: A mean 1.0e-2, worst 2.1e-2; B mean 2.4e-2, 90th percentile 3.3e-2, worst
# 4.3e-2; C mean 0.4e-2, worst 0.7e-2.  Which roundings meet at the sharp position differs from
# cut to cut, so the bound sits above the worst realisation seen; the faults these tests are
# made for (a wrong key, page or position at the sharp score) move the logits by tenths.
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
# The same positions through a different cut of the work, engine against engine: fp32 is
# bit-identical by construction of the kernels and asserted as such.  In bf16 a decoded
# token and a prompt portion go through different kernels (split-KV decode, tiled prefill)
# and the library picks GEMM tiles by batch size, so two cuts are two independent roundings;
# each is held to TOL against the plain implementation, which is the comparison that counts.

NAMES = ["A", "B", "C", "D", "E", "F", "Bs"]
FAST = ["D", "E", "F"]                   # head sizes 64 and 128: the attention kernels of the benchmark shapes
DTYPES = ["float32", "bfloat16"]
PAGE = {"A": 16, "B": 8, "C": 16, "D": 16, "E": 16, "F": 8, "Bs": 8}


def expect_fast_kernels(r, name):
    """In bfloat16 the models with head sizes 64 and 128 must run on the kernels made for
    them: keys and values by TMA when decoding, tcgen05 for prompt portions (a group of 3 heads
    included: 42 tokens a tile and two rows of padding), and the chained products for steps of few tokens."""
    if name not in FAST or r.dtype != torch.bfloat16:
        return
    from rustinfer_b200.ops import library
    for b in r.model.blocks:
        a = b.mixer
        lib = library.attention_mma(a.hd)
        tma = int(lib.ri_attention_decode_tma_ctas_per_sm(r.page_size))
        assert tma > 0 and a.decode_ctas_per_sm == tma, "decode attention does not fetch by TMA"
        assert a.use_tc, "prompt attention is not on tcgen05"
    assert r.model.chained is not None and r.model.chained.max_tokens >= 16


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for n in NAMES:
        folder = make_sharp_model(str(root / n), n, seed=11 + ord(n[0]) + len(n))
        out[n] = (folder, Plain(folder))
    return out


def runner(folder, dtype, max_tokens=512, page=16, seqs=4, pages=None):
    from rustinfer_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_model_len=max_tokens, page_size=page,
                       num_pages=pages if pages is not None else max_tokens // page,
                       max_batch_seqs=seqs, max_batch_tokens=max_tokens)


def run_cuts(r, rid, ids, cuts):
    """Feed `ids` in portions of the given sizes; logits of every position."""
    from rustinfer_b200.engine.runner import StepEntry
    r.open(rid)
    outs, at = [], 0
    for c in cuts:
        outs.append(r.step([StepEntry(rid, ids[at: at + c], list(range(c)))]))
        at += c
    assert at == len(ids)
    r.close(rid)
    return torch.cat(outs)


@pytest.mark.parametrize("name", FAST)
def test_steps_of_many_tokens(models, name, monkeypatch):
    """Steps of 512 tokens or more take the q,k,v product with the rotary encoding and the cache
    write in its epilogue.  Every position of a 700-token prompt against the plain model; the same
    prompt in portions of 520 + 180 and 690 + ten single tokens (which read the keys that epilogue
    wrote); a second request's 600 tokens beside a decoded token of the first; and all of it again
    with the rotary kernel run on its own: the two ways round q and k at different places, so they
    differ by roundings, half the tolerance against the plain model at most (the bound the ways of
    decoding are held to further down)."""
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    ids = random_ids(700, V, 41)
    other = random_ids(600, V, 42)
    ref, ref_other = plain.logits(ids), plain.logits(other)
    outs = {}
    for fused in (True, False):
        monkeypatch.setenv("RUSTINFER_B200_FUSE_ROPE", "1" if fused else "0")
        r = ModelRunner(folder, dtype="bfloat16", max_model_len=1024, page_size=16, num_pages=2 * 64 + 4,
                        max_batch_seqs=4, max_batch_tokens=1024)
        assert r.model.blocks[0].mixer.fuse_rope == fused
        whole = run_cuts(r, "w", ids, [700])
        assert rel_err(whole, ref) <= TOL["bfloat16"]
        assert rel_err(run_cuts(r, "p", ids, [520, 180]), ref) <= TOL["bfloat16"]
        assert rel_err(run_cuts(r, "t", ids, [690] + [1] * 10), ref) <= TOL["bfloat16"]
        # 600 prompt tokens of one request beside a decoded token of another in one step
        r.open("a"); r.open("b")
        r.step([StepEntry("a", ids[:650], [])])
        lg = r.step([StepEntry("a", ids[650:651], [0]), StepEntry("b", other, list(range(600)))])
        assert rel_err(lg[:1], ref[650:651]) <= TOL["bfloat16"]
        assert rel_err(lg[1:], ref_other) <= TOL["bfloat16"]
        r.close("a"); r.close("b")
        torch.cuda.synchronize()
        r.check_kernel_errors()
        r.cache.check_invariants()
        outs[fused] = whole
    assert rel_err(outs[True], outs[False]) <= TOL["bfloat16"] / 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_tail_and_portions(models, name, dtype):
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    page = PAGE[name]
    r = runner(folder, dtype, page=page)
    expect_fast_kernels(r, name)
    for n, seed in [(100, 1), (70, 2), (33, 3)] + ([(300, 5)] if name in FAST else []):
        ids = random_ids(n, V, seed)
        ref = plain.logits(ids)
        whole = run_cuts(r, "w", ids, [n])
        assert rel_err(whole, ref) <= TOL[dtype]
        # most of it in one step, the last 32 tokens one by one
        tail = run_cuts(r, "t", ids, [n - 32] + [1] * 32)
        assert rel_err(tail, ref) <= TOL[dtype]
        # portions of changing size, down to two tokens (and one)
        cuts, left, sizes = [], n, [24, 7, 2, 13, 2, 1, 30, 3, 2, 16, 5]
        while left:
            c = min(left, sizes[len(cuts) % len(sizes)])
            cuts.append(c); left -= c
        parts = run_cuts(r, "p", ids, cuts)
        assert rel_err(parts, ref) <= TOL[dtype]
        if dtype == "float32":
            assert torch.equal(tail, whole) and torch.equal(parts, whole)
    r.cache.check_invariants()
    assert r.cache.free_pages() == {0: 512 // page}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(models, name, dtype):
    """Positions 0, 1, 2: one key, no earlier page, a one-token prompt."""
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    r = runner(folder, dtype)
    ids = random_ids(3, V, 9)
    ref = plain.logits(ids)
    assert rel_err(run_cuts(r, "a", ids, [1, 1, 1]), ref) <= TOL[dtype]
    assert rel_err(run_cuts(r, "b", ids, [3]), ref) <= TOL[dtype]
    assert rel_err(run_cuts(r, "c", ids[:1], [1]), ref[:1]) <= TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding(models, name, dtype):
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    n = {"A": 128, "B": 400, "C": 250, "D": 300, "E": 200, "F": 200, "Bs": 100}[name]   # within the model's positions
    r = runner(folder, dtype, page=8)
    ids = random_ids(n, V, 4)
    got = run_cuts(r, "d", ids, [5] + [1] * (n - 5))
    ref = plain.logits(ids)
    assert rel_err(got, ref) <= TOL[dtype]
    per_pos = (got.double().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
    assert float(per_pos[-50:].max()) <= TOL[dtype]      # no drift with distance


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_page_reuse(models, name, dtype):
    """Up to four live requests; portions of some beside decoded tokens of others in one
    step; a pool so small that pages of finished requests are used again at once; freed
    pages are poisoned with NaN so that a read of a stale page shows."""
    from rustinfer_b200.engine.runner import StepEntry
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    page = {"A": 16, "B": 8, "C": 4, "D": 16, "E": 8, "F": 32, "Bs": 8}[name]
    lens = [41, 17, 64, 9, 52, 30, 23, 70]
    seqs = [random_ids(n, V, 100 + i) for i, n in enumerate(lens)]
    # room for the four largest neighbours, far less than the sum of all eight
    pool_tokens = 64 * 4
    r = runner(folder, dtype, max_tokens=pool_tokens, page=page, seqs=4)
    expect_fast_kernels(r, name)
    got = {i: [] for i in range(len(seqs))}
    at = {i: 0 for i in range(len(seqs))}
    live, waiting = [], list(range(len(seqs)))
    portion = [5, 2, 11, 1, 24, 3, 1, 1, 7]
    turn = 0
    used_pages = set()
    while live or waiting:
        while waiting and len(live) < 4:
            i = waiting.pop(0)
            r.open(i); live.append(i)
        entries = []
        for j, i in enumerate(live):
            if (turn + j) % 5 == 4:
                continue                                  # a request may sit a step out
            left = len(seqs[i]) - at[i]
            # once a request is past three quarters it goes token by token, like decoding
            c = 1 if at[i] * 4 >= len(seqs[i]) * 3 else min(left, portion[(turn + 3 * j) % len(portion)])
            entries.append(StepEntry(i, seqs[i][at[i]: at[i] + c], list(range(c))))
        turn += 1
        if not entries:
            continue
        logits = r.step(entries)
        row = 0
        for e in entries:
            c = len(e.tokens)
            got[e.request_id].append(logits[row: row + c]); row += c
            at[e.request_id] += c
            used_pages.update(r.cache.block_table(e.request_id, 0))
        for i in list(live):
            if at[i] == len(seqs[i]):
                pages = list(r.cache.block_table(i, 0))
                r.close(i); live.remove(i)
                r.group_storage[0][:, pages] = float("nan")
        r.cache.check_invariants()
    total_blocks = sum((n + page - 1) // page for n in lens)
    assert total_blocks > pool_tokens // page                 # pages had to be used again
    assert r.cache.free_pages() == {0: pool_tokens // page}
    for i, ids in enumerate(seqs):
        assert rel_err(torch.cat(got[i]), plain.logits(ids)) <= TOL[dtype], (name, dtype, i)


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_refuses_bad_batches_and_leaves_the_cache_alone(models, dtype):
    from rustinfer_b200.cache.pages import OutOfPages
    from rustinfer_b200.engine.runner import StepEntry, StepError
    folder, _ = models["A"]
    r = runner(folder, dtype, max_tokens=64, page=16, seqs=2)
    r.open("a")
    with pytest.raises(StepError, match="token id"):
        r.step([StepEntry("a", [1, 256], [0])])
    with pytest.raises(StepError, match="not open"):
        r.step([StepEntry("zz", [1], [0])])
    with pytest.raises(StepError, match="twice"):
        r.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(StepError, match="wanted place"):
        r.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="no tokens"):
        r.step([StepEntry("a", [], [])])
    with pytest.raises(StepError, match="max_model_len"):
        r.step([StepEntry("a", [1] * 65, [])])
    r.open("b")
    r.step([StepEntry("a", [1] * 40, [])])
    with pytest.raises(OutOfPages):
        r.step([StepEntry("b", [1] * 30, [0])])              # 3 + 2 pages > 4
    assert r.cache.length("b") == 0 and r.cache.free_pages() == {0: 1}
    assert r.step([StepEntry("b", [1] * 16, [15])]).shape == (1, 256)
    assert r.step([StepEntry("a", [3], [])]) is None           # nothing wanted: nothing returned


def test_trace_run_program(models, tmp_path):
    """bin/trace_run as a user runs it: JSON lines in, `done <step>` lines and .f32 files out."""
    folder, plain = models["B"]
    V = TINY["B"]["vocab_size"]
    a, b = random_ids(50, V, 1), random_ids(20, V, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []},
                                {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[32:], "want": [17]}], "end": ["a"]},
        {"step": 7, "entries": [{"id": "c", "tokens": b, "want": [19]}], "end": ["c"]},
    ]
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                            "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                           input="".join(json.dumps(s) + "\n" for s in steps), text=True,
                           capture_output=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "7"]
        import numpy as np
        rd = lambda s: torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, V))
        ra, rb = plain.logits(a), plain.logits(b)
        assert rel_err(rd(0), ra[[0, 29]]) <= TOL[dtype]
        assert rel_err(rd(1), rb[[18]]) <= TOL[dtype]
        assert rel_err(rd(2), rb[[19]]) <= TOL[dtype]
        assert rel_err(rd(3), ra[[49]]) <= TOL[dtype]
        assert rel_err(rd(7), rb[[19]]) <= TOL[dtype]
        assert not (out / "4.f32").exists()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D", "E", "F"])
def test_greedy_generation_through_the_entry_point(models, name, dtype):
    import plain_llama
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    prompts = [random_ids(n, V, 50 + n) for n in (5, 17, 32, 1)]
    eng = Engine(folder, dtype=dtype, max_batch_tokens=40, max_batch_seqs=3, max_model_len=64,
                 paged_block_size=8, chunked_prefill_size=24, num_blocks=20)
    expect_fast_kernels(eng.runner, name)
    res = eng.generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True))
    for p, out in zip(prompts, res):
        assert out.finish_reason == "length" and len(out.tokens) == 16
        if dtype == "float32":
            assert out.tokens == plain_llama.greedy_generate(plain.cfg, plain.w, p, 16)
        else:
            # bf16 may flip a near-tie; every chosen token must be (almost) the plain argmax
            seq = list(p)
            for t in out.tokens:
                row = plain.logits(seq)[-1]
                assert float(row.max() - row[t]) <= TOL[dtype] * float(row.abs().max()) * 2
                seq.append(t)
    assert eng.runner.cache.free_pages() == {0: 20}
    assert eng.stats.generated_tokens == 64
    assert eng.stats.stop_flag_mismatches == 0                # the device's stop check agrees with the host's


def test_seeded_sampling_does_not_depend_on_the_batch(models):
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, _ = models["B"]
    V = TINY["B"]["vocab_size"]
    prompts = [random_ids(n, V, 70 + n) for n in (1, 9, 40, 100)]
    sp = SamplingParams(temperature=0.8, seed=1234, max_tokens=12, ignore_eos=True)
    eng = Engine(folder, dtype="float32", max_batch_tokens=64, max_batch_seqs=4, max_model_len=128,
                 paged_block_size=8, chunked_prefill_size=24)
    together = [r.tokens for r in eng.generate(prompts, sp)]
    assert eng.stats.chained_steps > 0                        # drawn tokens stay in the device pipeline too
    alone = [eng.generate([p], sp)[0].tokens for p in prompts]
    assert together == alone
    other = [r.tokens for r in eng.generate(prompts, SamplingParams(temperature=0.8, seed=99, max_tokens=12,
                                                                   ignore_eos=True))]
    assert other != together
    # and they are the tokens the plain sampler draws from the plain model's logits with the same
    # uniform numbers: u(seed, position of the token being chosen), 53 bits of splitmix64 (the
    # generator is written out here, not imported)
    import plain_llama
    M = (1 << 64) - 1

    def draw(seed, position):
        x = ((seed ^ ((position * 0x9E3779B97F4A7C15) & M)) + 0x9E3779B97F4A7C15) & M
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
        return ((x ^ (x >> 31)) >> 11) / float(1 << 53)

    plain = models["B"][1]
    for p, got in zip(prompts, together):
        seq = list(p)
        for t in got:
            row = plain.logits(seq)[-1]
            assert t == plain_llama.sample_filtered(row, 0.8, 0, 1.0, 0.0, draw(1234, len(seq)))
            seq.append(t)


def test_preemption_recomputes_to_the_same_tokens(models):
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, _ = models["A"]
    V = TINY["A"]["vocab_size"]
    prompts = [random_ids(6, V, 80 + i) for i in range(3)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    roomy = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=64, paged_block_size=4, num_blocks=48)
    tight = Engine(folder, dtype="float32", max_batch_seqs=3, max_model_len=64, paged_block_size=4, num_blocks=8)
    a = roomy.generate(prompts, sp)
    b = tight.generate(prompts, sp)
    assert tight.stats.preemptions > 0 and roomy.stats.preemptions == 0
    assert [x.tokens for x in a] == [x.tokens for x in b]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_decode_graphs_equal_eager_steps(models, name, dtype):
    """Steps of single tokens replayed from a captured graph give the logits of the eager
    step: with rows that change owner, padding rows, a request id that returns with other
    pages, and token ids fed back on the device."""
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    mk = lambda sizes: ModelRunner(folder, dtype=dtype, max_model_len=128, page_size=8, num_pages=48,
                                   max_batch_seqs=4, max_batch_tokens=128, capture_sizes=sizes)
    eager, graph = mk(None), mk([1, 2, 4])
    assert not eager.use_graphs and graph.use_graphs
    expect_fast_kernels(graph, name)
    seqs = {i: random_ids(40 + 7 * i, V, 200 + i) for i in range(5)}
    for r in (eager, graph):
        r.got = {i: [] for i in seqs}
        for i in (0, 1, 2):
            r.open(i)
            r.got[i].append(r.step([StepEntry(i, seqs[i][:9 + i], list(range(9 + i)))]))
    at = {0: 9, 1: 10, 2: 11}
    live = [0, 1, 2]
    nxt = 3
    for turn in range(2000):
        if not live:
            break
        batch = [i for i in live if (turn + i) % 4 != 3] or live[:1]      # 1 to 3 rows: buckets 1, 2, 4
        for r in (eager, graph):
            lg = r.step([StepEntry(i, [seqs[i][at[i]]], [0]) for i in batch])
            for k, i in enumerate(batch):
                r.got[i].append(lg[k: k + 1])
        for i in batch:
            at[i] += 1
            if at[i] == len(seqs[i]):
                live.remove(i)
                for r in (eager, graph):
                    r.close(i)
                if nxt < 5:                                               # a new request takes the row
                    for r in (eager, graph):
                        r.open(nxt)
                        r.got[nxt].append(r.step([StepEntry(nxt, seqs[nxt][:5], list(range(5)))]))
                    at[nxt] = 5
                    live.append(nxt)
                    nxt += 1
    assert graph.graph_replays > 50 and sorted(graph._graphs) == [1, 2, 4]
    for i in seqs:
        e, g = torch.cat(eager.got[i]), torch.cat(graph.got[i])
        assert rel_err(g, plain.logits(seqs[i])) <= TOL[dtype]
        if dtype == "float32":
            assert torch.equal(e, g)
    # the same id again, on other pages, with device-fed tokens
    graph.open(0), graph.open(99)
    graph.step([StepEntry(99, seqs[1][:20], [])])
    graph.step([StepEntry(0, seqs[0][:6], [])])
    toks = torch.tensor(seqs[0][6:12], dtype=torch.int32, device="cuda:0")
    outs = [graph.step([StepEntry(0, [0], [0])], device_tokens=toks[k: k + 1]) .clone() for k in range(6)]
    assert rel_err(torch.cat(outs), plain.logits(seqs[0])[6:12]) <= TOL[dtype]


def test_stop_ids_end_generation_where_the_plain_model_says(models, tmp_path):
    """Stop ids from config.json end a request at the first of them (unless ignored); the
    device-side stop check and the host agree on every token, also while steps are chained."""
    import json
    import shutil
    import plain_llama
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    folder, plain = models["A"]
    V = TINY["A"]["vocab_size"]
    prompts = [random_ids(n, V, 300 + n) for n in (4, 9, 15, 2, 11, 6)]
    free_run = [plain_llama.greedy_generate(plain.cfg, plain.w, p, 24) for p in prompts]
    # stop ids: for each sequence, a token from the middle of its free-running continuation
    eos = sorted({seq[8 + i] for i, seq in enumerate(free_run)})
    stop_folder = str(tmp_path / "with_eos")
    shutil.copytree(folder, stop_folder)
    cfg = dict(plain.cfg, eos_token_id=eos)
    with open(os.path.join(stop_folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    eng = Engine(stop_folder, dtype="float32", max_batch_tokens=64, max_batch_seqs=4, max_model_len=64,
                 paged_block_size=8, num_blocks=40)
    res = eng.generate(prompts, SamplingParams(max_tokens=24))
    for seq, out in zip(free_run, res):
        cut = next((i for i, t in enumerate(seq) if t in eos), None)
        want = seq if cut is None else seq[: cut + 1]
        assert out.tokens == want
        assert out.finish_reason == ("length" if cut is None else "stop")
    assert any(o.finish_reason == "stop" for o in res)
    assert eng.stats.stop_flag_mismatches == 0
    ignored = eng.generate(prompts[:2], SamplingParams(max_tokens=24, ignore_eos=True))
    assert [o.tokens for o in ignored] == free_run[:2] and eng.stats.stop_flag_mismatches == 0
    assert eng.runner.cache.free_pages() == {0: 40}


@pytest.mark.parametrize("name", FAST)
def test_long_decoding_on_the_tma_fed_attention_with_and_without_dependent_launch(models, name):
    """Decoding at 450 to 640 keys with two key ranges of five 64-key tiles each: the decode
    attention's TMA thread sends its first tiles before it waits for the kernel that wrote this
    step's key, which is only right if that kernel (the chain that ends in the rotary encoding
    and the cache write) is the sole writer of anything those tiles hold.  Run eagerly and from
    captured graphs, with programmatic dependent launch on and off, three requests side by side
    (one padding row in the bucket of four); every decoded position against the plain model.
    The models are sharp, so a key read before it was written moves the logits by tenths."""
    from rustinfer_b200.engine.runner import ModelRunner, StepEntry
    from rustinfer_b200.ops import library
    folder, plain = models[name]
    V = TINY[name]["vocab_size"]
    lens, tail = [640, 450, 577], 60
    seqs = [random_ids(n, V, 900 + i) for i, n in enumerate(lens)]
    refs = [plain.logits(s) for s in seqs]
    results = {}
    try:
        for pdl in (True, False):
            library.set_pdl(pdl)
            for sizes in (None, [1, 2, 4]):
                r = ModelRunner(folder, dtype="bfloat16", max_model_len=704, page_size=16, num_pages=3 * 44 + 8,
                                max_batch_seqs=4, max_batch_tokens=1024, capture_sizes=sizes)
                expect_fast_kernels(r, name)
                for b in r.model.blocks:
                    b.mixer.MAX_SPLITS = 2                      # ranges of five tiles: more than the ring holds
                got = [[] for _ in seqs]
                for i, s in enumerate(seqs):
                    r.open(i)
                    r.step([StepEntry(i, s[: lens[i] - tail], [])])
                for t in range(tail):
                    lg = r.step([StepEntry(i, [s[lens[i] - tail + t]], [0]) for i, s in enumerate(seqs)])
                    for i in range(len(seqs)):
                        got[i].append(lg[i: i + 1])
                torch.cuda.synchronize()
                r.check_kernel_errors()
                assert (sizes is None) == (r.graph_replays == 0)
                for i in range(len(seqs)):
                    out = torch.cat(got[i])
                    assert rel_err(out, refs[i][lens[i] - tail:]) <= TOL["bfloat16"], (name, pdl, sizes, i)
                results[(pdl, sizes is not None)] = [torch.cat(g) for g in got]
    finally:
        library.set_pdl(True)
    # the four ways agree with one another far below what a misplaced key would do (they differ
    # only in the order in which K slices were added into the fp32 stream)
    base = results[(True, True)]
    for key, outs in results.items():
        for a, b in zip(base, outs):
            assert rel_err(b, a) <= TOL["bfloat16"] / 2, key
