"""Decode and prefill throughput of the engine on one B200, in the contract's one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--shape 1b|3b|8b]

A step is one decode step of the whole batch.  The default run has the layer sizes of the
Llama-3.2-1B-shaped benchmark configuration with random weights ~N(0, 0.02) (seed 2), a
batch of 8 and a context that reaches 4,096 tokens.  `value` is decoded tokens a second
timed on the device over K steps fed with the previous step's tokens on the device; `e2e`
is the same through `Engine.add_request` / `Engine.step`, host token ids in and out.
Every timed window is repeated (five times for the headline) and the median is reported with the
smallest and largest beside it.  Also reported: a 2,048-token prefill, the decode step against the
HBM roofline, clocks sampled while timing, how many of this package's kernels ran, and under
`points`: decode and end-to-end decode at batch 1 and 64, decode at batch 8 with temperature
sampling, the Llama-3.1-8B-shaped model at 8 of its 32 layers (decode at batch 1, 8, 64, a
2,048-token prefill, one 32,768-token prompt in portions of 8,192 with the share of time spent in
attention), the Llama-3.2-3B-shaped model at 8 of its 28 layers serving 64 requests at once, and
this engine's attention and GEMM kernels timed against the reference's own attention kernels
(compiled unmodified, see baseline/reference_kernels.py) and the library GEMM on the same data.
`--shape` takes the layer sizes of the 3B or 8B benchmark configuration for the headline instead;
`--only decode|prefill|serve` runs one part alone and prints its time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

def _llama(layers, hidden, heads, kv_heads, head_dim, inter, factor, tied):
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=layers,
                hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                intermediate_size=inter, vocab_size=128256, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=tied, max_position_embeddings=131072)


# the benchmark configurations: the Llama-3.2-1B shape is the default and the headline; the
# 3B and 8B shapes are there for --shape (further sizes, head size 128, an untied head)
SHAPES = {"1b": ("Llama-3.2-1B-shaped", _llama(16, 2048, 32, 8, 64, 8192, 32.0, True)),
          "3b": ("Llama-3.2-3B-shaped", _llama(28, 3072, 24, 8, 128, 8192, 32.0, True)),
          "8b": ("Llama-3.1-8B-shaped", _llama(32, 4096, 32, 8, 128, 14336, 8.0, False))}
SEED, STD = 2, 0.02
CONTEXT, PREFILL_TOKENS, PAGE = 4096, 2048, 16
# Decode steps run untimed between the burst that fills the context and the warm-up: for some 80
# steps after such a burst a step takes up to 14 % longer (1.20, 1.14, 1.11, 1.07, 1.06, 1.055 ms in
# windows of 16 steps at batch 8), the GPU's clocks coming back from the burst's power draw; what
# is measured is the steady state the metric names.
SETTLE_STEPS = 96
NOMINAL_HBM_GBS, NOMINAL_BF16_TFLOPS = 6650.0, 1590.0      # fallback when no measured peaks are given


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return NOMINAL_HBM_GBS, NOMINAL_BF16_TFLOPS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        # the timed regions are tens of milliseconds long and follow one another closely:
        # every sample from the first region's start to the last one's end was taken under load
        if windows:
            windows = [(min(a for a, _ in windows), max(b for _, b in windows))]
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, c in self.rows:
            if len(c) < 7 or not any(a <= t <= b for a, b in windows):
                continue
            try:
                sm.append(float(c[0])); mx = max(mx, float(c[1]))
            except ValueError:
                continue
            for n, v in zip(names, c[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers):
    d, inter, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * inter
    weight_bytes = 2 * (layers * (per_layer + 2 * d) + V * d + d)       # bf16; the head is the tied table
    kv_bytes_per_token = layers * 2 * kv * 2
    return per_layer, weight_bytes, kv_bytes_per_token, q


def fill_context(engine, batch, ctx0, vocab, seed):
    """Open `batch` requests and bring each to ctx0 cached tokens through the step function."""
    import random
    from rustinfer_b200.engine.runner import StepEntry
    r = engine.runner
    rng = random.Random(seed)
    ids = []
    for b in range(batch):
        rid = ("bench", seed, b)
        r.open(rid)
        ids.append(rid)
        at = 0
        while at < ctx0:
            n = min(ctx0 - at, r.max_batch_tokens)
            r.step([StepEntry(rid, [rng.randrange(vocab) for _ in range(n)], [])])
            at += n
    return ids


def median_of(run, repeats):
    """`run()` -> (ms, ...): the run whose ms is the median of `repeats` runs, with all the ms."""
    runs = sorted((run() for _ in range(repeats)), key=lambda r: r[0])
    return runs[len(runs) // 2], [round(r[0], 4) for r in runs]


def decode_device_timed(engine, batch, steps, warmup, vocab, seed, context=CONTEXT, sampling=None):
    """K decode steps of `batch` requests that end at `context` tokens; device time.  With
    `sampling` (SamplingParams) every row's token is drawn on the device instead of the argmax."""
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.ops import library
    r = engine.runner
    settle = min(SETTLE_STEPS, max(0, context - (steps + warmup) - 16))     # (a short context leaves less room)
    ctx0 = context - (steps + warmup + settle)
    ids = fill_context(engine, batch, ctx0, vocab, seed)
    tokens = torch.randint(0, vocab, (batch,), dtype=torch.int32, device=r.device)
    entries = [StepEntry(rid, [0], [0]) for rid in ids]

    at = [ctx0]

    def one():
        nonlocal tokens
        logits = r.step(entries, device_tokens=tokens)
        if sampling is None:
            tokens = engine.sampler.argmax_device(logits)
        else:
            at[0] += 1
            tokens = engine.sampler.sample_device(logits, [sampling] * batch, list(range(batch)), [at[0]] * batch)

    r_step = r.step
    r.step = lambda e, device_tokens=None: r_step(e, device_tokens=device_tokens, borrow_logits=True)
    for _ in range(settle + warmup):
        one()
    torch.cuda.synchronize()
    l0 = library.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    w1 = time.time()
    ms = e0.elapsed_time(e1)
    launches = library.launch_count - l0
    r.step = r_step
    for rid in ids:
        r.close(rid)
    return ms / steps, launches, (w0, w1)


def decode_e2e(engine, batch, steps, warmup, vocab, seed, trace=False):
    """The same decode steps through the public entry point: host token ids in and out.  With
    `trace`, `engine.stats.host_seconds` holds the host's time in the timed steps afterwards."""
    import random
    import torch
    from rustinfer_b200.sampling.params import SamplingParams
    rng = random.Random(seed)
    # requests whose prompt is done keep decoding while the others' prompts are computed, so
    # leave room for those extra tokens and end nothing inside the timed region
    ctx0 = CONTEXT - (steps + warmup + SETTLE_STEPS) - 4 * batch - 8
    if batch > 8:                                            # prompts of 64 requests take many steps of 8,192 tokens
        ctx0 = CONTEXT - (steps + warmup + SETTLE_STEPS) - (batch * CONTEXT) // 8192 - batch - 16
    sp = SamplingParams(max_tokens=CONTEXT, ignore_eos=True)
    for _ in range(batch):
        engine.add_request([rng.randrange(vocab) for _ in range(ctx0)], sp)
    while any(q.computed < len(q.prompt) for q in engine._requests.values()):
        engine.step()                                       # prompts (untimed)
    for _ in range(SETTLE_STEPS + warmup):
        engine.step()
    torch.cuda.synchronize()
    if trace:
        engine.stats.host_seconds.clear()
        engine.trace_host = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    got = 0
    for _ in range(steps - 1):
        got += len(engine.step())
    e1.record()
    engine.trace_host = False
    torch.cuda.synchronize()
    w1 = time.time()
    ms = e0.elapsed_time(e1) / (steps - 1)
    h2d = engine.runner.h2d_bytes_last
    for rid in list(engine._requests):
        engine.abort(rid)
    torch.cuda.synchronize()
    assert got == batch * (steps - 1), (got, batch, steps)
    return ms, h2d, batch * 8, (w0, w1)       # read back per step: a token id and a stop flag per request


def prefill_timed(engine, vocab, tokens, repeats=3):
    import random
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    r = engine.runner
    rng = random.Random(7)
    times, windows = [], []
    for i in range(repeats + 1):                            # the first run warms up
        rid = ("prefill", i)
        r.open(rid)
        prompt = [rng.randrange(vocab) for _ in range(tokens)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        logits = r.step([StepEntry(rid, prompt, [tokens - 1])])
        engine.sampler.argmax_device(logits)
        e1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        ms = e0.elapsed_time(e1)
        r.close(rid)
        if i > 0:
            times.append(ms)
    return statistics.median(times), windows[1:]


def serve_workload(folder, vocab, layers, quiet=False):
    """Continuous batching through the public entry point: 64 requests arrive at once, prompt
    lengths uniform in [128, 2048], 256 tokens out each, prompts computed in portions of 512
    beside the decoding of the others.  Tokens a second over the whole run (host time:
    scheduling, launches and the reading of every token included), and the time from one
    step's launch to the next."""
    import random
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.sampling.params import SamplingParams
    engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64, max_model_len=CONTEXT,
                    paged_block_size=PAGE, chunked_prefill_size=512, num_blocks=64 * 2560 // PAGE,
                    ignore_eos=True)
    rng = random.Random(3)
    prompts = [[rng.randrange(vocab) for _ in range(rng.randint(128, 2048))] for _ in range(64)]
    engine.generate([p[:64] for p in prompts[:8]], SamplingParams(max_tokens=8, ignore_eos=True))   # warm-up
    torch.cuda.synchronize()
    steps0 = engine.stats.steps
    ids = [engine.add_request(p, SamplingParams(max_tokens=256, ignore_eos=True)) for p in prompts]
    marks = []
    t0 = time.perf_counter()
    while engine.has_unfinished():
        engine.step()
        marks.append(time.perf_counter())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    results = [engine.take_finished(i) for i in ids]
    gaps = sorted((b - a) * 1e3 for a, b in zip(marks, marks[1:]))
    n_in, n_out = sum(len(p) for p in prompts), sum(len(r.tokens) for r in results)
    out = {"seconds": round(dt, 4), "out_tok_s": round(n_out / dt, 1), "tok_s": round((n_in + n_out) / dt, 1),
           "steps": engine.stats.steps - steps0, "preemptions": engine.stats.preemptions,
           "step_ms_mean": round(sum(gaps) / len(gaps), 4), "step_ms_p99": round(gaps[int(0.99 * (len(gaps) - 1))], 4),
           "prompt_tokens": n_in, "out_tokens": n_out}
    if not quiet:
        print(f"serve layers{layers}: {len(prompts)} requests, {n_in} prompt tokens, {n_out} tokens out in {dt:.3f} s: "
              f"{n_out / dt:.0f} out tok/s, {(n_in + n_out) / dt:.0f} tok/s in all, {out['steps']} steps "
              f"(mean {out['step_ms_mean']} ms, p99 {out['step_ms_p99']} ms), {out['preemptions']} preemptions")
    del engine
    torch.cuda.empty_cache()
    return out


def long_prompt(folder, vocab, cfg, layers, tokens=32768, portion=8192):
    """One prompt of `tokens` tokens computed in portions through the step function; the time of
    the attention kernels alone is taken with events around every layer's attention."""
    import random
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.parts.attention import GQAAttention
    engine = Engine(folder, dtype="bfloat16", max_batch_tokens=portion, max_batch_seqs=1, max_model_len=tokens + 64,
                    paged_block_size=PAGE, num_blocks=(tokens + 64) // PAGE + 8, capture_sizes=[], ignore_eos=True)
    r = engine.runner
    rng = random.Random(5)
    prompt = [rng.randrange(vocab) for _ in range(tokens)]
    marks = []
    plain_attend = GQAAttention.attend

    def timed_attend(self, q, step, cache, out=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        res = plain_attend(self, q, step, cache, out)
        e1.record()
        marks.append((e0, e1))
        return res

    best = None
    for rep in range(2):                                    # the first run warms up
        r.open(("long", rep))
        marks.clear()
        GQAAttention.attend = timed_attend if rep == 1 else plain_attend
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for at in range(0, tokens, portion):
            n = min(portion, tokens - at)
            logits = r.step([StepEntry(("long", rep), prompt[at: at + n], [n - 1] if at + n == tokens else [])])
        engine.sampler.argmax_device(logits)
        e1.record()
        torch.cuda.synchronize()
        best = e0.elapsed_time(e1)
        r.close(("long", rep))
    GQAAttention.attend = plain_attend
    attn_ms = sum(a.elapsed_time(b) for a, b in marks)
    per_layer, _, _, q_dim = model_numbers(cfg, layers)
    flops = 2 * tokens * layers * per_layer + 2 * vocab * cfg["hidden_size"] + 2 * tokens * tokens * q_dim * layers
    del engine
    torch.cuda.empty_cache()
    return {"ms": round(best, 2), "tok_s": round(tokens / best * 1e3, 1), "attention_share": round(attn_ms / best, 4),
            "tflops": round(flops / (best * 1e-3) / 1e12, 1)}


def time_kernel(fn, repeats=20, flush=None):
    """Median device time of fn() in microseconds; `flush` (a large tensor) is rewritten between
    runs so that nothing of the last run stays in L2."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(repeats):
        if flush is not None:
            flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(times)


def kernel_ratios():
    """This engine's attention kernels against the reference's own (compiled unmodified, called
    through their C launchers with the cache laid out their way), and its tcgen05 GEMM against the
    library's, on the same data.  reference time / own time: above 1, this engine's kernel is the
    faster.  The reference's kernels are absent where baseline/_ref was never built: null then."""
    import math
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_kernels as R
    from rustinfer_b200.ops import kernels as K
    dev = torch.device("cuda:0")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    out = {}
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)           # 256 MB: twice the L2
    have_ref = R.load() is not None
    g = torch.Generator(device="cuda").manual_seed(1)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for tag, (Hq, Hkv, hd) in {"1b": (32, 8, 64), "8b": (32, 8, 128)}.items():
        scale = 1 / math.sqrt(hd)
        # ---- decode: 8 requests at 4,096 keys
        B, ctx = 8, CONTEXT
        blocks = ctx // PAGE
        cache = torch.randn(B * blocks, 2, Hkv, PAGE, hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        table = torch.randperm(B * blocks, device=dev).to(torch.int32).view(B, blocks).contiguous()
        q = torch.randn(B, Hq * hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        o = torch.empty_like(q)
        kv_len, cu = i32([ctx] * B), i32(list(range(B + 1)))
        from rustinfer_b200.parts.base import MIXERS, BuildContext
        from rustinfer_b200.parts.spec import PartSpec
        part = MIXERS.build(PartSpec("gqa_attention", {"hidden_size": 64, "num_heads": Hq, "num_kv_heads": Hkv,
                                                       "head_dim": hd, "scale": scale, "window": None, "position": None}))
        part.prepare(BuildContext(dev, torch.bfloat16, ctx, PAGE, max_batch_seqs=64, num_sms=sms))
        splits = part._splits(B, ctx)
        no, nl = K.decode_scratch_floats(B, Hq, hd, splits)
        po, pl = torch.empty(no, device=dev), torch.empty(nl, device=dev)
        own = time_kernel(lambda: K.attention_decode_bf16(q, o, cache, table, cu, kv_len, None, B, Hq, Hkv, hd, scale,
                                                          None, splits, po, pl), flush=flush)
        out[f"attn_decode_{tag}_b8_us"] = round(own, 1)
        if have_ref:
            kp, vp = R.pools_from_pages(cache, PAGE)
            ws = R.decode_workspace(B, Hq, hd)
            o2 = torch.empty_like(q)
            ref = time_kernel(lambda: R.paged_decode(q, kp, vp, o2, table, kv_len, ws, Hq, Hkv, hd, scale, sms,
                                                     [ctx] * B), flush=flush)
            out[f"attn_decode_{tag}_b8_ref_us"] = round(ref, 1)
            out[f"attn_decode_{tag}_b8_vs_ref"] = round(ref / own, 2)
            del kp, vp
        # ---- prompt portion: one request of 2,048 tokens
        T = PREFILL_TOKENS
        qp = torch.randn(T, Hq * hd, generator=g, device=dev, dtype=torch.float32).bfloat16()
        op = torch.empty_like(qp)
        kvl, cup = i32([T]), i32([0, T])
        tbl = table[:1, : T // PAGE].contiguous()
        tc = K.tc_attention_supports(Hq, Hkv, hd, PAGE)
        tpt = K.tc_tokens_per_tile(Hq, Hkv) if tc else K.mma_tokens_per_tile(Hq, Hkv)
        te, tq = i32([0] * (T // tpt)), i32(list(range(0, T, tpt)))
        fn = K.attention_prefill_tc if tc else K.attention_prefill_bf16
        own = time_kernel(lambda: fn(qp, op, cache, tbl, cup, kvl, te, tq, Hq, Hkv, hd, scale, None), flush=flush)
        out[f"attn_prefill_{tag}_2048_us"] = round(own, 1)
        if have_ref:
            kp, vp = R.pools_from_pages(cache, PAGE)
            tiles = R.prefill_tiles([T])
            o2 = torch.empty_like(qp)
            ref = time_kernel(lambda: R.paged_prefill(qp, kp, vp, o2, tbl, kvl, cup, tiles, [T], [T], Hq, Hkv, hd, scale),
                              flush=flush)
            out[f"attn_prefill_{tag}_2048_ref_us"] = round(ref, 1)
            out[f"attn_prefill_{tag}_2048_vs_ref"] = round(ref / own, 2)
            del kp, vp
        del cache
    # ---- GEMM: the 2,048-token products of the 1B shape against the library's
    for name, (M, N, Kd) in {"qkv": (2048, 3072, 2048), "gate_up": (2048, 16384, 2048), "down": (2048, 2048, 8192),
                             "square8192": (8192, 8192, 8192)}.items():
        x = (torch.randn(M, Kd, generator=g, device=dev) * 0.5).bfloat16()
        w = (torch.randn(N, Kd, generator=g, device=dev) * 0.02).bfloat16()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        own = time_kernel(lambda: K.gemm_tc(x, w, y, K.EPI_BF16, num_sms=sms), flush=flush)
        lib = time_kernel(lambda: torch.mm(x, w.t(), out=y), flush=flush)
        out[f"gemm_{name}_tflops"] = round(2 * M * N * Kd / own / 1e6, 1)
        out[f"gemm_{name}_vs_library"] = round(lib / own, 2)
        del x, w, y
    del flush
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes (default: the 1B shape)")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true", help="leave out everything under `points`")
    ap.add_argument("--repeats", type=int, default=5, help="timed windows of the headline (the median is reported)")
    ap.add_argument("--only", choices=["decode", "prefill", "serve", "e2e"],
                    help="run one part alone and print its time (for profiler captures; no JSON line); "
                         "serve: 64 requests, prompts of 128 to 2,048 tokens, 256 tokens out each, "
                         "prompt portions of 512, through Engine.generate; e2e: the decode steps through "
                         "Engine.step with host tokens in and out, and where the host's time in a step goes")
    ap.add_argument("--eager", action="store_true", help="with --only decode: no CUDA graphs")
    ap.add_argument("--sampled", action="store_true",
                    help="with --only decode: every token drawn (temperature 0.8, top-k 50, top-p 0.9) instead of the argmax")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only: context the decode ends at")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only prefill: length of the prompt, computed in one step (up to 8192)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: --gpus {args.gpus} is not supported by this engine")
        return 2
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip install of the reference fails at metadata generation (a Rust workspace whose "
                          "pyproject.toml declares no Python package) and no cargo/rustc is in this image"}))
        return 0
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 2)

    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.weights.random_init import write_random_model

    hbm_gbs, bf16_tflops, peak_kind = peaks()
    shape_name, shape = SHAPES[args.shape]
    if args.layers <= 0:
        args.layers = shape["num_hidden_layers"]
    cfg = dict(shape, num_hidden_layers=args.layers)
    vocab = cfg["vocab_size"]
    per_layer, weight_bytes, kv_per_token, q_dim = model_numbers(cfg, args.layers)
    clocks = ClockSampler()
    clocks.start()
    windows = []
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=SEED, std=STD)
        if args.only == "serve":
            serve_workload(folder, vocab, args.layers)
            clocks.stop()
            return 0
        if args.only:
            seqs = max(args.batch, 1)
            longest = max(CONTEXT, min(args.prompt_tokens, 8192))
            engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=seqs,
                            max_model_len=longest, paged_block_size=PAGE, num_blocks=seqs * longest // PAGE + 64,
                            capture_sizes=[] if args.eager else [1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
            if args.only == "e2e":
                decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, 1)          # graphs captured: untimed
                ms, _, _, _ = decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, 2, trace=True)
                host = dict(engine.stats.host_seconds)
                ms_dev, _, _ = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 3)
                print(f"e2e b{args.batch} layers{args.layers}: {ms:.4f} ms/step through Engine.step, {ms_dev:.4f} device-timed")
                n = args.steps - 1
                for what, sec in host.items():
                    print(f"  host, {what}: {sec / n * 1e6:8.1f} us a step")
                busy = sum(sec for what, sec in host.items() if not what.startswith("wait"))
                print(f"  host busy {busy / n * 1e6:.1f} us of the step's {ms * 1e3:.1f} us; the rest it waits for the GPU")
            elif args.only == "decode":
                global_ctx = args.context
                sp = None
                if args.sampled:
                    from rustinfer_b200.sampling.params import SamplingParams
                    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1, max_tokens=CONTEXT, ignore_eos=True)
                ms, n, _ = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 1, global_ctx, sampling=sp)
                print(f"decode b{args.batch} ctx{global_ctx} layers{args.layers}{' sampled' if sp else ''}: {ms:.4f} ms/step, {n} launches")
            else:
                tokens = max(2, min(args.prompt_tokens, 8192))
                ms, _ = prefill_timed(engine, vocab, tokens, repeats=max(1, min(args.steps, 3)))
                print(f"prefill {tokens} layers{args.layers}: {ms:.3f} ms")
            clocks.stop()
            return 0
        engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64,
                        max_model_len=CONTEXT, paged_block_size=PAGE, chunked_prefill_size=0,
                        num_blocks=64 * CONTEXT // PAGE + 64, capture_sizes=[1, 2, 4, 8, 16, 32, 64],
                        ignore_eos=True)
        say = lambda msg: print(f"[bench] {msg}", file=sys.stderr, flush=True)
        reps = args.repeats
        seeds = iter(range(100, 10_000))
        # ---- the headline: K decode steps at the asked batch, device-timed, repeated
        (ms_step, launches, w), decode_ms = median_of(
            lambda: decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, next(seeds)), reps)
        windows.append(w)
        say(f"decode b{args.batch}: {ms_step:.4f} ms/step (of {decode_ms})")
        (e2e_ms, h2d, d2h, w), e2e_all = median_of(
            lambda: decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, next(seeds)), reps)
        windows.append(w)
        say(f"e2e b{args.batch}: {e2e_ms:.4f} ms/step (of {e2e_all})")
        prefill_ms, pw = prefill_timed(engine, vocab, PREFILL_TOKENS, repeats=reps)
        windows += pw
        say(f"prefill {PREFILL_TOKENS}: {prefill_ms:.3f} ms")
        points = {}
        if not args.skip_points:
            from rustinfer_b200.sampling.params import SamplingParams
            k = max(args.steps, 64)                       # (the headline keeps exactly --steps; these are its company)
            for b in (1, 64):
                (ms_b, _, w), _all = median_of(lambda: decode_device_timed(engine, b, k, args.warmup, vocab, next(seeds)), 3)
                windows.append(w)
                points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
                points[f"decode_b{b}_hbm_frac"] = round(step_bytes_of(cfg, args.layers, b, CONTEXT - k / 2) / (ms_b * 1e-3) / 1e9 / hbm_gbs, 4)
                (ms_e, _, _, w), _all = median_of(lambda: decode_e2e(engine, b, k, args.warmup, vocab, next(seeds)), 3)
                windows.append(w)
                points[f"e2e_b{b}"] = round(b / ms_e * 1e3, 1)
                say(f"decode b{b}: {ms_b:.4f} ms/step, e2e {ms_e:.4f}")
            # the same steps with every token drawn (temperature 0.8, top-k 50, top-p 0.9) instead of the
            # argmax.  Windows of the two kinds alternate and each drawn one is set against the greedy
            # one before it: minutes into a run the clocks under the power cap move a window by
            # several per cent, more than the sampler costs.
            sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1, max_tokens=CONTEXT, ignore_eos=True)
            drawn, ratios = [], []
            for _ in range(3):
                ms_g, _, w = decode_device_timed(engine, args.batch, k, args.warmup, vocab, next(seeds))
                windows.append(w)
                ms_s, _, w = decode_device_timed(engine, args.batch, k, args.warmup, vocab, next(seeds), sampling=sp)
                windows.append(w)
                drawn.append(ms_s)
                ratios.append(ms_g / ms_s)
            ms_s = statistics.median(drawn)
            points[f"decode_b{args.batch}_sampled"] = round(args.batch / ms_s * 1e3, 1)
            points[f"decode_b{args.batch}_sampled_vs_greedy"] = round(statistics.median(ratios), 4)
            say(f"decode b{args.batch} sampled: {ms_s:.4f} ms/step, {statistics.median(ratios):.3f} of greedy windows beside it")
        del engine
        torch.cuda.empty_cache()
    if not args.skip_points and args.shape == "1b":
        points.update(further_shapes(args, hbm_gbs, bf16_tflops, windows, say))
        try:
            points.update(kernel_ratios())
        except Exception as e:                                # the comparison must not cost the headline its line
            points["kernel_ratios_error"] = f"{type(e).__name__}: {e}"[:200]
    clocks.stop()

    value = args.batch / ms_step * 1e3
    mean_ctx = CONTEXT - args.steps / 2
    step_bytes = step_bytes_of(cfg, args.layers, args.batch, mean_ctx)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    T = PREFILL_TOKENS
    prefill_flops = prefill_flops_of(cfg, args.layers, T)
    prefill_frac = prefill_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12)
    out = {
        "metric": f"decode tok/s @ batch {args.batch}, context {CONTEXT} ({shape_name}, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids",
        "config": {"model": shape_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_head": cfg["tie_word_embeddings"],
                   "page_size": PAGE, "prefill_tokens": T, "cuda_graphs": True,
                   "l2": "each step reads %.2f GB of weights and cache, far beyond the 126 MB L2" % (step_bytes / 1e9),
                   "peaks": peak_kind,
                   "windows": f"median of {reps} windows of {args.steps} steps, each after {SETTLE_STEPS} untimed "
                              f"decode steps behind the burst that fills the context, then the warm-up"},
        "spread": {"decode_ms": decode_ms, "e2e_ms": e2e_all},
        "e2e": {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": launches,
        "prefill": {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "clocks": clocks.summary(windows),
    }
    print(json.dumps(out))
    return 0


def step_bytes_of(cfg, layers, batch, mean_ctx):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    _, weight_bytes, kv_per_token, _ = model_numbers(cfg, layers)
    if not cfg["tie_word_embeddings"]:
        weight_bytes += 0                                    # the untied head is the table counted; the embedding is only gathered
    return weight_bytes + batch * mean_ctx * kv_per_token


def prefill_flops_of(cfg, layers, T):
    per_layer, _, _, q_dim = model_numbers(cfg, layers)
    return 2 * T * layers * per_layer + 2 * cfg["vocab_size"] * cfg["hidden_size"] + 2 * T * T * q_dim * layers


def further_shapes(args, hbm_gbs, bf16_tflops, windows, say):
    """The other benchmark configurations, at 8 of their layers each (both numbers are in the
    keys): the 8B shape (decode at batch 1, 8, 64, a 2,048-token prefill, one 32,768-token prompt)
    and the 3B shape serving 64 requests at once."""
    import torch
    from rustinfer_b200.engine.engine import Engine
    from rustinfer_b200.weights.random_init import write_random_model
    out = {}
    seeds = iter(range(20_000, 30_000))
    # (windows as long as the headline's: the steps right after the burst that fills the context run
    # several per cent slower than the ones that follow, and a short window is mostly those)
    k = max(args.steps, 64)
    # ---- Llama-3.1-8B-shaped, 8 of 32 layers
    name, shape = SHAPES["8b"]
    layers = 8
    cfg = dict(shape, num_hidden_layers=layers)
    tag = f"8b_l{layers}of{shape['num_hidden_layers']}"
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=4, std=STD)
        engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64, max_model_len=CONTEXT,
                        paged_block_size=PAGE, num_blocks=64 * CONTEXT // PAGE + 64,
                        capture_sizes=[1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
        for b in (1, 8, 64):
            (ms_b, _, w), _all = median_of(lambda: decode_device_timed(engine, b, k, args.warmup, cfg["vocab_size"], next(seeds)), 3)
            windows.append(w)
            out[f"{tag}_decode_b{b}"] = round(b / ms_b * 1e3, 1)
            out[f"{tag}_decode_b{b}_hbm_frac"] = round(step_bytes_of(cfg, layers, b, CONTEXT - k / 2) / (ms_b * 1e-3) / 1e9 / hbm_gbs, 4)
            say(f"{tag} decode b{b}: {ms_b:.4f} ms/step")
        ms_p, pw = prefill_timed(engine, cfg["vocab_size"], PREFILL_TOKENS, repeats=3)
        windows += pw
        out[f"{tag}_prefill_2048"] = round(PREFILL_TOKENS / ms_p * 1e3, 1)
        out[f"{tag}_prefill_2048_tc_frac"] = round(prefill_flops_of(cfg, layers, PREFILL_TOKENS) / (ms_p * 1e-3) / (bf16_tflops * 1e12), 4)
        say(f"{tag} prefill 2048: {ms_p:.3f} ms")
        del engine
        torch.cuda.empty_cache()
        w0 = time.time()
        lp = long_prompt(folder, cfg["vocab_size"], cfg, layers)
        windows.append((w0, time.time()))
        out[f"{tag}_prompt_32768"] = lp["tok_s"]
        out[f"{tag}_prompt_32768_attention_share"] = lp["attention_share"]
        out[f"{tag}_prompt_32768_tc_frac"] = round(lp["tflops"] / bf16_tflops, 4)
        say(f"{tag} prompt of 32,768: {lp['ms']} ms, attention {lp['attention_share']:.0%}")
    # ---- Llama-3.2-3B-shaped, 8 of 28 layers: 64 requests at once through Engine
    name, shape = SHAPES["3b"]
    cfg = dict(shape, num_hidden_layers=layers)
    tag = f"3b_l{layers}of{shape['num_hidden_layers']}"
    with tempfile.TemporaryDirectory(prefix="rustinfer_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "model"), cfg, seed=3, std=STD)
        w0 = time.time()
        sv = serve_workload(folder, cfg["vocab_size"], layers, quiet=True)
        windows.append((w0, time.time()))
        out[f"{tag}_serve64_tok_s"] = sv["tok_s"]
        out[f"{tag}_serve64_out_tok_s"] = sv["out_tok_s"]
        out[f"{tag}_serve64_step_ms_mean"] = sv["step_ms_mean"]
        out[f"{tag}_serve64_step_ms_p99"] = sv["step_ms_p99"]
        out[f"{tag}_serve64_preemptions"] = sv["preemptions"]
        say(f"{tag} serve: {sv}")
    return out


if __name__ == "__main__":
    sys.exit(main())
