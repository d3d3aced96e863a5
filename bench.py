"""Decode and prefill throughput of the engine on one B200, in the contract's one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--shape 1b|3b|8b]

A step is one decode step of the whole batch.  The default run has the layer sizes of the
Llama-3.2-1B-shaped benchmark configuration with random weights ~N(0, 0.02) (seed 2), a
batch of 8 and a context that reaches 4,096 tokens.  `value` is decoded tokens a second
timed on the device over K steps fed with the previous step's tokens on the device; `e2e`
is the same through `Engine.add_request` / `Engine.step`, host token ids in and out.
Also reported: a 2,048-token prefill, the decode step against the HBM roofline, decode at
batch 1 and 64, clocks sampled while timing, and how many of this package's kernels ran.
`--shape` takes the layer sizes of the 3B or 8B benchmark configuration instead; `--only
decode|prefill|serve` runs one part alone and prints its time.
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


def decode_device_timed(engine, batch, steps, warmup, vocab, seed, context=CONTEXT):
    """K decode steps of `batch` requests that end at `context` tokens; device time."""
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    from rustinfer_b200.ops import library
    r = engine.runner
    ctx0 = context - (steps + warmup)
    ids = fill_context(engine, batch, ctx0, vocab, seed)
    tokens = torch.randint(0, vocab, (batch,), dtype=torch.int32, device=r.device)
    entries = [StepEntry(rid, [0], [0]) for rid in ids]

    def one():
        nonlocal tokens
        logits = r.step(entries, device_tokens=tokens)
        tokens = engine.sampler.argmax_device(logits)

    r_step = r.step
    r.step = lambda e, device_tokens=None: r_step(e, device_tokens=device_tokens, borrow_logits=True)
    for _ in range(warmup):
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


def decode_e2e(engine, batch, steps, warmup, vocab, seed):
    """The same decode steps through the public entry point: host token ids in and out."""
    import random
    import torch
    from rustinfer_b200.sampling.params import SamplingParams
    rng = random.Random(seed)
    # requests whose prompt is done keep decoding while the others' prompts are computed, so
    # leave room for those extra tokens and end nothing inside the timed region
    ctx0 = CONTEXT - (steps + warmup) - 4 * batch - 8
    sp = SamplingParams(max_tokens=CONTEXT, ignore_eos=True)
    for _ in range(batch):
        engine.add_request([rng.randrange(vocab) for _ in range(ctx0)], sp)
    while any(q.computed < len(q.prompt) for q in engine._requests.values()):
        engine.step()                                       # prompts (untimed)
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    got = 0
    for _ in range(steps - 1):
        got += len(engine.step())
    e1.record()
    torch.cuda.synchronize()
    w1 = time.time()
    ms = e0.elapsed_time(e1) / (steps - 1)
    h2d = engine.runner.h2d_bytes_last
    for rid in list(engine._requests):
        engine.abort(rid)
    assert got == batch * (steps - 1), (got, batch, steps)
    return ms, h2d, batch * 8, (w0, w1)       # read back per step: a token id and a stop flag per request


def prefill_timed(engine, vocab, tokens, repeats=3):
    import random
    import torch
    from rustinfer_b200.engine.runner import StepEntry
    r = engine.runner
    rng = random.Random(7)
    best, windows = None, []
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
            best = ms if best is None else min(best, ms)
    return best, windows[1:]


def serve_workload(folder, vocab, layers):
    """Continuous batching through the public entry point: 64 requests arrive at once, prompt
    lengths uniform in [128, 2048], 256 tokens out each, prompts computed in portions of 512
    beside the decoding of the others.  Prints tokens a second over the whole run (host time:
    scheduling, launches and the reading of every token included)."""
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
    t0 = time.perf_counter()
    results = engine.generate(prompts, SamplingParams(max_tokens=256, ignore_eos=True))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_in, n_out = sum(len(p) for p in prompts), sum(len(r.tokens) for r in results)
    print(f"serve layers{layers}: {len(prompts)} requests, {n_in} prompt tokens, {n_out} tokens out in {dt:.3f} s: "
          f"{n_out / dt:.0f} out tok/s, {(n_in + n_out) / dt:.0f} tok/s in all, {engine.stats.steps - steps0} steps, "
          f"{engine.stats.preemptions} preemptions")


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
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--only", choices=["decode", "prefill", "serve"],
                    help="run one part alone and print its time (for profiler captures; no JSON line); "
                         "serve: 64 requests, prompts of 128 to 2,048 tokens, 256 tokens out each, "
                         "prompt portions of 512, through Engine.generate")
    ap.add_argument("--eager", action="store_true", help="with --only decode: no CUDA graphs")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only: context the decode ends at")
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
            engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=seqs,
                            max_model_len=CONTEXT, paged_block_size=PAGE, num_blocks=seqs * CONTEXT // PAGE + 64,
                            capture_sizes=[] if args.eager else [1, 2, 4, 8, 16, 32, 64], ignore_eos=True)
            if args.only == "decode":
                global_ctx = args.context
                ms, n, _ = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 1, global_ctx)
                print(f"decode b{args.batch} ctx{global_ctx} layers{args.layers}: {ms:.4f} ms/step, {n} launches")
            else:
                ms, _ = prefill_timed(engine, vocab, PREFILL_TOKENS, repeats=max(1, min(args.steps, 3)))
                print(f"prefill {PREFILL_TOKENS} layers{args.layers}: {ms:.3f} ms")
            clocks.stop()
            return 0
        engine = Engine(folder, dtype="bfloat16", max_batch_tokens=8192, max_batch_seqs=64,
                        max_model_len=CONTEXT, paged_block_size=PAGE, chunked_prefill_size=0,
                        num_blocks=64 * CONTEXT // PAGE + 64, capture_sizes=[1, 2, 4, 8, 16, 32, 64],
                        ignore_eos=True)
        ms_step, launches, w = decode_device_timed(engine, args.batch, args.steps, args.warmup, vocab, 1)
        windows.append(w)
        print(f"[bench] decode b{args.batch}: {ms_step:.4f} ms/step", file=sys.stderr, flush=True)
        e2e_ms, h2d, d2h, w = decode_e2e(engine, args.batch, args.steps, args.warmup, vocab, 2)
        windows.append(w)
        print(f"[bench] e2e b{args.batch}: {e2e_ms:.4f} ms/step", file=sys.stderr, flush=True)
        prefill_ms, pw = prefill_timed(engine, vocab, PREFILL_TOKENS)
        windows += pw
        print(f"[bench] prefill {PREFILL_TOKENS}: {prefill_ms:.3f} ms", file=sys.stderr, flush=True)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                k = min(args.steps, 64)
                ms_b, _, w = decode_device_timed(engine, b, k, args.warmup, vocab, 10 + b)
                windows.append(w)
                points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
    clocks.stop()

    value = args.batch / ms_step * 1e3
    mean_ctx = CONTEXT - args.steps / 2
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * args.layers * per_layer + 2 * vocab * cfg["hidden_size"] + 2 * T * T * q_dim * args.layers
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
                   "peaks": peak_kind},
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


if __name__ == "__main__":
    sys.exit(main())
