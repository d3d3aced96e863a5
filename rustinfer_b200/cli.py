"""Command line, in RustInfer's manner: every binary of the reference takes
`--config <toml>` (crates/infer-worker/src/bin/worker_main.rs:39-53), and so does this.

    rustinfer --config run.toml            generate for the [[request]] tables of the run file
    rustinfer random-weights --config config.json --seed 0 --out DIR
                                           write a model folder with random weights
    rustinfer replay ...                   the trace replay (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _run(path: str) -> int:
    import tempfile

    from .config.run_config import RunConfig
    from .sampling.params import SamplingParams
    cfg = RunConfig.load(path)
    scratch = None
    if cfg.random_weights:
        from .weights.random_init import write_random_model
        rw = cfg.random_weights
        with open(rw["config"]) as f:
            model_cfg = json.load(f)
        if not cfg.model:                                     # no place named: a folder that goes with the run
            scratch = tempfile.TemporaryDirectory(prefix="rustinfer_b200_random_")
            cfg.model = scratch.name
        write_random_model(cfg.model, model_cfg, int(rw.get("seed", 0)), float(rw.get("std", 0.02)),
                           float(rw.get("norm_std", 0.0)), str(rw.get("dtype", "bfloat16")))
    from .engine.engine import Engine
    engine = Engine.from_run_config(cfg)
    vocab = engine.runner.spec.vocab_size
    prompts: List[List[int]] = []
    import random
    for i, r in enumerate(cfg.requests):
        if "prompt_ids" in r:
            prompts.append([int(t) for t in r["prompt_ids"]])
        elif "random_len" in r:
            rng = random.Random(int(r.get("seed", i)))
            prompts.append([rng.randrange(vocab) for _ in range(int(r["random_len"]))])
        else:
            raise SystemExit(f"[[request]] #{i}: give prompt_ids or random_len")
    if not prompts:
        raise SystemExit("the run file has no [[request]] table")
    s = dict(cfg.sampling)
    params = SamplingParams(temperature=float(s.get("temperature", 0.0)), top_k=int(s.get("top_k", 0)),
                            top_p=float(s.get("top_p", 1.0)), min_p=float(s.get("min_p", 0.0)),
                            seed=s.get("seed"), max_tokens=int(s.get("max_tokens", 16)),
                            ignore_eos=bool(s.get("ignore_eos", cfg.ignore_eos)))
    for res in engine.generate(prompts, params):
        print(json.dumps({"request": res.request_id, "prompt_tokens": len(res.prompt),
                          "tokens": res.tokens, "finish_reason": res.finish_reason}))
    st = engine.stats
    print(json.dumps({"steps": st.steps, "prompt_tokens": st.prompt_tokens,
                      "generated_tokens": st.generated_tokens, "preemptions": st.preemptions,
                      "seconds": round(st.seconds, 4)}), file=sys.stderr)
    if scratch is not None:
        scratch.cleanup()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random-weights":
        ap = argparse.ArgumentParser(prog="rustinfer random-weights")
        ap.add_argument("--config", required=True, help="a config.json of the architecture")
        ap.add_argument("--seed", type=int, default=0)
        ap.add_argument("--std", type=float, default=0.02)
        ap.add_argument("--norm-std", type=float, default=0.0)
        ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
        ap.add_argument("--out", required=True)
        a = ap.parse_args(argv[1:])
        from .weights.random_init import write_random_model
        with open(a.config) as f:
            write_random_model(a.out, json.load(f), a.seed, a.std, a.norm_std, a.dtype)
        print(a.out)
        return 0
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    ap = argparse.ArgumentParser(prog="rustinfer", description=__doc__)
    ap.add_argument("--config", required=True, help="the TOML run file")
    a = ap.parse_args(argv)
    return _run(a.config)


if __name__ == "__main__":
    sys.exit(main())
