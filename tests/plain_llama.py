"""Plain, slow statement of the Llama-3 dense decoder, written from the formulas of
Vinci-hit/RustInfer's sources (each function cites file:line within that project).

Whole sequences, no cache, one function per part, float64 on the CPU.  It shares no
code with ``rustinfer_b200``: it reads ``config.json`` as a raw dict and the weights
through the ``safetensors`` package, so a fault in the framework's own configuration
or loader cannot hide here.

RustInfer's own model code is Rust and no Rust toolchain exists on the build machine, so
the model as a whole could not be run.  Its CUDA kernels could: compiled unmodified and run
on a B200, their outputs on small inputs lie in tests/golden/reference_kernels.safetensors
(made by tests/golden/make_reference_goldens.py), and tests/test_reference_goldens.py holds
the functions of this file to them: rotary tables with llama3 scaling, the rotation,
RMSNorm alone and fused with the residual add, SwiGLU, and paged grouped-query attention for
decoding and for prompt portions.  How the parts are put together (decoder_block,
forward_logits) rests on the formulas.
Where RustInfer's CPU and CUDA back ends disagree (pairing of RoPE elements, tie-break
of argmax) the CUDA definition is taken, since that is what serves requests.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- io
def read_model_folder(folder: str):
    """Raw config dict and name->float64 tensor map of a model folder."""
    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(F64)
    return cfg, weights


def head_dim_of(cfg: dict) -> int:
    # crates/infer-worker/src/bin/worker_main.rs:390-392: head_dim defaults to
    # hidden_size / num_attention_heads when config.json does not give it.
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h[t,:] = E[ids[t],:], no scaling.
    crates/infer-backend-cuda/src/kernels/embedding/emb.cu:9-38;
    crates/infer-backend-cpu/src/lib.rs:533-559 (ids must lie in [0, vocab))."""
    for i in ids:
        if not 0 <= int(i) < table.shape[0]:
            raise ValueError(f"token id {i} outside [0, {table.shape[0]})")
    return table[torch.tensor(list(ids), dtype=torch.long)].to(F64)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i * w_i / sqrt(mean_j x_j^2 + eps); the weight multiplies directly.
    crates/infer-backend-cpu/src/lib.rs:701-728."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = theta^(-2i/head_dim), then the llama3 rescaling by wavelength band.
    crates/infer-worker/src/models/loader.rs:1543-1571.  The scaling is applied only
    when rope_type == "llama3" and the four numbers are present
    (crates/infer-worker/src/bin/worker_main.rs:393-404)."""
    half = head_dim // 2
    f = [1.0 / (theta ** (2.0 * i / head_dim)) for i in range(half)]
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type"))
        keys = ("factor", "low_freq_factor", "high_freq_factor",
                "original_max_position_embeddings")
        if kind == "llama3" and all(k in scaling for k in keys):
            orig = float(scaling["original_max_position_embeddings"])
            low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
            factor = float(scaling["factor"])
            lam_low, lam_high = orig / low, orig / high
            for i in range(half):
                lam = 2.0 * math.pi / f[i]
                if lam < lam_high:
                    pass
                elif lam > lam_low:
                    f[i] = f[i] / factor
                else:
                    s = (orig / lam - low) / (high - low)
                    f[i] = (1.0 - s) * (f[i] / factor) + s * f[i]
    return torch.tensor(f, dtype=F64)


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half on x[T, heads, head_dim]: pair (i, i + hd/2),
    x'_i = x_i c - x_{i+hd/2} s, x'_{i+hd/2} = x_i s + x_{i+hd/2} c, angle = pos * f_i.
    crates/infer-backend-cuda/src/kernels/rope/rope.cu:107-132; table
    crates/infer-worker/src/models/loader.rs:1574-1589."""
    half = x.shape[-1] // 2
    ang = positions.to(F64)[:, None] * inv_freq[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         scale: float, window: Optional[int] = None) -> torch.Tensor:
    """q[T,Hq,hd], k/v[T,Hkv,hd] of one whole sequence.  Row t sees keys 0..t,
    kv head of q head h is h*Hkv//Hq, scores (q.k)*scale, softmax with the maximum
    subtracted, output sum softmax*v.
    crates/infer-core/src/ports/fused_ops.rs:484-523.  RustInfer has no window;
    `window` (keys t-window+1..t) exists for tests of the kernels' mask only."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    out = torch.zeros(T, Hq, hd, dtype=F64)
    for h in range(Hq):
        g = h * Hkv // Hq
        s = (q[:, h, :] @ k[:, g, :].T) * scale                   # [T, T]
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] <= idx[:, None] - window)
        s = s.masked_fill(mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """m_j = silu(gate_j) * up_j, silu(x) = x / (1 + e^-x).
    crates/infer-backend-cuda/src/kernels/swiglu/swiglu.cu:319-325;
    crates/infer-backend-cpu/src/lib.rs:756-774."""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_sublayer(h, w, prefix, cfg, positions, inv_freq, window=None):
    """norm -> q,k,v projections -> RoPE on q and k -> attention -> o projection.
    crates/infer-worker/src/components/attention.rs:83-179; scale 1/sqrt(head_dim)
    crates/infer-worker/src/models/decoder.rs:276."""
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    x = rmsnorm(h, w[prefix + "input_layernorm.weight"], eps)
    T = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).view(T, Hq, hd)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).view(T, Hkv, hd)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).view(T, Hkv, hd)
    q = rope_rotate(q, positions, inv_freq)
    k = rope_rotate(k, positions, inv_freq)
    a = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(hd), window)
    return a.reshape(T, Hq * hd) @ w[prefix + "self_attn.o_proj.weight"].T


def ffn_sublayer(h, w, prefix, cfg):
    """norm -> gate, up -> silu(gate)*up -> down.
    crates/infer-worker/src/components/ffn_dense.rs:39-115."""
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    x = rmsnorm(h, w[prefix + "post_attention_layernorm.weight"], eps)
    m = swiglu(x @ w[prefix + "mlp.gate_proj.weight"].T, x @ w[prefix + "mlp.up_proj.weight"].T)
    return m @ w[prefix + "mlp.down_proj.weight"].T


def decoder_block(h, w, layer, cfg, positions, inv_freq):
    """h = h + Attn(norm(h)); h = h + FFN(norm(h)).
    crates/infer-worker/src/components/decoder_block.rs:13-32 with the deferred
    residual of crates/infer-core/src/component.rs:8-15 written out."""
    p = f"model.layers.{layer}."
    h = h + attention_sublayer(h, w, p, cfg, positions, inv_freq)
    h = h + ffn_sublayer(h, w, p, cfg)
    return h


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence at positions 0..T-1.
    crates/infer-worker/src/models/decoder.rs:68-199: embed, layers in order, final
    norm, head; the head is the embedding table when `lm_head.weight` is absent
    (crates/infer-worker/src/models/decoder.rs:245-262)."""
    hd = head_dim_of(cfg)
    inv_freq = rope_inv_freq(hd, float(cfg.get("rope_theta", 10000.0)), cfg.get("rope_scaling"))
    positions = torch.arange(len(ids))
    h = embedding(w["model.embed_tokens.weight"], ids)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_block(h, w, layer, cfg, positions, inv_freq)
    n = rmsnorm(h, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return n @ head.T


# ------------------------------------------------------------------------ sampling
def argmax_lowest(row: torch.Tensor) -> int:
    """Greedy token; the lowest index wins ties.
    crates/infer-backend-cuda/src/kernels/sampler/sampler.cu:66-78."""
    m = row.max()
    return int(torch.nonzero(row == m)[0, 0])


def sample_filtered(row: torch.Tensor, temperature: float, top_k: int, top_p: float,
                    min_p: float, draw: float) -> int:
    """logit/T -> sort descending -> top-k -> exp(x-max) -> min-p -> normalise ->
    top-p (keep until cumulative >= p, at least one) -> walk the CDF with draw*total.
    crates/infer-worker/src/application/sampler_stack.rs:242-351.  Greedy when
    temperature <= 0, top_k == 1 or top_p <= 0
    (crates/infer-core/src/ports/sampler.rs:43-46).  Equal logits are ordered by
    ascending token id (the reference's unstable sort leaves that open)."""
    if temperature <= 0.0 or top_k == 1 or top_p <= 0.0:
        return argmax_lowest(row)
    vals = [float(x) / float(temperature) for x in row.to(F64).tolist()]
    order = sorted(range(len(vals)), key=lambda i: (-vals[i], i))
    if top_k > 0:
        order = order[: min(top_k, len(order))]
    mx = vals[order[0]]
    weighted = [(i, math.exp(vals[i] - mx)) for i in order]
    if min_p > 0.0:
        thr = weighted[0][1] * min_p
        weighted = [(i, wgt) for i, wgt in weighted if wgt >= thr]
    total = sum(wgt for _, wgt in weighted)
    if top_p < 1.0:
        cum, keep = 0.0, 0
        for _, wgt in weighted:
            cum += wgt / total
            keep += 1
            if cum >= top_p:
                break
        weighted = weighted[: max(keep, 1)]
    ftotal = sum(wgt for _, wgt in weighted)
    target = min(max(draw, 0.0), 1.0 - 2.0 ** -52) * ftotal
    chosen = weighted[0][0]
    for i, wgt in weighted:
        chosen = i
        if target < wgt:
            break
        target -= wgt
    return chosen


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int],
                    max_new_tokens: int) -> List[int]:
    """Greedy continuation by recomputing the whole sequence each token."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(max_new_tokens):
        nxt = argmax_lowest(forward_logits(cfg, w, ids)[-1])
        out.append(nxt)
        ids.append(nxt)
    return out
