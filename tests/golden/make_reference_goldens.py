"""Makes `reference_kernels.safetensors`: small seeded inputs and what Vinci-hit/RustInfer's own
CUDA kernels (compiled unmodified, see baseline/reference_kernels.py) computed from them on a B200.

    python baseline/reference_kernels.py            # where the reference tree and nvcc are
    python tests/golden/make_reference_goldens.py OUT.safetensors      # on a machine with the GPU

`tests/test_reference_goldens.py` holds the plain implementation to these outputs on the CPU, so
the plain implementation rests on executed reference code for rotary tables (llama3 scaling
included), the rotation, RMSNorm (alone and fused with the residual add), SwiGLU, and paged
grouped-query attention for decoding and for prompt portions.  The reference's model code itself
is Rust and could not be run; its kernels could.
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

import reference_kernels as R  # noqa: E402

DEV = "cuda:0"
BF = torch.bfloat16


def paged_case(g, Hq, Hkv, hd, block, kv_lens, q_lens):
    """K/V pools [blocks, block, Hkv, hd] with requests' blocks in shuffled order, NaN where no key lies."""
    n_blocks = sum((n + block - 1) // block for n in kv_lens) + 2
    perm = torch.randperm(n_blocks, generator=g).tolist()
    kp = torch.full((n_blocks, block, Hkv, hd), float("nan"), dtype=BF)
    vp = torch.full((n_blocks, block, Hkv, hd), float("nan"), dtype=BF)
    table = torch.zeros(len(kv_lens), max((n + block - 1) // block for n in kv_lens), dtype=torch.int32)
    ks, vs, at = [], [], 0
    for b, n in enumerate(kv_lens):
        k, v = torch.randn(n, Hkv, hd, generator=g).to(BF), torch.randn(n, Hkv, hd, generator=g).to(BF)
        ks.append(k); vs.append(v)
        for j in range((n + block - 1) // block):
            pg = perm[at]; at += 1
            table[b, j] = pg
            lo, hi = j * block, min((j + 1) * block, n)
            kp[pg, : hi - lo], vp[pg, : hi - lo] = k[lo:hi], v[lo:hi]
    q = torch.randn(sum(q_lens), Hq * hd, generator=g).to(BF)
    return kp, vp, table, ks, vs, q


def main(out_path):
    assert R.load() is not None, "build baseline/_ref/libref_kernels.so first"
    g = torch.Generator().manual_seed(20240611)
    out = {}
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    # rotary tables: no scaling, and llama3 scaling where all three bands are hit
    for tag, (hd, theta, factor, low, high, orig) in {"rope_plain": (64, 10000.0, 1.0, 1.0, 1.0, 64.0),
                                                       "rope_llama3_a": (32, 500000.0, 8.0, 1.0, 4.0, 64.0),
                                                       "rope_llama3_b": (128, 500000.0, 32.0, 1.0, 4.0, 8192.0)}.items():
        sin, cos = R.rope_tables(hd, 300, theta, factor, low, high, orig)
        out[tag + ".sin"], out[tag + ".cos"] = sin.cpu(), cos.cpu()
        out[tag + ".params"] = torch.tensor([hd, theta, factor, low, high, orig], dtype=torch.float64)

    # rotation of q and k
    T, Hq, Hkv, hd = 9, 6, 2, 64
    q, k = torch.randn(T, Hq * hd, generator=g).to(BF), torch.randn(T, Hkv * hd, generator=g).to(BF)
    pos = torch.randint(0, 300, (T,), generator=g, dtype=torch.int32)
    sin, cos = R.rope_tables(hd, 300, 10000.0, 1.0, 1.0, 1.0, 64.0)
    qd, kd = q.to(DEV).clone(), k.to(DEV).clone()
    R.rope(qd, kd, pos.to(DEV), sin, cos, hd)
    out.update({"rotate.q": q, "rotate.k": k, "rotate.positions": pos, "rotate.q_out": qd.cpu(), "rotate.k_out": kd.cpu()})

    # norms
    for dim in (80, 2048):
        x = (torch.randn(7, dim, generator=g) * 3).to(BF)
        w = (1 + 0.3 * torch.randn(dim, generator=g)).to(BF)
        d = torch.randn(7, dim, generator=g).to(BF)
        out[f"rmsnorm{dim}.x"], out[f"rmsnorm{dim}.w"], out[f"rmsnorm{dim}.delta"] = x, w, d
        out[f"rmsnorm{dim}.out"] = R.rmsnorm(x.to(DEV), w.to(DEV), 1e-5).cpu()
        res = x.to(DEV).clone()
        out[f"rmsnorm{dim}.fused_out"] = R.fused_add_rmsnorm(res, d.to(DEV), w.to(DEV), 1e-5).cpu()
        out[f"rmsnorm{dim}.fused_residual"] = res.cpu()

    # SwiGLU over [gate | up]
    gu = (torch.randn(5, 2 * 104, generator=g) * 3).to(BF)
    out["swiglu.gate_up"], out["swiglu.out"] = gu, R.swiglu_packed(gu.to(DEV)).cpu()

    # paged attention: single query tokens, then prompt portions that end their sequences
    for tag, (Hq, Hkv, hd) in {"attn_g4_hd64": (8, 2, 64), "attn_g3_hd128": (3, 1, 128)}.items():
        block, scale = 16, 1.0 / hd ** 0.5
        kv_lens = [1, 17, 64, 65, 130, 200]
        kp, vp, table, ks, vs, _ = paged_case(g, Hq, Hkv, hd, block, kv_lens, [1] * 6)
        for b in range(6):
            out[f"{tag}.k{b}"], out[f"{tag}.v{b}"] = ks[b], vs[b]
        for kind, q_lens in (("decode", [1] * 6), ("prefill", [1, 17, 1, 2, 41, 129])):
            q = torch.randn(sum(q_lens), Hq * hd, generator=g).to(BF)
            o = torch.full_like(q, float("nan")).to(DEV)
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
            if kind == "decode":
                R.paged_decode(q.to(DEV), kp.to(DEV), vp.to(DEV), o, table.to(DEV), i32(kv_lens),
                               R.decode_workspace(6, Hq, hd), Hq, Hkv, hd, scale, sms, kv_lens)
            else:
                cu = [0]
                for n in q_lens:
                    cu.append(cu[-1] + n)
                R.paged_prefill(q.to(DEV), kp.to(DEV), vp.to(DEV), o, table.to(DEV), i32(kv_lens), i32(cu),
                                R.prefill_tiles(q_lens), q_lens, kv_lens, Hq, Hkv, hd, scale)
            torch.cuda.synchronize()
            p = f"{tag}.{kind}."
            out[p + "q"], out[p + "out"] = q, o.cpu()
            out[p + "lens"] = torch.tensor([kv_lens, q_lens], dtype=torch.int32)
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in out.items()}, out_path)
    print(f"wrote {out_path}: {len(out)} tensors, {os.path.getsize(out_path)} bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                            "reference_kernels.safetensors"))
