"""Grouped-query attention over the paged cache
(crates/infer-worker/src/components/attention.rs:21-37,83-179): fused q,k,v projection,
rotary encoding of q and k, write of k and v into the request's pages, attention of every
new token over the keys it may see, output projection.  The residual add and the norm
before it belong to the block, not to this part.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..ops import kernels as K
from ..ops import library as L
from .base import (BuildContext, Mixer, PagedKV, PagedLayerCache, ParamDecl, POSITIONS, StepContext,
                   register_mixer, single_token_entries, token_tiles)
from .linear import Linear
from .spec import PartSpec


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window (None: all keys),
    position (PartSpec of a rotary encoding, or None), own_kv (False: the layer projects no
    keys or values and reads the cache another layer wrote)."""

    graph_safe = True
    adds_to_residual = True
    MAX_SPLITS = 16

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden_size"])
        self.Hq, self.Hkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.own_kv = bool(p.get("own_kv", True))
        if self.Hq % self.Hkv:
            raise ValueError(f"{self.Hq} heads are not a multiple of {self.Hkv} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 512:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take multiples of 16 up to 512")
        pos = p.get("position")
        self.position_spec: Optional[PartSpec] = pos
        self.position = None
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        q, kv = self.Hq * self.hd, self.Hkv * self.hd
        d = {"q_proj.weight": ParamDecl((q, self.hidden)),
             "o_proj.weight": ParamDecl((self.hidden, q))}
        if self.own_kv:
            d["k_proj.weight"] = ParamDecl((kv, self.hidden))
            d["v_proj.weight"] = ParamDecl((kv, self.hidden))
        return d

    def cache_need(self):
        return PagedKV(self.Hkv, self.hd, self.window)

    def prepare(self, ctx: BuildContext) -> None:
        super().prepare(ctx)
        # bf16 runs on the tensor-core kernels (head sizes up to 256); fp32, and larger heads,
        # on the plain fp32-arithmetic kernel
        self.use_mma = ctx.dtype == torch.bfloat16 and self.hd <= L.MMA_MAX_HEAD_DIM
        # steps of 512 tokens or more: rotary encoding and cache write inside the q,k,v product
        self.fuse_rope = (ctx.dtype == torch.bfloat16 and self.hd in (64, 128)
                          and os.environ.get("RUSTINFER_B200_FUSE_ROPE", "1") != "0")
        # prompt portions: the tcgen05 kernel where it takes the geometry, else the mma.sync one
        self.use_tc = (self.use_mma and os.environ.get("RUSTINFER_B200_PREFILL_ATTENTION", "tc") != "mma"
                       and K.tc_attention_supports(self.Hq, self.Hkv, self.hd, ctx.page_size))
        if self.use_mma:
            self.tokens_per_tile = (K.tc_tokens_per_tile(self.Hq, self.Hkv) if self.use_tc
                                    else K.mma_tokens_per_tile(self.Hq, self.Hkv))
            # entries of one token go to the split-KV kernel, the others are cut into tiles
            self._single = single_token_entries()
            self._tiles = token_tiles(self.tokens_per_tile, skip_single_token=True)
            key = ("decode_scratch", self.Hq, self.hd)
            if key not in ctx.shared:
                no, nl = K.decode_scratch_floats(ctx.max_batch_seqs, self.Hq, self.hd, self.MAX_SPLITS)
                ctx.shared[key] = (torch.empty(no, dtype=torch.float32, device=ctx.device),
                                   torch.empty(nl, dtype=torch.float32, device=ctx.device))
            self.part_o, self.part_lse = ctx.shared[key]
            lib = L.attention_mma(self.hd)
            # the kernel that fetches keys and values by TMA where it is built for this geometry
            self.decode_ctas_per_sm = (int(lib.ri_attention_decode_tma_ctas_per_sm(ctx.page_size))
                                       or int(lib.ri_attention_decode_ctas_per_sm()))
            self.decode_tile_keys = int(lib.ri_attention_decode_tile_keys())
        else:
            self._single = None
            self._tiles = token_tiles(16, skip_single_token=False)
        if self.position_spec is not None:
            key = ("position", self.position_spec.key(), ctx.max_model_len)
            if key not in ctx.shared:
                part = POSITIONS.build(self.position_spec)
                part.prepare(ctx)
                ctx.shared[key] = part
            self.position = ctx.shared[key]

    def step_indices(self):
        return [self._tiles] if self._single is None else [self._single, self._tiles]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # q, k, v fused by rows into one matrix, gate rows first
        # (crates/infer-worker/src/models/loader.rs:419-454)
        parts = [tensors["q_proj.weight"]]
        if self.own_kv:
            parts += [tensors["k_proj.weight"], tensors["v_proj.weight"]]
        dt = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
        self.qkv = Linear(torch.cat([t.to(dt) for t in parts], dim=0), self.ctx.num_sms)
        self.o = Linear(tensors["o_proj.weight"], self.ctx.num_sms)

    def _project_out(self, out: torch.Tensor, residual: Optional[torch.Tensor]):
        if residual is not None and self.o.add_into(out, residual):
            return None
        return self.o(out, out_dtype=self.ctx.dtype)

    def forward(self, x: torch.Tensor, step: StepContext, cache: PagedLayerCache,
                residual: Optional[torch.Tensor] = None):
        """Returns the sublayer's output, or None when it was added into `residual`."""
        g = step.groups[cache.group]
        writes = self.own_kv and cache.writes
        # many tokens: the product rotates q and k and writes keys and values into their pages in
        # its own epilogue (no pass over q, k, v in between)
        if (self.fuse_rope and self.position is not None and self.position.rotary_dim == self.hd
                and x.shape[0] >= 512 and (writes or not self.own_kv) and self.qkv.tensor_core):
            q = torch.empty((x.shape[0], self.Hq * self.hd), dtype=torch.bfloat16, device=x.device)
            if K.gemm_tc_rope(x, self.qkv.weight, q, step.positions, self.position.cos, self.position.sin,
                              g.slot_of_token if writes else None, cache.kv if writes else None,
                              self.Hq, self.Hkv if writes else 0, self.hd):
                return self._project_out(self.attend(q, step, cache), residual)
        qkv = self.qkv(x, out_dtype=self.ctx.dtype)
        if self.position is not None:
            # a layer that reads another's cache has only the q projection: qkv is q alone
            K.rope_scatter(qkv, step.positions, self.position.cos,
                           self.position.sin, g.slot_of_token if writes else None,
                           cache.kv if writes else None, self.Hq, self.Hkv if writes else 0, self.hd,
                           self.position.rotary_dim)
        elif writes:
            # no position encoding inside the mixer: keys and values go into their pages as they are
            K.rope_scatter(qkv, step.positions, None, None, g.slot_of_token, cache.kv, self.Hq, self.Hkv,
                           self.hd, 0)
        return self._project_out(self.attend(qkv[:, : self.Hq * self.hd], step, cache), residual)

    def unmerged_ranges(self, step: StepContext) -> int:
        """Key ranges a step of single tokens only is cut into when its caller merges them itself
        (`attend(..., merge=False)`); 0 when there is nothing to merge (another kind of step, one
        range, or the kernel without ranges)."""
        if not self.use_mma or not step.decode_only:
            return 0
        splits = self._splits(step.num_tokens, step.max_kv_len)
        return splits if splits > 1 else 0

    def attend(self, q: torch.Tensor, step: StepContext, cache: PagedLayerCache,
               out: Optional[torch.Tensor] = None, merge: bool = True) -> torch.Tensor:
        """Attention of the rotated queries q [T, Hq*hd] (unit column stride) over the cache, whose
        pages already hold this step's keys and values: [T, Hq*hd] (into `out` if given).  With
        `merge` False in a step for which `unmerged_ranges` is not 0, the key ranges' partial
        results stay in `self.part_o` / `self.part_lse` and `out` is not written."""
        T = step.num_tokens
        g = step.groups[cache.group]
        if out is None:
            out = torch.empty((T, self.Hq * self.hd), dtype=self.ctx.dtype, device=q.device)
        if not self.use_mma:
            tile_entry, tile_q0 = step.index(self._tiles)
            K.attention_plain(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_q0,
                              self.Hq, self.Hkv, self.hd, self.scale, self.window)
            return out
        (single,) = step.index(self._single)
        if single.numel():
            splits = self._splits(single.numel(), step.max_kv_len)
            K.attention_decode_bf16(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len,
                                    single, single.numel(), self.Hq, self.Hkv, self.hd,
                                    self.scale, self.window, splits, self.part_o, self.part_lse,
                                    merge=merge or not step.decode_only)
        tile_entry, tile_tok0 = step.index(self._tiles)
        if tile_entry.numel():
            prefill = K.attention_prefill_tc if self.use_tc else K.attention_prefill_bf16
            prefill(q, out, cache.kv, g.block_table, step.cu_q, step.kv_len, tile_entry, tile_tok0,
                    self.Hq, self.Hkv, self.hd, self.scale, self.window)
        return out

    def _splits(self, n_decode: int, max_kv_len: int) -> int:
        """Ranges each decoding request's keys are cut into.  A few CTAs sit on an SM (the
        kernel says how many).  A grid that fits one wave is best filled as far as it goes; a
        grid of several waves pays for every wave's start and end, so it is scored by how
        full its last wave is, at a discount.  Measured on B200 at 4,096 keys with 5 CTAs per
        SM: batch 8, 11 ranges (704 CTAs, one wave) 20.6 us, 13 ranges (a second wave) 26.1 us;
        batch 64, 4 ranges 107 us, 1 range 138 us.  Never more ranges than tiles of keys."""
        chunks = (self.Hq // self.Hkv + 15) // 16
        ctas = n_decode * self.Hkv * chunks
        span = min(max_kv_len, self.window) if self.window else max_kv_len
        tiles = max(1, -(-span // self.decode_tile_keys))
        slots = self.decode_ctas_per_sm * self.ctx.num_sms
        best, best_score = 1, -1.0
        for s in range(1, min(tiles, self.MAX_SPLITS) + 1):
            waves = ctas * s / slots
            score = waves if waves <= 1.0 else 0.85 * waves / float(-(-ctas * s // slots))
            if score > best_score + 0.02:
                best, best_score = s, score
        return best
