"""Steps of a few tokens through a pre-norm decoder of grouped-query attention, SwiGLU and
RMSNorm with the products between two attentions chained into one kernel:

    chain 0:  norm + q,k,v of entry 0, rotary, cache write
    entry i:  attention over the cache (its own kernels)
    chain i+1: output product of entry i into the stream, norm + gate/up + SiLU, down product
               into the stream, norm + q,k,v of entry i+1, rotary, cache write

which is what `Block` does part by part (crates/infer-worker/src/components/decoder_block.rs:13-32),
with three launches a layer instead of nine.  This is an optimisation over parts that are
already built and loaded: it is made only when every block of the model is of that shape and
the kernel takes its sizes; otherwise, and for larger steps, the parts run one by one.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..parts.attention import GQAAttention
from ..parts.base import PagedLayerCache, StepContext
from ..parts.ffn import SwiGLU
from ..parts.norm import RMSNorm


def _chainable_linear(lin) -> bool:
    return lin is not None and lin.tensor_core and lin.weight.data_ptr() % 16 == 0


class ChainedDecoder:
    """Built by `ChainedDecoder.build(decoder)`; `takes(step)` says whether a step can go this
    way, `forward` has the contract of `Decoder.forward`."""

    PAGE = 2 << 20

    def __init__(self, decoder, max_tokens: int):
        self.d = decoder
        self.ctx = decoder.ctx
        self.max_tokens = max_tokens
        self.fold_merge = os.environ.get("RUSTINFER_B200_FOLD_MERGE", "1") != "0"
        self.entries = [(decoder.blocks[e.layer], i) for i, e in enumerate(decoder.spec.run_order)]
        # Everything small that the chains touch (stream, activations, norm weights) lies in one
        # arena that starts on a 2 MB boundary: while gigabytes of weights stream past, these
        # few lines then share one or two translation entries instead of one each.
        rows = K.CHAIN_MAX_TOKENS
        need = {("h", decoder.spec.hidden_size, torch.float32): None}
        for block in decoder.blocks:
            a, f = block.mixer, block.ffn
            need[("qkv", a.qkv.out_features, torch.float32)] = None
            need[("q", a.Hq * a.hd, torch.bfloat16)] = None
            need[("attn", a.Hq * a.hd, torch.bfloat16)] = None
            need[("mid", f.inter, torch.bfloat16)] = None
            need[("xn", a.hidden, torch.bfloat16)] = None            # wide steps: the normed operand
        need[("rowsq_a", 1, torch.float32)] = None                   # ... and the rows' sums of squares
        need[("rowsq_b", 1, torch.float32)] = None
        norms = [n for block in decoder.blocks for n in (block.mixer_norm, block.ffn_norm)]
        size = sum(-(-n.weight.numel() * n.weight.element_size() // 256) * 256 for n in norms)
        size += sum(-(-rows * cols * torch.empty((), dtype=dt).element_size() // 256) * 256 for _, cols, dt in need)
        raw = torch.zeros(size + self.PAGE, dtype=torch.uint8, device=self.ctx.device)
        at = -raw.data_ptr() % self.PAGE
        self._arena = raw

        def take(nbytes: int) -> torch.Tensor:
            nonlocal at
            t = raw[at: at + nbytes]
            at += -(-nbytes // 256) * 256
            return t

        self.norm_w: Dict[int, torch.Tensor] = {}
        for n in norms:
            w = take(n.weight.numel() * n.weight.element_size()).view(n.weight.dtype)
            w.copy_(n.weight.reshape(-1))
            self.norm_w[id(n)] = w
        self._buffers: Dict[Tuple, torch.Tensor] = {}
        for kind, cols, dt in need:
            el = torch.empty((), dtype=dt).element_size()
            self._buffers[(kind, cols, dt)] = take(rows * cols * el).view(dt).view(rows, cols)
        self.h = self._buffers[("h", decoder.spec.hidden_size, torch.float32)]

    def _buffer(self, kind: str, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """Buffers live as long as the model (captured graphs keep their addresses); layers of
        the same width share them.  The q,k,v accumulator is kept at zero by the kernel."""
        return self._buffers[(kind, cols, dtype)]

    # ------------------------------------------------------------------------- build
    @classmethod
    def build(cls, decoder) -> Optional["ChainedDecoder"]:
        ctx = decoder.ctx
        if (ctx.dtype != torch.bfloat16 or ctx.device.type != "cuda"
                or os.environ.get("RUSTINFER_B200_DECODE_CHAIN", "1") == "0"):
            return None
        for block in decoder.blocks:
            a, f = block.mixer, block.ffn
            if (block.spec.arrangement != "pre_norm" or type(a) is not GQAAttention or type(f) is not SwiGLU
                    or type(block.mixer_norm) is not RMSNorm or type(block.ffn_norm) is not RMSNorm):
                return None
            if (a.position is None or not a.use_mma or not getattr(f, "paired", False)
                    or not all(_chainable_linear(l) for l in (a.qkv, a.o, f.gate_up, f.down))
                    or a.hidden % 8 or (a.Hq * a.hd) % 8 or f.inter % 8
                    or any(n.weight.data_ptr() % 16 for n in (block.mixer_norm, block.ffn_norm))):
                return None
        self = cls(decoder, 0)
        tokens = 0
        for t in (8, 16, 32, K.CHAIN_MAX_TOKENS):          # the widest step every chain of the model takes
            if all(K.decode_chain_fits(products, t, ctx.num_sms) for products, _ in self._chains(t, None, None)):
                tokens = t
        limit = int(os.environ.get("RUSTINFER_B200_DECODE_CHAIN_TOKENS", str(K.CHAIN_MAX_TOKENS)))
        self.max_tokens = min(tokens, limit)
        return self if self.max_tokens > 0 else None

    # ---------------------------------------------------------------------- products
    def _qkv_product(self, block, T):
        a = block.mixer
        width = a.qkv.out_features
        acc = self._buffer("qkv", width, torch.float32)
        return K.ChainProduct(a.qkv.weight, self.h[:T], acc[:T], K.CHAIN_ADD_F32,
                              norm=(self.norm_w[id(block.mixer_norm)], block.mixer_norm.eps),
                              xn=self._buffer("xn", a.hidden, torch.bfloat16),
                              rowsq=self._buffer("rowsq_b", 1, torch.float32).view(-1))

    def _rope(self, block, T, step: Optional[StepContext], cache: Optional[PagedLayerCache]):
        a = block.mixer
        if step is None:
            return None
        writes = a.own_kv and cache.writes
        g = step.groups[cache.group]
        acc = self._buffer("qkv", a.qkv.out_features, torch.float32)
        q = self._buffer("q", a.Hq * a.hd, torch.bfloat16)
        return K.ChainRope(acc[:T], step.positions, a.position.cos, a.position.sin,
                           g.slot_of_token if writes else None, q[:T], cache.kv if writes else None,
                           a.Hq, a.Hkv if a.own_kv else 0, a.hd, a.position.rotary_dim)

    def _chains(self, T: int, step: Optional[StepContext], caches: Optional[List]):
        """[(products, rope)] for a step of T tokens: len(run order) + 1 chains."""
        chains = []
        first = self.entries[0][0]
        chains.append(([self._qkv_product(first, T)], self._rope(first, T, step, caches[0] if caches else None)))
        for i, (block, _) in enumerate(self.entries):
            a, f = block.mixer, block.ffn
            attn = self._buffer("attn", a.Hq * a.hd, torch.bfloat16)
            mid = self._buffer("mid", f.inter, torch.bfloat16)
            rows = K.CHAIN_MAX_TOKENS
            # up to 16 single tokens whose keys were cut into ranges: the output product merges the
            # ranges itself while it lays out its operand, and the attention launches no merge
            # (heads of 64: the 1B shape's step 1.061 -> 1.054 ms.  With heads of 128 the operand's
            # lay-out takes twice as long and the 8B shape's step went from 1.40 to 1.47 ms, so those
            # keep the merge launch.)
            ranges = a.unmerged_ranges(step) if (step is not None and T <= 16 and self.fold_merge and a.hd <= 64) else 0
            partials = (a.part_o, a.part_lse, ranges, a.Hq, a.hd) if ranges else None
            products = [K.ChainProduct(a.o.weight, attn[:T], self.h[:T], K.CHAIN_ADD_F32, x_rows=rows, partials=partials),
                        K.ChainProduct(f.gate_up.weight, self.h[:T], mid[:T], K.CHAIN_SILU_BF16,
                                       norm=(self.norm_w[id(block.ffn_norm)], block.ffn_norm.eps),
                                       xn=self._buffer("xn", a.hidden, torch.bfloat16),
                                       rowsq=self._buffer("rowsq_a", 1, torch.float32).view(-1)),
                        K.ChainProduct(f.down.weight, mid[:T], self.h[:T], K.CHAIN_ADD_F32, x_rows=rows)]
            rope = None
            if i + 1 < len(self.entries):
                nxt = self.entries[i + 1][0]
                products.append(self._qkv_product(nxt, T))
                rope = self._rope(nxt, T, step, caches[i + 1] if caches else None)
            chains.append((products, rope))
        return chains

    # --------------------------------------------------------------------------- run
    def takes(self, step: StepContext) -> bool:
        return 1 <= step.num_tokens <= self.max_tokens

    def forward(self, step: StepContext, caches: List, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        d, T, sms = self.d, step.num_tokens, self.ctx.num_sms
        h = self.h[:T]
        d.embed.forward(step, h)
        chains = self._chains(T, step, caches)
        K.decode_chain(chains[0][0], chains[0][1], T, sms)
        for i, (block, _) in enumerate(self.entries):
            a = block.mixer
            q = self._buffer("q", a.Hq * a.hd, torch.bfloat16)[:T]
            attn = self._buffer("attn", a.Hq * a.hd, torch.bfloat16)
            a.attend(q, step, caches[i], out=attn[:T], merge=chains[i + 1][0][0].partials is None)
            K.decode_chain(chains[i + 1][0], chains[i + 1][1], T, sms)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        n = d.final_norm.add_norm(h, None, rows=logit_rows)
        return d.head.forward(n)
