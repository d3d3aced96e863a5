"""Choosing next tokens from logits on the device.

All rows greedy: one argmax kernel, only the ids cross to the host
(crates/infer-worker/src/application/runtime/mod.rs:713-758).  Otherwise one kernel sorts
and filters each row in the order of RustInfer's host sampler
(crates/infer-worker/src/application/sampler_stack.rs:242-351).  The uniform draw of a
row is a function of (the request's seed, the position of the token being chosen) alone,
so a request's tokens do not depend on which rows share its batch; the reference mixes
the row index into the seed (:77-85), which makes them depend on it.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from ..ops import kernels as K
from .params import SamplingParams

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_draw(seed: int, position: int) -> float:
    """A double in [0, 1) from (seed, position): 53 bits of splitmix64."""
    mixed = (seed ^ ((position * 0x9E3779B97F4A7C15) & _MASK)) & _MASK
    return (_splitmix64(mixed) >> 11) * (1.0 / (1 << 53))


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class Sampler:
    def __init__(self, device: torch.device, vocab_size: int, max_rows: int):
        self.device = device
        self.vocab = vocab_size
        self.max_rows = max_rows
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._argmax_state = K.argmax_state(device, max_rows)
        self._scratch: Optional[torch.Tensor] = None
        # per-row options and draws of a step travel in one pinned buffer and one copy:
        # [draw f64 | temperature f32 | top_p f32 | min_p f32 | top_k i32], max_rows each
        self._stage: List[torch.Tensor] = []
        self._stage_events: List[Optional[torch.cuda.Event]] = []
        self._stage_dev: Optional[torch.Tensor] = None
        self._turn = 0

    def argmax_device(self, logits: torch.Tensor) -> torch.Tensor:
        out = self._out[: logits.shape[0]]
        K.argmax(logits, out, self._argmax_state)
        return out

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               positions: Sequence[int]) -> List[int]:
        """logits fp32 [R, vocab]; row i is drawn with params[i], seeds[i] at positions[i]."""
        return self.sample_device(logits, params, seeds, positions).tolist()

    def _views(self, buf: torch.Tensor):
        n = self.max_rows
        draw = buf[: 8 * n].view(torch.float64)
        f = buf[8 * n: 20 * n].view(torch.float32)
        return draw, f[:n], f[n: 2 * n], f[2 * n: 3 * n], buf[20 * n: 24 * n].view(torch.int32)

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                      positions: Sequence[int]) -> torch.Tensor:
        """As `sample`, but the chosen ids stay on the device (int32 [R], valid until the
        next call); nothing here waits for the device."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"{R} rows exceed the sampler's {self.max_rows}")
        if all(p.is_greedy() for p in params):
            return self.argmax_device(logits)
        if self._scratch is None:
            self._scratch = torch.empty(K.sample_scratch_elems(self.max_rows, self.vocab),
                                        dtype=torch.int64, device=self.device)
            self._stage = [torch.empty(24 * self.max_rows, dtype=torch.uint8).pin_memory() for _ in range(4)]
            self._stage_events = [None] * 4
            self._stage_dev = torch.empty(24 * self.max_rows, dtype=torch.uint8, device=self.device)
        i = self._turn
        self._turn = (i + 1) % len(self._stage)
        if self._stage_events[i] is not None:
            self._stage_events[i].synchronize()               # its last copy has left the host buffer
        draw, temp, top_p, min_p, top_k = (v.numpy() for v in self._views(self._stage[i]))
        for r, (p, seed, pos) in enumerate(zip(params, seeds, positions)):
            draw[r] = uniform_draw(seed, pos)
            temp[r] = p.temperature if not p.is_greedy() else 0.0
            top_p[r], min_p[r], top_k[r] = p.top_p, p.min_p, max(p.top_k, 0)
        self._stage_dev.copy_(self._stage[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_events[i] = ev
        d_draw, d_temp, d_top_p, d_min_p, d_top_k = self._views(self._stage_dev)
        out = self._out[:R]
        K.sample(logits, self._scratch, d_temp[:R], d_top_k[:R], d_top_p[:R], d_min_p[:R], d_draw[:R], out)
        return out
