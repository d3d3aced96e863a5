"""Per-request sampling options, with RustInfer's names and meanings
(crates/infer-core/src/ports/sampler.rs:18-47; `max_tokens`, `ignore_eos`:
crates/infer-protocol/src/scheduler_to_worker_data.rs:56-62)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0            # 0 => greedy
    top_k: int = 0                      # 0 or -1 => off; 1 => greedy
    top_p: float = 1.0                  # (0, 1]; <= 0 => greedy
    min_p: float = 0.0
    repetition_penalty: float = 1.0     # anything but 1 is refused, as in the reference
    seed: Optional[int] = None
    max_tokens: int = 16
    ignore_eos: bool = False

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1 or self.top_p <= 0.0

    def validate(self) -> None:
        # crates/infer-worker/src/application/sampler_stack.rs:221-240
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("sampling temperature must be finite and non-negative")
        if not math.isfinite(self.top_p) or not 0.0 <= self.top_p <= 1.0:
            raise ValueError("sampling top_p must be in [0, 1]")
        if not math.isfinite(self.min_p) or not 0.0 <= self.min_p <= 1.0:
            raise ValueError("sampling min_p must be in [0, 1]")
        if self.repetition_penalty != 1.0:
            raise ValueError("repetition-penalty sampling is not supported (it needs token history)")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.top_k < -1:
            raise ValueError("top_k must be -1, 0 (both: off) or positive")
