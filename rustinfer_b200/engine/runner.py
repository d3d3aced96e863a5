"""The step function: one batch of (request, its next tokens) through the model.

A step takes entries that may be whole prompts, portions of prompts cut anywhere, and
single decoded tokens, side by side.  It runs exactly the tokens it is given, as one
ragged batch, over what earlier steps left in the cache, and returns fp32 logits at the
wanted places.  Generation, the scheduler and trace replay all go through this one
function.

RustInfer's counterpart is `Runtime::step` over a `StepRequest`
(crates/infer-worker/src/application/runtime/mod.rs:561-593) with the plan built by
`build_plan` (crates/infer-worker/src/application/runtime/plan.rs:24-154); it returns
sampled tokens, where this returns logits and leaves sampling to the caller.  The checks
before launch are the ones the reference's plan builder makes (:42-105): nothing is
launched with an index the kernels could not follow.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheLayout, CacheManager
from ..cache.pages import OutOfPages
from ..config.registry import load_model_description
from ..models.decoder import Decoder
from ..parts.base import (BuildContext, FixedState, GroupStep, HostEntry, PagedKV, PagedLayerCache,
                          StateLayerCache, StepContext, StepShape)
from ..weights.loader import load_weights

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                 "float32": torch.float32, "fp32": torch.float32}
_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class StepError(ValueError):
    """The batch handed to `step` cannot be run as given."""


@dataclass
class StepEntry:
    request_id: Any
    tokens: Sequence[int]
    want: Sequence[int] = ()            # places among `tokens` whose logits are returned


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _TORCH_DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r}: choose bfloat16 or float32")


class _Staging:
    """A ring of pinned host buffers and the device buffer each step's index arrays are
    copied into with one transfer."""

    def __init__(self, n_ints: int, device: torch.device, depth: int = 3):
        self.host = [torch.empty(n_ints, dtype=torch.int32).pin_memory() for _ in range(depth)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.dev = torch.empty(n_ints, dtype=torch.int32, device=device)
        self.turn = 0

    def next_host(self) -> Tuple[int, torch.Tensor]:
        i = self.turn
        self.turn = (self.turn + 1) % len(self.host)
        if self.events[i] is not None:
            self.events[i].synchronize()
        return i, self.host[i]

    def upload(self, i: int, n: int) -> None:
        self.dev[:n].copy_(self.host[i][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class _DecodeGraph:
    """A captured step of `bucket` single tokens.  Its index arrays live in one device
    buffer at fixed addresses; rows beyond the live entries are padding that reads one key
    of page 0 and writes nothing (RustInfer pads with one-token rows on a scratch block,
    crates/infer-worker/src/application/worker_scheduler.rs:685-718)."""

    def __init__(self, runner: "ModelRunner", bucket: int):
        self.bucket = bucket
        P = runner.max_pages_per_request
        groups = runner.layout.paged_groups()
        self.spare_slot = runner.max_batch_seqs               # the state row padding rows point at
        # what the parts' index arrays look like for `bucket` rows of one token each
        shape = self._shape(np.zeros(bucket, dtype=np.int64), np.full(bucket, self.spare_slot, dtype=np.int64))
        built = [(need, need.build(shape)) for need in runner.index_needs]
        # fixed layout: token_ids, positions, cu_q, kv_len, slots, rows, [table, slot_of_token]*, index arrays
        sizes = [bucket, bucket, bucket + 1, bucket, bucket, bucket]
        for _ in groups:
            sizes += [bucket * P, bucket]
        for _need, arrays in built:
            sizes += [int(a.size) for a in arrays]
        self.offsets = []
        at = 0
        for n in sizes:
            self.offsets.append((at, n))
            at += (n + 3) & ~3
        self.host = torch.zeros(at, dtype=torch.int32).pin_memory()
        self.hv = self.host.numpy()
        self.dev = torch.zeros(at, dtype=torch.int32, device=runner.device)
        self.event: Optional[torch.cuda.Event] = None
        self.row_owner: List[Any] = [None] * bucket          # uid of the request whose table sits in a row
        self.row_pages: List[List[int]] = [[0] * len(groups) for _ in range(bucket)]
        v = [self.dev[o: o + n] for o, n in self.offsets]
        hv = [self.hv[o: o + n] for o, n in self.offsets]
        self.h_tokens, self.h_pos, h_cu, self.h_kv, self.h_slots, h_rows = hv[:6]
        h_cu[:] = np.arange(bucket + 1)
        h_rows[:] = np.arange(bucket)
        self.h_pos[:] = 0
        self.h_kv[:] = 1
        self.h_slots[:] = self.spare_slot
        it, hit = iter(v[6:]), iter(hv[6:])
        gsteps, self.h_tables, self.h_slot_of_token = [], [], []
        for _ in groups:
            gsteps.append(GroupStep(next(it).view(bucket, P), next(it)))
            self.h_tables.append(next(hit).reshape(bucket, P))
            h = next(hit)
            h[:] = -1
            self.h_slot_of_token.append(h)
        indices = {}
        self.moving_indices = []                             # (need, host views): made anew at every replay
        for need, arrays in built:
            devs, hosts = [], []
            for a in arrays:
                devs.append(next(it))
                h = next(hit)
                h[:] = a
                hosts.append(h)
            indices[need.key] = tuple(devs)
            if need.depends_on_positions:
                self.moving_indices.append((need, hosts))
        self.dev.copy_(self.host)
        self.step = StepContext(
            num_tokens=bucket, num_entries=bucket, token_ids=v[0], positions=v[1], cu_q=v[2], kv_len=v[3],
            state_slots=v[4], groups=gsteps, entries=[], max_q_len=1,
            max_kv_len=runner.max_model_len, decode_only=True, indices=indices)
        self.rows = v[5]
        # one eager run (libraries pick their algorithms, lazy kernels get built), then capture
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runner.model.forward(self.step, runner.entry_caches, self.rows)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import library as _lib
        before = _lib.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=runner._graph_pool):
            self.logits = runner.model.forward(self.step, runner.entry_caches, self.rows)
        self.kernels_per_replay = _lib.launch_count - before
        if runner._graph_pool is None:
            runner._graph_pool = self.graph.pool()

    def _shape(self, pos0: np.ndarray, slots: np.ndarray) -> StepShape:
        ones = np.ones(self.bucket, dtype=np.int64)
        return StepShape(ones, pos0, np.arange(self.bucket + 1, dtype=np.int64), pos0 + 1, slots)

    def forget_rows(self) -> None:
        """Every row's block table is written afresh at its next use."""
        self.row_owner = [-1] * self.bucket

    def fill(self, runner: "ModelRunner", entries: Sequence[StepEntry], host_tokens: bool) -> None:
        """Write this step's indices into the pinned buffer and send it.  A row keeps the
        block table of the request it held last step; only pages added since are written."""
        if self.event is not None:
            self.event.synchronize()                         # the last upload has left the host buffer
        ps = runner.page_size
        cache = runner.cache
        groups = runner.layout.paged_groups()
        for i, e in enumerate(entries):
            rid = e.request_id
            pos = cache.length(rid)
            if host_tokens:
                self.h_tokens[i] = e.tokens[0]
            self.h_pos[i] = pos
            self.h_kv[i] = pos + 1
            self.h_slots[i] = cache.slot(rid)
            uid = cache.uid(rid)
            if self.row_owner[i] != uid:
                self.row_owner[i] = uid
                self.row_pages[i] = [0] * len(groups)
            for gi, g in enumerate(groups):
                table = cache.block_table(rid, g)
                start, n = self.row_pages[i][gi], len(table)
                if start < n:
                    row = self.h_tables[gi][i]
                    row[start:n] = table[start:n]
                    np.maximum(row[start:n], 0, out=row[start:n])
                    self.row_pages[i][gi] = n
                page = table[pos // ps]
                if page < 0:
                    raise StepError("a token would be written to a page that was given back")
                self.h_slot_of_token[gi][i] = page * ps + pos % ps
        for i in range(len(entries), self.bucket):           # padding rows
            if self.row_owner[i] is not None:
                self.row_owner[i] = None
                self.h_pos[i] = 0
                self.h_kv[i] = 1
                self.h_tokens[i] = 0
                self.h_slots[i] = self.spare_slot            # no live request's state is touched
                for h in self.h_slot_of_token:
                    h[i] = -1
        if self.moving_indices:
            shape = self._shape(self.h_pos.astype(np.int64), self.h_slots.astype(np.int64))
            for need, hosts in self.moving_indices:
                arrays = need.build(shape)
                if [int(a.size) for a in arrays] != [h.size for h in hosts]:
                    raise StepError(f"index arrays {need.key!r} change their lengths between steps of "
                                    f"{self.bucket} single tokens; such a part cannot run from a captured step")
                for h, a in zip(hosts, arrays):
                    h[:] = a
        self.dev.copy_(self.host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.event = ev


class ModelRunner:
    """Model, cache and step function of one model folder on one GPU."""

    def __init__(self, model_dir: str, dtype="bfloat16", device="cuda:0", max_model_len: int = 4096,
                 page_size: int = 16, num_pages: Optional[int] = None, max_batch_seqs: int = 64,
                 max_batch_tokens: int = 8192, mem_fraction_static: float = 0.9,
                 capture_sizes: Optional[Sequence[int]] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("rustinfer_b200 runs on a CUDA device (sm_100a) only; there is no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        # the 32-bit path is true fp32 everywhere: no TF32 in any library product either
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.family, self.config, self.spec = load_model_description(model_dir)
        self.max_model_len = int(max_model_len)
        self.page_size = int(page_size)
        self.max_batch_seqs = int(max_batch_seqs)
        self.max_batch_tokens = int(max_batch_tokens)
        self.model = Decoder(self.spec)
        self.ctx = BuildContext(self.device, self.dtype, self.max_model_len, self.page_size,
                                max_batch_seqs=self.max_batch_seqs,
                                num_sms=torch.cuda.get_device_properties(self.device).multi_processor_count)
        self.model.prepare(self.ctx)
        self.model.load(load_weights(model_dir, self.model.param_decls(), self.dtype, self.device))

        self.layout = CacheLayout.from_needs(self.model.cache_needs())
        self.max_pages_per_request = (self.max_model_len + self.page_size - 1) // self.page_size
        paged = self.layout.paged_groups()
        if num_pages is None:
            num_pages = self._auto_pages(mem_fraction_static)
        self.num_pages = int(num_pages)
        # graph buckets: the sizes asked for that fit, and the largest batch itself when a larger
        # size was asked for (else steps between the last fitting size and the limit would run eagerly)
        sizes = set(int(c) for c in (capture_sizes or ()))
        if any(c > self.max_batch_seqs for c in sizes):
            sizes.add(self.max_batch_seqs)
        self.capture_sizes = sorted(c for c in sizes if 1 <= c <= self.max_batch_seqs)
        self.cache = CacheManager(self.layout, [self.num_pages] * len(paged), self.page_size,
                                  self.max_batch_seqs)
        self._alloc_storage()
        self.index_needs = self.model.step_indices()          # arrays the parts want made for every step
        cap_t, cap_b = self.max_batch_tokens, self.max_batch_seqs
        n_ints = 5 * cap_t + 5 * cap_b + 64
        n_ints += len(paged) * (cap_b * self.max_pages_per_request + cap_t + 16)
        for need in self.index_needs:
            n_ints += int(need.capacity(cap_t, cap_b)) + 32
        self._staging = _Staging(n_ints, self.device)
        # per-request counters the device keeps by state slot: {generated, max_tokens, ignore_eos, last_token}
        self.slot_state = torch.zeros((self.max_batch_seqs, 4), dtype=torch.int32, device=self.device)
        eos = [t for t in self.spec.eos_token_ids if 0 <= t < self.spec.vocab_size]
        self.eos_dev = torch.tensor(eos, dtype=torch.int32, device=self.device) if eos else None
        self.last_want_slots: Optional[torch.Tensor] = None   # state slot of every wanted row of the last step
        self.steps_run = 0
        self.h2d_bytes_last = 0
        self.graph_replays = 0
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        self._graph_pool = None
        self.use_graphs = bool(self.capture_sizes) and self.model.graph_safe

    # ------------------------------------------------------------------------ storage
    def _auto_pages(self, fraction: float) -> int:
        """Pages per group from the memory that is free once the weights are loaded:
        (free - 1 GiB) * fraction / bytes per page over all groups, at most what
        max_batch_seqs requests of max_model_len tokens can use
        (crates/infer-worker/src/application/serve_loop.rs:425-449)."""
        esize = torch.empty((), dtype=self.dtype).element_size()
        per_page = 0
        for g in self.layout.groups:
            if isinstance(g.need, PagedKV):
                per_page += len(g.entries) * 2 * g.need.num_kv_heads * self.page_size * g.need.head_dim * esize
        cap = self.max_batch_seqs * self.max_pages_per_request
        if per_page == 0:
            return 1
        free, _total = torch.cuda.mem_get_info(self.device)
        by_memory = int(max(0, free - (1 << 30)) * fraction) // per_page
        if by_memory < self.max_pages_per_request:
            raise RuntimeError(f"free GPU memory holds {by_memory} cache pages; one request of "
                               f"max_model_len {self.max_model_len} needs {self.max_pages_per_request}")
        return min(cap, by_memory)

    def _alloc_storage(self) -> None:
        self.group_storage: List[torch.Tensor] = []
        self._paged_index: Dict[int, int] = {}
        for gi, g in enumerate(self.layout.groups):
            n = len(g.entries)
            if isinstance(g.need, PagedKV):
                self._paged_index[gi] = len(self._paged_index)
                t = torch.zeros((n, self.num_pages, 2, g.need.num_kv_heads, self.page_size, g.need.head_dim),
                                dtype=self.dtype, device=self.device)
            elif isinstance(g.need, FixedState):
                # one row more than there are slots: padding rows of a captured step point there
                t = torch.zeros((n, self.max_batch_seqs + 1) + tuple(g.need.shape),
                                dtype=_STATE_DTYPES[g.need.dtype], device=self.device)
            else:
                raise TypeError(f"unknown cache need {g.need!r}")
            self.group_storage.append(t)
        self.entry_caches: List[Any] = []
        for i, loc in enumerate(self.layout.entry_cache):
            if loc is None:
                self.entry_caches.append(None)
                continue
            gi, idx = loc
            if isinstance(self.layout.groups[gi].need, PagedKV):
                self.entry_caches.append(PagedLayerCache(self.group_storage[gi][idx], self._paged_index[gi],
                                                         self.layout.entry_writes[i]))
            else:
                self.entry_caches.append(StateLayerCache(self.group_storage[gi][idx]))

    def cache_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.group_storage)

    # ----------------------------------------------------------------------- requests
    def open(self, request_id: Any) -> None:
        self.cache.open(request_id)

    def set_request_limits(self, request_id: Any, generated: int, max_tokens: int, ignore_eos: bool) -> None:
        """What the device-side stop check knows of a request: tokens generated so far, the
        count at which it stops, whether stop ids are ignored."""
        row = torch.tensor([generated, max_tokens, 1 if ignore_eos else 0, 0], dtype=torch.int32)
        self.slot_state[self.cache.slot(request_id)].copy_(row, non_blocking=True)

    def close(self, request_id: Any) -> None:
        self.cache.close(request_id)

    # --------------------------------------------------------------------------- plan
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_batch_seqs:
            raise StepError(f"{len(entries)} entries exceed max_batch_seqs {self.max_batch_seqs}")
        seen = set()
        total = 0
        vocab = self.spec.vocab_size
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if not self.cache.is_open(e.request_id):
                raise StepError(f"request {e.request_id!r} is not open")
            q = len(e.tokens)
            if q < 1:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            total += q
            if self.cache.length(e.request_id) + q > self.max_model_len:
                raise StepError(f"request {e.request_id!r} would reach {self.cache.length(e.request_id) + q} "
                                f"tokens, max_model_len is {self.max_model_len}")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise StepError(f"request {e.request_id!r}: token id {t} outside [0, {vocab})")
            for w in e.want:
                if not 0 <= int(w) < q:
                    raise StepError(f"request {e.request_id!r}: wanted place {w} outside its {q} tokens")
        if total > self.max_batch_tokens:
            raise StepError(f"{total} tokens exceed max_batch_tokens {self.max_batch_tokens}")

    def _build(self, entries: Sequence[StepEntry]) -> Tuple[StepContext, Optional[torch.Tensor]]:
        ps = self.page_size
        B = len(entries)
        q_lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        pos0 = np.fromiter((self.cache.length(e.request_id) for e in entries), dtype=np.int64, count=B)
        cu_q = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu_q[1:])
        T = int(cu_q[-1])
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        entry_of_token = np.repeat(np.arange(B), q_lens)
        positions = np.arange(T) - cu_q[entry_of_token] + pos0[entry_of_token]
        kv_len = pos0 + q_lens
        slots = np.fromiter((self.cache.slot(e.request_id) for e in entries), dtype=np.int64, count=B)
        rows: List[int] = []
        row_slots: List[int] = []
        for i, e in enumerate(entries):
            rows.extend(int(cu_q[i]) + int(w) for w in e.want)
            row_slots.extend([int(slots[i])] * len(e.want))

        sections: List[np.ndarray] = [token_ids, positions, cu_q, kv_len, slots,
                                      np.asarray(rows, dtype=np.int64)]
        max_blocks = int(((kv_len + ps - 1) // ps).max())
        for gi in self.layout.paged_groups():
            table = np.zeros((B, max_blocks), dtype=np.int64)
            for i, e in enumerate(entries):
                t = self.cache.block_table(e.request_id, gi)
                n = min(len(t), max_blocks)
                table[i, :n] = t[:n]
            page_of_token = table[entry_of_token, positions // ps]
            if (page_of_token < 0).any():
                raise StepError("a token would be written to a page that was given back")
            slot_of_token = page_of_token * ps + positions % ps
            np.maximum(table, 0, out=table)
            sections += [table.reshape(-1), slot_of_token]
        sections.append(np.asarray(row_slots, dtype=np.int64))
        shape = StepShape(q_lens, pos0, cu_q, kv_len, slots)
        built = [(need, need.build(shape)) for need in self.index_needs]
        for _need, arrays in built:
            sections += [np.asarray(a) for a in arrays]

        idx, host = self._staging.next_host()
        offsets: List[Tuple[int, int]] = []
        at = 0
        hv = host.numpy()
        for s in sections:
            n = s.size
            hv[at: at + n] = s
            offsets.append((at, n))
            at += (n + 3) & ~3                      # every section starts on a 16-byte boundary
        self._staging.upload(idx, at)
        self.h2d_bytes_last = at * 4
        dev = self._staging.dev
        views = [dev[o: o + n] for o, n in offsets]
        it = iter(views[6:])
        groups = []
        for _ in self.layout.paged_groups():
            table = next(it).view(B, max_blocks)
            groups.append(GroupStep(table, next(it)))
        self.last_want_slots = next(it)
        indices = {need.key: tuple(next(it) for _ in arrays) for need, arrays in built}
        host_entries = [HostEntry(e.request_id, int(slots[i]), int(q_lens[i]), int(pos0[i]))
                        for i, e in enumerate(entries)]
        step = StepContext(
            num_tokens=T, num_entries=B, token_ids=views[0], positions=views[1], cu_q=views[2],
            kv_len=views[3], state_slots=views[4], groups=groups, entries=host_entries,
            max_q_len=int(q_lens.max()), max_kv_len=int(kv_len.max()), decode_only=bool((q_lens == 1).all()),
            indices=indices)
        return step, (views[5] if rows else None)

    # --------------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             borrow_logits: bool = False) -> Optional[torch.Tensor]:
        """Run one batch.  Returns fp32 logits [wanted, vocab] on the device in the order of
        the entries and of their `want`, or None when nothing is wanted.  Raises `OutOfPages`
        before anything runs if the cache cannot hold the new tokens (nothing is changed).

        `device_tokens` (int32 on the device, one per entry) replaces the entries' token ids
        in a step of single tokens: the ids chosen by the last step need not visit the host
        before they are fed back.  With `borrow_logits` the result may be a view of a buffer
        that the next step overwrites (for callers that consume it at once)."""
        self._validate(entries)
        lease = self.cache.lease([(e.request_id, len(e.tokens)) for e in entries])
        try:
            self._zero_new_state()
            bucket = self._bucket_for(entries)
            if bucket:
                logits = self._graph_step(entries, bucket, device_tokens)
                if logits is not None and not borrow_logits:
                    logits = logits.clone()
            else:
                step, rows = self._build(entries)
                if device_tokens is not None:
                    if not step.decode_only:
                        raise StepError("device_tokens only stands for steps of single tokens")
                    step.token_ids[: step.num_tokens].copy_(device_tokens[: step.num_tokens])
                logits = self.model.forward(step, self.entry_caches, rows)
        except BaseException:
            # the step did not happen: its pages go back, and no captured step may trust a
            # block table it wrote earlier (tables have shrunk under it)
            lease.release()
            for g in self._graphs.values():
                g.forget_rows()
            raise
        lease.commit()
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ decode graphs
    def _bucket_for(self, entries: Sequence[StepEntry]) -> int:
        """Smallest captured batch size that holds a step of single tokens, else 0
        (crates/infer-worker/src/application/runtime/graph_exec.rs:98-134)."""
        if not self.use_graphs or any(len(e.tokens) != 1 for e in entries):
            return 0
        for c in self.capture_sizes:
            if c >= len(entries):
                return c if c <= self.max_batch_seqs else 0
        return 0

    def _graph_step(self, entries: Sequence[StepEntry], bucket: int,
                    device_tokens: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        g = self._graphs.get(bucket)
        if g is None:
            g = _DecodeGraph(self, bucket)
            self._graphs[bucket] = g
        g.fill(self, entries, device_tokens is None)
        if device_tokens is not None:
            g.step.token_ids[: len(entries)].copy_(device_tokens[: len(entries)])
        g.graph.replay()
        self.graph_replays += 1
        self.h2d_bytes_last = g.host.numel() * 4
        from ..ops import library as _lib
        _lib.launch_count += g.kernels_per_replay
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            self.last_want_slots = None
            return None
        if len(wanted) == len(entries):
            self.last_want_slots = g.step.state_slots[: len(entries)]
            return g.logits[: len(entries)]
        idx = torch.tensor(wanted, device=self.device)
        self.last_want_slots = g.step.state_slots[idx]
        return g.logits[idx]

    def check_kernel_errors(self) -> None:
        """Raise if a kernel recorded a fault it survived (a bounded wait that ran out).
        Reads one word from the device, so it synchronises; callers use it where they
        synchronise anyway."""
        from ..ops import kernels as _k
        code = _k.gemm_tc_error(self.device)
        if code:
            what = ("its shared memory did not start on a 1024-byte boundary" if code == 14
                    else "a bounded wait ran out")
            raise RuntimeError(f"a tensor-core kernel gave up (code {code}: {what}); "
                               f"results of the last steps are not valid")

    def _zero_new_state(self) -> None:
        new = self.cache.newly_opened_slots
        if not new:
            return
        for gi, g in enumerate(self.layout.groups):
            if isinstance(g.need, FixedState):
                self.group_storage[gi][:, new] = 0
        new.clear()
