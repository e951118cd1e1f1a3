"""The step function: a model, its cache, and one call that runs a batch of tokens.

``Engine.step`` takes, for each sequence of the batch, its slot, its next tokens
and the places among them whose logits are wanted.  It appends to the cache and
returns the float32 logits of the wanted places, in the order given.  Sequences
may bring different numbers of tokens; a result does not depend on what else is
in the batch (reference: one sequence per call, src/model.rs:565-589; prefill
and decode are the same code there too).

A step in which every sequence brings one token is launch-bound, so it is
replayed from a CUDA graph: one graph per batch-size bucket, captured the first
time the bucket is met.  The batch is padded to the bucket with rows that belong
to no sequence (``seq_of_token = -1``): they read and write only the scratch page,
get no expert and change no result.  Every other step of up to 512 tokens and 64
sequences (prompts, chunks, continued and fresh sequences mixed, any wanted
places) is replayed the same way from a graph of its padded shape.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

import ctypes
import os

from ..cache.allocator import _IP, PAGE_TOKENS, _ok, host_lib, ints
from ..cache.kv import KVCache
from ..models.decoder import DecoderModel
from ..ops import core
from .batch import StepBatch, fill_host, layout

GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
# Short steps of any other kind (prompts, chunks of prompts, continued sequences, any wanted places)
# are bound by the host's launches (hundreds of kernels a step), so they too are replayed from
# graphs, padded to these numbers of token rows and of sequences.
STEP_TOKEN_BUCKETS = (64, 128, 256, 512)
STEP_SEQ_BUCKETS = (1, 2, 4, 8, 16, 32, 64)
# A step of more tokens than this is run in pieces of at most this many (the reference tiles a prompt
# at 64 tokens, src/main.rs:499-505): what a step needs beside the cache grows with its tokens.
MAX_STEP_TOKENS = int(os.environ.get("MOE_B200_MAX_STEP_TOKENS", "8192"))
MAX_GRAPHS = 48      # captured steps an engine keeps; the one used longest ago goes first
LAST_TOKEN = -1      # as a token id (with ``from_last``): the token sampled last for the sequence


class _StepGraph:
    """Static buffers and the captured graph of one padded shape of step.

    The first use runs the shape once with NO live sequence (every row a padding row: lazy builds,
    kernel attributes and workspaces happen outside the capture, and nothing that belongs to a
    sequence is touched), then captures, then replays: the step itself runs exactly once, so a part
    with state of its own is advanced once.  All graphs of an engine share one memory pool; they
    never run at the same time and keep nothing between replays but their logits."""

    batch: StepBatch
    upd_off: List[int]
    upd_rows: int

    def _buffers(self, engine: "Engine", words: int) -> None:
        self.host = torch.zeros(words, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(words, dtype=torch.int32, device=engine.rt.device)
        self.event = torch.cuda.Event()
        self.busy = False
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.traced: List[Tuple[object, list]] = []
        self.launches = 0

    def _wait_host(self) -> None:
        if self.busy:
            self.event.synchronize()
            self.busy = False

    def _send(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        self.event.record()
        self.busy = True

    def _pack(self, engine: "Engine", *step) -> None:
        raise NotImplementedError

    def fill(self, engine: "Engine", *step) -> None:
        """Pack the step into the pinned buffer (host runtime) and start its copy; capture first if new."""
        if self.graph is None:
            self._capture(engine)
        self._wait_host()
        self._pack(engine, *step)
        self._send()

    def _body(self, engine: "Engine"):
        for gi, o in enumerate(self.upd_off):
            core.table_update(engine.cache.groups[gi].table, self.dev[o:o + 3 * self.upd_rows], self.upd_rows)
        return engine.model.forward(self.batch, engine.cache)

    def _capture(self, engine: "Engine") -> None:
        tracing = [p for p in engine._tracers if getattr(p, "trace", None) is not None]
        kept = [p.trace for p in tracing]
        for p in tracing:
            p.trace = None                      # the run below is nobody's step: it leaves no record
        self._wait_host()
        self._pack_empty(engine)
        self._send()
        try:
            self._body(engine)                  # every row belongs to no sequence
            torch.cuda.synchronize()
        except BaseException:
            for p, t in zip(tracing, kept):
                p.trace = t
            raise
        for p in tracing:
            p.trace = []
        g = torch.cuda.CUDAGraph()
        l0 = core.launches
        try:
            with torch.cuda.graph(g, pool=engine._graph_pool):
                self.logits = self._body(engine)
        finally:
            # what the parts recorded during the capture are buffers that every replay fills again
            self.traced = [(p, p.trace) for p in tracing]
            for p, t in zip(tracing, kept):
                p.trace = t
        self.launches = core.launches - l0
        self.graph = g

    def run(self, engine: "Engine") -> torch.Tensor:
        core.launches += self.launches
        self.graph.replay()
        for p, items in self.traced:
            if p.trace is not None:
                p.trace.extend(item.clone() if isinstance(item, torch.Tensor) else tuple(t.clone() for t in item)
                               for item in items)
        return self.logits


class _DecodeGraph(_StepGraph):
    """One token per sequence, padded to ``size`` sequences."""

    def __init__(self, engine: "Engine", size: int, max_end: int = 0):
        self.size = size
        ngroups = len(engine.cache.groups)
        offs, o = {}, 0
        for name, n in layout(size, size, size):
            offs[name] = (o, n)
            o += n
        self.upd_off = []
        self.upd_rows = size
        for _ in range(ngroups):
            self.upd_off.append(o)
            o += 3 * size
        self._upd_off_c, _ = ints(self.upd_off)
        self._buffers(engine, o)
        views = {k: self.dev[a:a + n] for k, (a, n) in offs.items()}
        # max_end: the longest sequence this graph will see (kernels size their grids by it)
        self.batch = StepBatch(**views, num_tokens=size, num_seqs=size, num_want=size, max_new=1, max_end=max_end,
                               all_decode=True, all_fresh=False, last_token=engine.cache.last_token)

    def _pack(self, engine: "Engine", slots, starts, tokens, updates: np.ndarray) -> None:
        sl, B = ints(slots)
        st, _ = ints(starts)
        tk, _ = ints(tokens)
        upd = np.ascontiguousarray(updates, dtype=np.int32)
        _ok(host_lib().moe_pack_decode(ctypes.cast(self.host.data_ptr(), _IP), self.size, B, sl, st, tk,
                                       engine.cache.padding_slot, len(self.upd_off), self._upd_off_c,
                                       upd.ctypes.data_as(_IP), int(upd.shape[0])))

    def _pack_empty(self, engine: "Engine") -> None:
        self._pack(engine, [], [], [], np.zeros((0, 4), dtype=np.int32))


class _PaddedGraph(_StepGraph):
    """Any step of several tokens a sequence, padded to ``tokens`` rows, ``seqs`` sequences and
    ``wants`` wanted places.  ``fresh``: every sequence starts at position 0 (whole prompts, which
    read nothing from the cache and take the kernels for that); else sequences go on from any
    position and may be mixed with fresh ones."""

    def __init__(self, engine: "Engine", tokens: int, seqs: int, wants: int, fresh: bool):
        self.tokens, self.seqs, self.wants = tokens, seqs, wants
        ngroups = len(engine.cache.groups)
        offs, o = {}, 0
        for name, n in layout(tokens, seqs, wants):
            offs[name] = (o, n)
            o += n
        # most pages a group can hand out in such a step: a sequence that goes on from the middle of
        # a page may touch one page more than its tokens fill
        self.upd_rows = -(-tokens // PAGE_TOKENS) + (1 if fresh else 2) * seqs
        self.upd_off = []
        for _ in range(ngroups):
            self.upd_off.append(o)
            o += 3 * self.upd_rows
        self._upd_off_c, _ = ints(self.upd_off)
        self._buffers(engine, o)
        views = {k: self.dev[a:a + n] for k, (a, n) in offs.items()}
        self.batch = StepBatch(**views, num_tokens=tokens, num_seqs=seqs, num_want=wants, max_new=tokens,
                               max_end=tokens if fresh else 0, all_decode=False, all_fresh=fresh, has_padding=True)

    def _pack(self, engine: "Engine", slots, starts, counts, tokens, want, updates: np.ndarray) -> None:
        sl, B = ints(slots)
        st, _ = ints(starts)
        ct, _ = ints(counts)
        wc, _ = ints([len(w) for w in want])
        flat = np.fromiter((x for t in tokens for x in t), dtype=np.int32, count=sum(counts))
        wflat = np.fromiter((x for w in want for x in w), dtype=np.int32)
        upd = np.ascontiguousarray(updates, dtype=np.int32)
        _ok(host_lib().moe_pack_padded(ctypes.cast(self.host.data_ptr(), _IP), self.tokens, self.seqs, self.wants, B,
                                       sl, st, ct, flat.ctypes.data_as(_IP), wc, wflat.ctypes.data_as(_IP),
                                       engine.cache.padding_slot, len(self.upd_off), self._upd_off_c, self.upd_rows,
                                       upd.ctypes.data_as(_IP), int(upd.shape[0])))

    def _pack_empty(self, engine: "Engine") -> None:
        self._pack(engine, [], [], [], [], [], np.zeros((0, 4), dtype=np.int32))


class StepHandle:
    """A step that was begun: where its sampled tokens (and, if asked for, what the model thought of
    them) arrive on the host."""

    def __init__(self, host: torch.Tensor, event: torch.cuda.Event, rows: int):
        self.host, self.event, self.rows = host, event, rows
        self.probe_host: Optional[torch.Tensor] = None
        self.top = 0
        # after the step is finished, per row: (logprob of its token, [(token, logprob)] strongest first)
        self.probes: Optional[List[Tuple[float, List[Tuple[int, float]]]]] = None


class Engine:
    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: Optional[int] = None,
                 use_graphs: Optional[bool] = None):
        self.model = model
        self.rt = model.rt
        if self.rt.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device; there is no CPU path")
        core.lib()   # fail now, loudly, if the kernels cannot be built or loaded
        if max_slots is None:
            max_slots = max(1, min(1024, -(-max_tokens // 64)))
        self.cache = KVCache(model.kv_requests(), model.state_requests(), max_tokens, max_slots,
                             self.rt.compute_dtype, self.rt.device)
        self.vocab_size = model.spec.vocab_size
        self._stage_host: Optional[torch.Tensor] = None
        self._stage_dev: Optional[torch.Tensor] = None
        self._stage_event = torch.cuda.Event()
        self._stage_busy = False
        self.steps_run = 0
        self.max_step_tokens = MAX_STEP_TOKENS
        parts = [p for b in model.blocks for p in b.parts()] + [model.embedding, model.final_norm, model.head]
        graph_safe = all(getattr(p, "graph_safe", False) for p in parts)
        self.use_graphs = graph_safe if use_graphs is None else (use_graphs and graph_safe)
        # any part may record what it decided, per call, as tuples of tensors appended to its
        # ``trace`` list (``Part.trace``, None when off)
        self._tracers = list({id(p): p for p in parts}.values())
        self.padded_graphs = os.environ.get("MOE_B200_PADDED_GRAPHS", "1") != "0"
        self._graphs: "OrderedDict[tuple, _StepGraph]" = OrderedDict()
        self._graph_pool = torch.cuda.graph_pool_handle() if self.use_graphs else None
        self._table_caps = [0 if g.ring_pages else g.max_pages_per_seq for g in self.cache.groups]
        self._results: List[Tuple[torch.Tensor, torch.cuda.Event]] = []     # pinned buffers for sampled tokens

    # ---- sequences -----------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- staging ---------------------------------------------------------------------
    def _staging(self, n: int) -> Tuple[np.ndarray, torch.Tensor]:
        if self._stage_busy:
            self._stage_event.synchronize()
            self._stage_busy = False
        if self._stage_host is None or self._stage_host.numel() < n:
            size = max(4096, 1 << (n - 1).bit_length())
            self._stage_host = torch.empty(size, dtype=torch.int32).pin_memory()
            self._stage_dev = torch.empty(size, dtype=torch.int32, device=self.rt.device)
        return self._stage_host.numpy(), self._stage_dev

    # ---- the step ----------------------------------------------------------------------
    def _reserve(self, slots: Sequence[int], counts: Sequence[int]) -> Tuple[List[int], np.ndarray]:
        """Give every sequence room for its new tokens, or change nothing and raise.  Returns each
        sequence's length before the step and the page-table entries that changed, [n, 4] of
        (group, slot, index, page).  (``moe_ledger_reserve`` of the host runtime.)"""
        return self.cache.ledger.reserve(slots, counts, self._table_caps, self.cache.max_tokens)

    def _graph(self, key: tuple, make) -> _StepGraph:
        """The captured step of this shape; the least recently used one is dropped beyond MAX_GRAPHS."""
        g = self._graphs.get(key)
        if g is None:
            while len(self._graphs) >= MAX_GRAPHS:
                self._graphs.popitem(last=False)
            g = self._graphs[key] = make()
        else:
            self._graphs.move_to_end(key)
        return g

    def graphs_of(self, kind: str) -> List[tuple]:
        """Keys of the captured steps of one kind: "decode" (one token each), "prompt" (every
        sequence from position 0) or "continued" (any other step)."""
        return [k for k in self._graphs if k[0] == kind]

    def truncate(self, slot: int, new_length: int) -> None:
        """Forget the sequence's tokens from ``new_length`` on (src/model.rs:176-189): the next step
        continues at that position.  Refused, changing nothing, where what was forgotten cannot be
        brought back: a windowed layer whose ring no longer holds the keys the next token needs, or a
        layer with state of fixed size."""
        self.cache.truncate(slot, new_length)

    def _bucket(self, B: int) -> Optional[int]:
        for b in GRAPH_BUCKETS:
            if b >= B:
                return b
        return None

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, check: bool = True,
             from_last: bool = False) -> Optional[torch.Tensor]:
        """Run ``tokens[i]`` for the sequence in ``slots[i]``; return logits at ``want[i]``.

        With ``from_last`` a token id of ``LAST_TOKEN`` (-1) stands for the token that the
        sampler picked last for that sequence; it is read on the device, so the step can be
        launched before the host has seen that token.

        ``want[i]`` lists places among ``tokens[i]`` (0 = its first token of this
        step); by default the last place of each sequence.  The result is a float32
        CUDA tensor [sum(len(w)), vocab], or None if nothing is wanted.  It may alias
        a buffer that the next step overwrites."""
        B = len(slots)
        if B == 0:
            return None
        if len(tokens) != B:
            raise ValueError("slots and tokens differ in length")
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        counts = [len(t) for t in tokens]
        if len(want) != B:
            raise ValueError("slots and want differ in length")
        for n, w in zip(counts, want):
            for i in w:
                if not 0 <= i < n:
                    raise ValueError(f"wanted place {i} is not among the {n} tokens of this step")
        if sum(counts) > self.max_step_tokens and not from_last:
            return self._step_in_pieces(slots, tokens, want, counts, check)
        starts, updates = self._reserve(slots, counts)
        self.steps_run += 1

        # ---- one token each: replay the bucket's graph -----------------------------------
        tracing = any(getattr(p, "trace", None) is not None for p in self._tracers)
        if (self.use_graphs and all(n == 1 for n in counts) and all(len(w) == 1 for w in want)
                and (from_last or min(t[0] for t in tokens) >= 0)):
            size = self._bucket(B)
            if size is not None:
                # one graph per (batch bucket, bucket of the longest sequence: powers of two from 256)
                reach = max(256, 1 << max(starts).bit_length())
                g = self._graph(("decode", size, reach, tracing), lambda: _DecodeGraph(self, size, reach))
                g.fill(self, slots, starts, [t[0] for t in tokens], updates)
                logits = g.run(self)
                self.last_batch = g.batch
                self.last_rows = B
                if check:
                    self.rt.check()
                return logits[:B]

        # ---- any other short step: replay the graph of its padded shape ------------------------
        T, W = sum(counts), sum(len(w) for w in want)
        if (self.use_graphs and self.padded_graphs and T <= STEP_TOKEN_BUCKETS[-1] and B <= STEP_SEQ_BUCKETS[-1]
                and W <= T and not from_last):
            tb = next(b for b in STEP_TOKEN_BUCKETS if b >= T)
            sb = next(b for b in STEP_SEQ_BUCKETS if b >= B)
            wb = sb if W <= sb else tb          # the last place of each sequence, or up to every place
            fresh = not any(starts)
            g = self._graph(("prompt" if fresh else "continued", tb, sb, wb, tracing),
                            lambda: _PaddedGraph(self, tb, sb, wb, fresh))
            g.fill(self, slots, starts, counts, tokens, want, updates)
            logits = g.run(self)
            self.last_batch = g.batch
            self.last_rows = B
            if check:
                self.rt.check()
            return logits[:W] if W else None

        # ---- the general step -----------------------------------------------------------------
        n_upd = int(updates.shape[0])
        host, dev = self._staging(3 * T + 4 * B + 2 + max(W, 1) + 3 * n_upd)
        info = fill_host(host, slots, starts, tokens, want)
        used = info["used"]
        upd_off: Dict[int, Tuple[int, int]] = {}
        if n_upd:
            o = used
            for gi in range(len(self.cache.groups)):
                mine = updates[updates[:, 0] == gi, 1:]
                if mine.shape[0]:
                    host[o:o + 3 * mine.shape[0]] = mine.reshape(-1)
                    upd_off[gi] = (o, int(mine.shape[0]))
                    o += 3 * mine.shape[0]
            used = o
        dev[:used].copy_(self._stage_host[:used], non_blocking=True)
        self._stage_event.record()
        self._stage_busy = True
        for gi, (o, n) in upd_off.items():
            core.table_update(self.cache.groups[gi].table, dev[o:o + 3 * n], n)
        views = {k: dev[a:a + n] for k, (a, n) in info["offsets"].items()}
        batch = StepBatch(**views, **info["facts"], last_token=self.cache.last_token if from_last else None)
        self.last_batch = batch
        self.last_rows = B
        logits = self.model.forward(batch, self.cache)
        if check:
            self.rt.check()
        return logits

    def _step_in_pieces(self, slots, tokens, want, counts, check) -> Optional[torch.Tensor]:
        """A step too large for one go: the sequences' tokens are fed in pieces of at most
        ``max_step_tokens`` together, sequence after sequence, each piece a step of its own that goes
        on from the cache.  The logits come back in the order asked for.  The cache is asked first
        whether the WHOLE step fits, so that it fails before the first piece or not at all."""
        self.cache.ledger.check(slots, counts, self._table_caps, self.cache.max_tokens)
        B = len(slots)
        done = [0] * B
        rows: Dict[Tuple[int, int], torch.Tensor] = {}
        while any(d < n for d, n in zip(done, counts)):
            room = self.max_step_tokens
            sl, tk, wn, who = [], [], [], []
            for i in range(B):
                n = min(counts[i] - done[i], room)
                if n <= 0:
                    continue
                lo, hi = done[i], done[i] + n
                sl.append(slots[i]), tk.append(tokens[i][lo:hi]), who.append(i)
                wn.append([w - lo for w in want[i] if lo <= w < hi])
                room -= n
            lg = self.step(sl, tk, wn, check=False)
            at = 0
            for i, w in zip(who, wn):
                for x in w:
                    rows[(i, x + done[i])] = lg[at].clone()
                    at += 1
            for i, t in zip(who, tk):
                done[i] += len(t)
        if check:
            self.rt.check()
        order = [(i, w) for i in range(B) for w in want[i]]
        return torch.stack([rows[k] for k in order]) if order else None

    def begin_step_and_sample(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], sampler, params,
                              histories=None, from_last: bool = False, logprobs: Optional[int] = None):
        """Launch one step and the sampling of one token per sequence from the logits at its last
        place, and start the copy of those tokens (and of the device status word) to pinned host
        memory.  Nothing waits for the device; ``finish_step_and_sample`` does.  A token id of
        ``LAST_TOKEN`` (with ``from_last``) is the token sampled last for that sequence, so the next
        step can be begun before this one is finished.  With ``logprobs`` (a number of alternatives,
        0 for none) the handle also brings what the model thought of each token, from the raw logits
        (``StepHandle.probes`` after the step is finished)."""
        logits = self.step(slots, tokens, None, check=False, from_last=from_last)
        B = len(slots)
        raw = logits
        if logprobs is not None and params.repeat_penalty != 1.0:
            raw = logits.clone()             # the penalty is applied to the logits in place
        picked = sampler.sample(logits, self.last_batch.slots[:B], params, histories)
        host, event = self._results.pop() if self._results else (
            torch.empty(self.cache.max_slots + 2, dtype=torch.int32).pin_memory(), torch.cuda.Event())
        host[:B + 1].copy_(torch.cat([picked, self.rt.status[:1]]), non_blocking=True)
        handle = StepHandle(host, event, B)
        if logprobs is not None:
            lp, ids, lps = core.logprobs(raw[:B], picked, int(logprobs))
            n = int(logprobs)
            handle.probe_host = torch.empty((B, 1 + 2 * n), dtype=torch.float32).pin_memory()
            handle.probe_host.copy_(torch.cat([lp[:, None], ids.to(torch.float32), lps], dim=1), non_blocking=True)
            handle.top = n
        event.record()
        return handle

    def finish_step_and_sample(self, handle) -> List[int]:
        handle.event.synchronize()
        B = handle.rows
        out = handle.host[:B + 1].tolist()
        self._results.append((handle.host, handle.event))
        if out[-1]:
            self.rt.check()
        if handle.probe_host is not None:
            n = handle.top
            rows = handle.probe_host.tolist()
            handle.probes = [(r[0], [(int(i), l) for i, l in zip(r[1:1 + n], r[1 + n:]) if i >= 0]) for r in rows]
        return out[:-1]

    def step_and_sample(self, slots: Sequence[int], tokens: Sequence[Sequence[int]], sampler, params,
                        histories=None) -> List[int]:
        """One step, then one sampled token per sequence; the tokens come back to the host."""
        return self.finish_step_and_sample(self.begin_step_and_sample(slots, tokens, sampler, params, histories))
