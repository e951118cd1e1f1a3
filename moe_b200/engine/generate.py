"""The generation loop above the step function.

Per sequence it follows the reference's loop (src/generate.rs:142-320, without
drafting or grammars): the first token is sampled from the prompt's logits, so N
generated tokens cost N - 1 decode steps; a sampled end-of-sequence token is
neither emitted nor counted; the reasons to stop are Length, Eos, Caller and
Context (src/generate.rs:48-65).

What the reference does not have is the batch: requests are taken ``batch_size``
at a time; the prompts of a batch (of unequal lengths) run in one step, then
every live sequence advances by one token a step; a sequence that stops leaves
the batch and gives its slot back while the others go on; batches follow one
another until every request is served.  Results come back in request order.

The loop only decides; it drives a *stepper* (``EngineStepper`` in production, a
fake in the CPU tests) with four methods: ``new_sequence``, ``release``,
``seed`` and ``step_and_sample``.

A stepper may split ``step_and_sample`` into ``begin`` (launch, no waiting) and
``finish`` (the tokens).  The loop then works one step ahead: it begins step k+1
before it has finished step k, for the sequences that go on whatever token step k
gives them (by the counts: length and context), and feeds them ``LAST_TOKEN``,
which the device replaces by the token it sampled in step k.  The host's work for a
step is thereby hidden behind the device's.  A sequence that stops at step k for a
reason the counts do not show (end-of-sequence, the caller) has a row in step k+1
whose result is dropped.  The results are the same as without looking ahead.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.params import SamplingParams

LAST_TOKEN = -1      # fed for "the token sampled last for this sequence" when a step is begun ahead

LENGTH, EOS, CALLER, CONTEXT = "length", "eos", "caller", "context"


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    stop: str = LENGTH
    prompt_tokens: int = 0
    steps: int = 0            # decode steps this sequence took part in
    # with ``logprobs``: one entry per emitted token, (logprob of the token, [(token, logprob)] of the
    # most likely tokens at its place, strongest first), from the raw logits (src/generate.rs:78-105)
    logprobs: Optional[List[tuple]] = None

    @property
    def finish_reason(self) -> str:
        """'length' or 'stop', as the reference reports it (src/generate.rs:69-74)."""
        return "length" if self.stop in (LENGTH, CONTEXT) else "stop"


@dataclass
class GenerationStats:
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_seconds: float = 0.0


class EngineStepper:
    """Drives an ``Engine`` and the device sampler for the loop."""

    def __init__(self, engine):
        from ..sampling.sampler import DeviceSampler

        self.engine = engine
        self.sampler = DeviceSampler(engine.cache.rng_states, engine.rt.device, engine.cache.last_token)

    def new_sequence(self) -> int:
        return self.engine.new_sequence()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def seed(self, slots, seeds) -> None:
        self.sampler.seed(slots, seeds)

    def begin(self, slots, tokens, histories, params: SamplingParams, from_last: bool = False,
              logprobs: Optional[int] = None):
        return self.engine.begin_step_and_sample(slots, tokens, self.sampler, params, histories, from_last, logprobs)

    def finish(self, handle) -> List[int]:
        return self.engine.finish_step_and_sample(handle)

    def step_and_sample(self, slots, tokens, histories, params: SamplingParams) -> List[int]:
        return self.finish(self.begin(slots, tokens, histories, params))


def generate(stepper, prompts: Sequence[Sequence[int]], max_tokens: int = 128,
             sampling: Optional[SamplingParams] = None, eos: Sequence[int] = (), batch_size: Optional[int] = None,
             ctx: Optional[int] = None, on_token: Optional[Callable[[int, int], bool]] = None,
             stats: Optional[GenerationStats] = None, lookahead: Optional[bool] = None,
             logprobs: Optional[int] = None) -> List[GenerationResult]:
    """Generate up to ``max_tokens`` tokens after each prompt.

    ``on_token(request_index, token)`` sees every emitted token and returns False to
    stop that request (stop reason Caller).  ``ctx`` bounds a sequence's length in the
    cache (stop reason Context).  Request i samples with seed ``sampling.seed + i``.
    ``lookahead`` (default: on if the stepper has ``begin``/``finish``) begins each step
    before the one before it is finished; it is off with a repeat penalty, whose history
    the host must know.  ``logprobs`` (None: off; else the number of alternatives, 0 for none)
    reports for every emitted token what the model thought of it (``GenerationResult.logprobs``);
    it needs a stepper with ``begin``/``finish`` that brings them."""
    from ..cache.allocator import CacheError

    sampling = (sampling or SamplingParams()).validate()
    eos = set(int(e) for e in eos)
    n = len(prompts)
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
    results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
    if max_tokens <= 0 or n == 0:
        return results
    batch_size = batch_size or n
    stats = stats if stats is not None else GenerationStats()
    clock = time.perf_counter
    split = hasattr(stepper, "begin") and hasattr(stepper, "finish")
    look = split and (lookahead is None or lookahead) and sampling.repeat_penalty == 1.0
    if lookahead and not look:
        raise ValueError("lookahead needs a stepper with begin/finish and no repeat penalty")
    if logprobs is not None:
        if not split:
            raise ValueError("logprobs need a stepper with begin/finish")
        if not 0 <= int(logprobs) <= 64:
            raise ValueError("logprobs: between 0 and 64 alternatives")
        for r in results:
            r.logprobs = []

    for b0 in range(0, n, batch_size):
        ids = list(range(b0, min(n, b0 + batch_size)))
        slot = {i: stepper.new_sequence() for i in ids}
        try:
            stepper.seed([slot[i] for i in ids], [sampling.seed + i for i in ids])
            history = {i: list(prompts[i]) for i in ids}
            alive = set(ids)

            def commit(i: int, tok: int, cached: int, probe=None) -> bool:
                """Judge the token sampled for request i, whose sequence then holds ``cached`` tokens
                in the cache; True if the request goes on."""
                r = results[i]
                if tok in eos:
                    r.stop = EOS
                    return False
                if ctx is not None and cached >= ctx:
                    r.stop = CONTEXT
                    return False
                history[i].append(tok)
                r.tokens.append(tok)
                if r.logprobs is not None:
                    r.logprobs.append(probe)
                if on_token is not None and not on_token(i, tok):
                    r.stop = CALLER
                    return False
                if len(r.tokens) >= max_tokens:
                    r.stop = LENGTH
                    return False
                return True

            def launch(who, toks, cached, from_last):
                """Begin a step; ``cached[i]`` is the length of i's sequence in the cache after it."""
                sl, hs = [slot[i] for i in who], [history[i] for i in who]
                if split and logprobs is not None:
                    return who, stepper.begin(sl, toks, hs, sampling, from_last, logprobs=int(logprobs)), cached
                if split:
                    return who, stepper.begin(sl, toks, hs, sampling, from_last), cached
                return who, stepper.step_and_sample(sl, toks, hs, sampling), cached

            t0 = clock()
            flights = [launch(ids, [list(prompts[i]) for i in ids], {i: len(prompts[i]) for i in ids}, False)]
            prefill = True
            while flights:
                if look and len(flights) == 1:
                    # who goes on whatever the step in flight gives them: one more token fits both
                    # the request's budget and the context
                    who, _, cached = flights[0]
                    ahead = [i for i in who if i in alive and len(results[i].tokens) + 1 < max_tokens
                             and (ctx is None or cached[i] < ctx)]
                    if ahead:
                        try:
                            flights.append(launch(ahead, [[LAST_TOKEN]] * len(ahead),
                                                  {i: cached[i] + 1 for i in ahead}, True))
                        except CacheError:
                            pass        # no room for all of them: wait for the tokens, some may stop
                who, handle, cached = flights.pop(0)
                picked = stepper.finish(handle) if split else handle
                probes = getattr(handle, "probes", None) if logprobs is not None else None
                if prefill:
                    stats.prefill_seconds += clock() - t0
                    stats.prefill_tokens += sum(len(prompts[i]) for i in ids)
                    t0 = clock()
                elif any(i in alive for i in who):
                    stats.decode_steps += 1
                for row, (i, tok) in enumerate(zip(who, picked)):
                    if i not in alive:
                        continue            # stopped while this step was already in flight
                    if not prefill:
                        results[i].steps += 1
                        stats.decode_tokens += 1
                    if not commit(i, int(tok), cached[i], probes[row] if probes is not None else None):
                        alive.discard(i)
                        stepper.release(slot.pop(i))
                prefill = False
                if not flights:
                    live = [i for i in who if i in alive]
                    if live:
                        flights.append(launch(live, [[results[i].tokens[-1]] for i in live],
                                              {i: cached[i] + 1 for i in live}, False))
            stats.decode_seconds += clock() - t0
        finally:
            for s in slot.values():
                stepper.release(s)
    return results
