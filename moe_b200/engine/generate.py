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
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..sampling.params import SamplingParams

LENGTH, EOS, CALLER, CONTEXT = "length", "eos", "caller", "context"


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    stop: str = LENGTH
    prompt_tokens: int = 0
    steps: int = 0            # decode steps this sequence took part in

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
        self.sampler = DeviceSampler(engine.cache.rng_states, engine.rt.device)

    def new_sequence(self) -> int:
        return self.engine.new_sequence()

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def seed(self, slots, seeds) -> None:
        self.sampler.seed(slots, seeds)

    def step_and_sample(self, slots, tokens, histories, params: SamplingParams) -> List[int]:
        return self.engine.step_and_sample(slots, tokens, self.sampler, params, histories)


def generate(stepper, prompts: Sequence[Sequence[int]], max_tokens: int = 128,
             sampling: Optional[SamplingParams] = None, eos: Sequence[int] = (), batch_size: Optional[int] = None,
             ctx: Optional[int] = None, on_token: Optional[Callable[[int, int], bool]] = None,
             stats: Optional[GenerationStats] = None) -> List[GenerationResult]:
    """Generate up to ``max_tokens`` tokens after each prompt.

    ``on_token(request_index, token)`` sees every emitted token and returns False to
    stop that request (stop reason Caller).  ``ctx`` bounds a sequence's length in the
    cache (stop reason Context).  Request i samples with seed ``sampling.seed + i``."""
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

    for b0 in range(0, n, batch_size):
        ids = list(range(b0, min(n, b0 + batch_size)))
        slot = {i: stepper.new_sequence() for i in ids}
        try:
            stepper.seed([slot[i] for i in ids], [sampling.seed + i for i in ids])
            history = {i: list(prompts[i]) for i in ids}
            length = {i: len(prompts[i]) for i in ids}      # tokens in the cache after the next step

            def commit(i: int, tok: int) -> bool:
                """Judge the token sampled for request i; True if the request goes on."""
                r = results[i]
                if tok in eos:
                    r.stop = EOS
                    return False
                if ctx is not None and length[i] >= ctx:
                    r.stop = CONTEXT
                    return False
                history[i].append(tok)
                r.tokens.append(tok)
                if on_token is not None and not on_token(i, tok):
                    r.stop = CALLER
                    return False
                if len(r.tokens) >= max_tokens:
                    r.stop = LENGTH
                    return False
                return True

            t0 = clock()
            first = stepper.step_and_sample([slot[i] for i in ids], [list(prompts[i]) for i in ids],
                                            [history[i] for i in ids], sampling)
            stats.prefill_seconds += clock() - t0
            stats.prefill_tokens += sum(len(prompts[i]) for i in ids)
            live = []
            for i, tok in zip(ids, first):
                if commit(i, int(tok)):
                    live.append(i)
                else:
                    stepper.release(slot.pop(i))
            t0 = clock()
            while live:
                pend = [[results[i].tokens[-1]] for i in live]
                nxt = stepper.step_and_sample([slot[i] for i in live], pend, [history[i] for i in live], sampling)
                stats.decode_steps += 1
                stats.decode_tokens += len(live)
                still = []
                for i, tok in zip(live, nxt):
                    length[i] += 1
                    results[i].steps += 1
                    if commit(i, int(tok)):
                        still.append(i)
                    else:
                        stepper.release(slot.pop(i))
                live = still
            stats.decode_seconds += clock() - t0
        finally:
            for s in slot.values():
                stepper.release(s)
    return results
