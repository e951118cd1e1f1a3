"""The Python entry point for generation.

The reference's library API is ``Model::load(Store::open(path))``, ``State::new``,
``model.forward(&ids, &mut state)`` and ``generate(...)`` with a ``Plan``
(src/lib.rs:9-19, src/generate.rs:21-45).  Here:

    model  = moe_b200.load_model(path, dtype="bfloat16")
    engine = moe_b200.Engine(model, max_tokens=16384)
    outs   = moe_b200.generate(engine, [[1, 2, 3], [4, 5]], max_tokens=32, temp=0.8, seed=7)
    outs[0].tokens, outs[0].stop

Option names and defaults are the reference's (``Plan`` and ``Sampler``).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from .engine.generate import EngineStepper, GenerationResult, GenerationStats
from .engine.generate import generate as _loop
from .sampling.params import SamplingParams


def generate(engine, prompts: Sequence[Sequence[int]], max_tokens: int = 128, temp: float = 0.0,
             top_p: float = 0.95, top_k: int = 0, repeat_penalty: float = 1.0, seed: int = 0,
             eos: Optional[Sequence[int]] = None, batch_size: Optional[int] = None, ctx: Optional[int] = None,
             on_token: Optional[Callable[[int, int], bool]] = None,
             stats: Optional[GenerationStats] = None, lookahead: Optional[bool] = None,
             logprobs: int = 0) -> List[GenerationResult]:
    """Generate after each prompt (lists of token ids); see ``engine.generate.generate``.

    ``eos`` defaults to the model's ``eos_token_id``; pass ``()`` to ignore it.  ``logprobs`` N > 0
    (the reference's ``Plan::logprobs``, src/generate.rs:31): each result also lists, per emitted
    token, its logprob and the N most likely tokens at its place, from the raw logits."""
    if eos is None:
        eos = engine.model.spec.eos_token_ids
    params = SamplingParams(temp=temp, top_p=top_p, top_k=top_k, repeat_penalty=repeat_penalty, seed=seed)
    stepper = getattr(engine, "_stepper", None)
    if stepper is None:
        stepper = engine._stepper = EngineStepper(engine)
    return _loop(stepper, prompts, max_tokens=max_tokens, sampling=params, eos=eos, batch_size=batch_size, ctx=ctx,
                 on_token=on_token, stats=stats, lookahead=lookahead, logprobs=logprobs if logprobs > 0 else None)
