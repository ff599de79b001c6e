"""The Python entry point: token ids in, token ids out.

    from lia_rs_b200 import generate
    outputs = generate("model_dir", [[1, 2, 3], [4, 5]], max_tokens=16)            # greedy
    outputs = generate("model_dir", prompts, max_tokens=16, temperature=0.8, seed=7)

Options carry the reference's names and meanings where it has them: request fields `max_tokens`,
`temperature`, `top_k`, `top_p`, `seed`, `presence_penalty` (src/server/sampling.rs:32-90,
src/server/paged/request.rs:40-48) and service options `max_sequences` (1..64, default 8),
`kv_pool_tokens` (default 65536), `context` (default 16384) and the prefill batch, the step's
token budget (128..4096, default 512) (src/server/options.rs:24-76, src/main.rs:85-90,
src/inference/initialize.rs:175-182).  The reference tokenises chat requests; this engine takes
token ids.
"""
from __future__ import annotations

from typing import Optional, Sequence

from ..sampling import Sampling
from .engine import Engine
from .scheduler import Scheduler


class Generator:
    """An engine with its scheduler, kept for repeated calls."""

    def __init__(self, model: str, dtype: str = "bfloat16", context: int = 16384, max_sequences: int = 8,
                 kv_pool_tokens: int = 65536, prefill_batch: int = 512, page_size: int = 16,
                 device: str = "cuda:0", even_split: bool = False):
        if not 1 <= max_sequences <= 64:
            raise ValueError("max-sequences must be 1..=64")
        if kv_pool_tokens < page_size or kv_pool_tokens % page_size:
            raise ValueError(f"KV pool must be a positive number of whole {page_size}-token pages")
        if prefill_batch <= 0:
            raise ValueError("prefill batch must be positive")
        self.engine = Engine(model, dtype=dtype, device=device, page_size=page_size, max_tokens=kv_pool_tokens,
                             max_seqs=max_sequences, max_batch_tokens=max(prefill_batch, max_sequences),
                             max_context=None)
        self.context = min(int(context), self.engine.max_context)
        self.engine.config.validate_capacity(self.context) if hasattr(self.engine.config, "validate_capacity") else None
        self.prefill_batch = int(prefill_batch)
        self.even_split = even_split
        self.last_scheduler = None

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 8192, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 42, presence_penalty: float = 0.0,
                 sampler: str = "mt19937", eos_token_ids: Optional[Sequence[int]] = None,
                 sampling: Optional[Sequence[Sampling]] = None) -> list:
        """Generated token ids for each prompt, in order.  `sampling` (one per prompt) overrides
        the scalar options.  A request that cannot be served raises."""
        eos = self.engine.spec.eos_token_ids if eos_token_ids is None else eos_token_ids
        scheduler = Scheduler(self.engine, max_batch_tokens=self.prefill_batch, even_split=self.even_split,
                              eos_token_ids=eos, context=self.context)
        self.last_scheduler = scheduler
        requests = []
        for i, prompt in enumerate(prompts):
            params = sampling[i] if sampling is not None else Sampling(
                temperature=temperature, top_k=top_k, top_p=top_p, seed=seed,
                presence_penalty=presence_penalty, sampler=sampler)
            requests.append(scheduler.add(i, prompt, params, max_tokens))
        try:
            scheduler.run()
        finally:
            for request in scheduler.live():
                self.engine.release(request.slot)
        for request in requests:
            if request.error:
                raise ValueError(f"request {request.rid}: {request.error}")
        return [list(r.generated) for r in requests]


def generate(model: str, prompts, max_tokens: int = 8192, dtype: str = "bfloat16", **options) -> list:
    """One-shot form of `Generator(...).generate(...)`.  Engine options (context, max_sequences,
    kv_pool_tokens, prefill_batch, page_size, device) and request options are told apart by name."""
    engine_keys = ("context", "max_sequences", "kv_pool_tokens", "prefill_batch", "page_size", "device",
                   "even_split")
    engine_options = {k: options.pop(k) for k in engine_keys if k in options}
    return Generator(model, dtype=dtype, **engine_options).generate(prompts, max_tokens=max_tokens, **options)
