"""The step function: one batch of (request, its next tokens), prompt portions beside single
decoded tokens, cut anywhere; it runs only the tokens it is given, from the cache, and returns
the logits at the wanted places.

The reference's counterpart is `Engine::forward_paged(rows, tables, outputs)`
(src/inference/paging.rs:97-109): rows of (token, position, sequence), one block table per
sequence, and the indices of the rows whose logits are returned.  Its host checks are kept
(src/inference/paging.rs:120-172): positions of a request are consecutive, no request appears
twice in a step, every token id is in the vocabulary, pages exist for every row.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    """`tokens` are the next tokens of the request in `slot`, at positions start, start+1, ...;
    `want` lists the indices among these tokens whose logits are returned."""
    slot: int
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = field(default_factory=list)


class StepContext:
    """Everything the parts may ask for during one step."""

    def __init__(self, engine, n_tokens, n_out, segments):
        self.engine = engine
        self.n_tokens, self.n_out = n_tokens, n_out
        self.segments = segments                      # [(slot, start, count, offset in batch)]
        meta, cap = engine._meta_device, engine.max_batch_tokens
        self.tokens = meta[0:n_tokens]
        self.positions = meta[cap:cap + n_tokens]
        self.slots = meta[2 * cap:2 * cap + n_tokens]
        self.out_rows = meta[3 * cap:3 * cap + n_out]
        self.error_flag = engine._error_flag
        self.decode_only = all(count == 1 for _, _, count, _ in segments)
        self.max_context = max((start + count for _, start, count, _ in segments), default=0)

    def buffer(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        return self.engine._workspace(name, shape, dtype)

    def logits_buffer(self, rows: int, vocab: int) -> torch.Tensor:
        return self.engine._logits(rows, vocab)

    def kv_view(self, cache_id, writes):
        return self.engine.cache.kv_view(cache_id, writes)

    def state(self, state_id):
        return self.engine.cache.state(state_id)

    def attention(self, q, kv, out, nq, nkv, d, window, scale):
        """out = causal attention of q over the cache `kv`, for the tokens of this step."""
        self.engine._attention(self, q, kv, out, nq, nkv, d, window, scale)
