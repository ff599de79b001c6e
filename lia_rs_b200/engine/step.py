"""The step function: one batch of (request, its next tokens), prompt portions beside single
decoded tokens, cut anywhere; it runs only the tokens it is given, from the cache, and returns
the logits at the wanted places.

The reference's counterpart is `Engine::forward_paged(rows, tables, outputs)`
(src/inference/paging.rs:97-109): rows of (token, position, sequence), one block table per
sequence, and the indices of the rows whose logits are returned.  Its host checks are kept
(src/inference/paging.rs:120-172): positions of a request are consecutive, no request appears
twice in a step, every token id is in the vocabulary, pages exist for every row.

`StepRuntime` owns what a step needs besides the model: the cache manager, the staging of the
step's metadata (host pinned -> device, one copy), the workspace that parts take their buffers
from, and the device error flag.  `StepContext` is the view of one step that the parts see.  Which
attention kernel serves which rows is the mixer's side (parts/paged_attention.py).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import ctypes

import numpy as np
import torch

from ..cache.pages import host_library
from ..kernels import ops


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

    def __init__(self, runtime, n_tokens, n_out, segments, meta, padding=0):
        self.runtime = runtime
        # rows of the batch and of the logits, padding rows included: what the kernels run
        self.n_tokens, self.n_out = n_tokens, n_out
        # `padding` rows at the end of a step of single tokens bring it to a round number of rows (fewer shapes to
        # capture); they have slot -1 on the device, which every kernel that touches the cache skips, and are not
        # among the segments
        self.padding = padding
        self.segments = segments                      # [(slot, start, count, offset in the batch)]
        self.n_single = sum(1 for _, _, count, _ in segments if count == 1) + padding
        (self.tokens, self.positions, self.slots, self.out_rows, self.decode_rows, self.prefill_rows,
         self.prefill_segments) = meta
        self.n_prefill_segments = sum(1 for _, _, count, _ in segments if count > 1)
        self.error_flag = runtime.error_flag
        self.decode_only = all(count == 1 for _, _, count, _ in segments)
        self.max_context = max((start + count for _, start, count, _ in segments), default=0)
        # the longest context of the step, rounded up to a power of two (at least 1024): kernels that cut
        # their work by context length do it by this, and a captured step is replayed within one bucket
        self.context_bucket = 1 << max(10, (max(self.max_context, 1) - 1).bit_length())

    def buffer(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """A buffer [rows, width] of the workspace; the same name, width and type give the same
        memory in every step (a part must not expect it to survive a step)."""
        return self.runtime.workspace(name, shape, dtype)

    def logits_buffer(self, rows: int, vocab: int) -> torch.Tensor:
        return self.runtime.logits(rows, vocab)

    def kv_view(self, cache_id, writes):
        return self.runtime.cache.kv_view(cache_id, writes)

    def state(self, state_id):
        return self.runtime.cache.state(state_id)

    def attention(self, q, kv, out, nq, nkv, d, window, scale):
        """out = causal softmax attention of the encoded queries q over the cache `kv`, for the tokens of this
        step: a convenience for a mixer that keeps no `parts.PagedAttention` of its own (one is built, and its
        kernels chosen, the first time these sizes are asked for; a head size that no kernel takes raises
        ValueError with the kernels' limits)."""
        from ..parts.paged_attention import PagedAttention
        key = (q.dtype, nq, nkv, d, window, float(scale))
        attention = self.runtime._attentions.get(key)
        if attention is None:
            attention = self.runtime._attentions[key] = PagedAttention(q.dtype, nq, nkv, d, window, scale)
        attention.forward(self, q, kv, out)


class StepRuntime:
    def __init__(self, cache, vocab_size: int, max_batch_tokens: int, device):
        self.cache = cache
        self.vocab_size = int(vocab_size)
        self.max_batch_tokens = int(max_batch_tokens)
        self.device = torch.device(device)
        cap = self.max_batch_tokens
        self._meta_host = torch.zeros(7 * cap, dtype=torch.int32, pin_memory=True)
        self._meta_view = self._meta_host.numpy()       # the same memory, for writing slices without a tensor each
        self._meta_device = torch.zeros(7 * cap, dtype=torch.int32, device=self.device)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._error_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._copy_event = torch.cuda.Event()
        self._host = host_library()
        self._summary = (ctypes.c_int * 8)()
        self._buffers = {}
        self._attentions = {}
        self._logits_buffer = None
        self.generation = 0            # grows whenever a buffer is (re)allocated: captured graphs are stale then

    # ---- memory ----
    def workspace(self, name, shape, dtype):
        rows, width = shape
        key = (name, width, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            buf = torch.empty((max(rows, self.max_batch_tokens), width), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:rows]

    def scratch(self, name, numel, dtype):
        """A flat scratch buffer of at least `numel` elements (grows, never shrinks)."""
        buf = self._buffers.get((name, dtype))
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._buffers[(name, dtype)] = buf
            self.generation += 1
        return buf[:numel]

    def counters(self, count):
        """`count` int32 words that are zero and that every kernel using them leaves zero."""
        buf = self._buffers.get("counters")
        if buf is None or buf.numel() < count:
            buf = torch.zeros(max(count, 4096), dtype=torch.int32, device=self.device)
            self._buffers["counters"] = buf
            self.generation += 1
        return buf[:count]

    def logits(self, rows, vocab):
        buf = self._logits_buffer
        if buf is None or buf.shape[0] < rows or buf.shape[1] != vocab:
            buf = torch.empty((max(rows, self.cache.max_slots), vocab), dtype=torch.float32, device=self.device)
            self._logits_buffer = buf
            self.generation += 1
        return buf[:rows]

    # ---- a step's metadata ----
    def begin(self, entries, feed=None) -> StepContext:
        """Check the batch, stage its metadata and the changed block-table rows on the device,
        and return the context for the model.  `feed` (int32, on the device): the token of entry i is
        feed[i] (every entry then brings one token, whose id in the entry only stands in)."""
        # the entries, flattened for the native side: it checks the batch (no request twice, positions covered by
        # reserved pages, token ids inside the vocabulary, wanted places among an entry's tokens) and writes the
        # metadata straight into the pinned staging buffer (csrc/host/step_host.cpp)
        n_entries = len(entries)
        counts = [len(entry.tokens) for entry in entries]
        if n_entries and min(counts) == 1 == max(counts):
            tokens = [entry.tokens[0] for entry in entries]
        else:
            tokens = [t for entry in entries for t in entry.tokens]
        wants = [w for entry in entries for w in entry.want]
        Entries = ctypes.c_int * max(1, n_entries)
        try:
            slot_list, start_list = [entry.slot for entry in entries], [entry.start for entry in entries]
            for values in (slot_list, start_list, wants):       # (a ctypes integer would wrap silently)
                if values and not (-2**31 <= min(values) and max(values) < 2**31):
                    raise StepError("a step entry's slot, start and wanted places must fit 32 bits")
            slots, starts = Entries(*slot_list), Entries(*start_list)
            token_array = np.asarray(tokens, dtype=np.int64)
            if token_array.size and (token_array.min() < -2**31 or token_array.max() >= 2**31):
                bad = int(token_array.min() if token_array.min() < 0 else token_array.max())
                raise StepError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
            token_array = token_array.astype(np.int32)
            want_array = (ctypes.c_int * max(1, len(wants)))(*wants)
        except (TypeError, OverflowError) as error:
            raise StepError(f"a step entry's numbers must be integers: {error}") from None
        self._copy_event.synchronize()               # the staging buffer of the last step is free again
        self.raise_device_errors()
        host = self._meta_host
        if self._host.lia_step_stage(self.cache.native_handle(), n_entries, slots, starts, Entries(*counts),
                                     ctypes.c_void_p(token_array.ctypes.data), Entries(*[len(entry.want) for entry in entries]),
                                     want_array, self.vocab_size, self.max_batch_tokens, self.PAD_ABOVE, self.PAD_TO,
                                     ctypes.c_void_p(host.data_ptr()), ctypes.c_longlong(host.numel()), self._summary) < 0:
            message = self._host.lia_host_error()
            raise StepError(message.decode() if message else "the step was refused")
        n, n_out, padding, n_single, n_portions, total = self._summary[:6]
        real = n - padding
        segments, offset = [], 0
        for entry, count in zip(entries, counts):
            segments.append((entry.slot, entry.start, count, offset))
            offset += count
        self._meta_device[:total].copy_(host[:total], non_blocking=True)
        if feed is not None:
            if any(count != 1 for _, _, count, _ in segments) or feed.numel() < real or feed.dtype != torch.int32:
                raise StepError("tokens can be fed on the device only to a step of single tokens, one per entry")
            self._meta_device[:real].copy_(feed[:real], non_blocking=True)
        self.cache.flush()
        self._copy_event.record()
        dev = self._meta_device
        at = 3 * n + n_out
        meta = (dev[0:n], dev[n:2 * n], dev[2 * n:3 * n], dev[3 * n:at], dev[at:at + n_single],
                dev[at + n_single:at + n], dev[at + n:total])
        self.h2d_bytes = total * 4
        return StepContext(self, n, n_out, segments, meta, padding)

    PAD_ABOVE, PAD_TO = 8, 8

    def padding_for(self, n_tokens: int, n_entries: int) -> int:
        """Rows of nobody behind a step of single tokens: beyond PAD_ABOVE entries the batch is brought to a
        multiple of PAD_TO rows (while the step's buffers have room), so that the steps of a batch whose requests
        end one after another are a few shapes, each captured once and replayed, instead of one shape per size
        (two launched steps each before a replay).  Smaller batches run as they are.  (The native side's rule.)"""
        return int(host_library().lia_step_padding(int(n_tokens), int(n_entries), self.PAD_ABOVE, self.PAD_TO,
                                                    self.max_batch_tokens))

    def finish(self):
        self._error_host.copy_(self.error_flag, non_blocking=True)

    def raise_device_errors(self):
        code = int(self._error_host[0])
        if code:
            self._error_host[0] = 0
            self.error_flag.zero_()
            if "counters" in self._buffers:                  # a kernel that gave up may have left these mid-count
                self._buffers["counters"].zero_()
            ops.reset_scratch(self.device)                   # and the split-K tile counters of the products
            raise StepError({1: "a token id outside the vocabulary reached the embedding kernel",
                             2: "a token's block table entry has no page",
                             3: "a kernel gave up waiting on an mbarrier"}.get(code, f"device error {code}"))
