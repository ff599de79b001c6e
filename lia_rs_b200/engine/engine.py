"""The engine: a model from a folder, its cache manager, its workspace, and `step()`.

    engine = Engine("model_dir", dtype="bfloat16", max_tokens=4096)
    slot = engine.admit()
    engine.reserve(slot, 0, 3)                       # pages for positions 0..2
    logits = engine.step([StepEntry(slot, [5, 17, 3], 0, want=[2])])
    engine.release(slot)

`dtype="bfloat16"` runs the kernels and precisions that serving uses; `dtype="float32"` runs the
whole model in true 32-bit: 32-bit weights, activations, cache, and products on the FMA pipes.
"""
from __future__ import annotations

import torch

from ..cache import CacheManager
from ..config import read_config_json, resolve_architecture
from ..kernels import ops
from ..models import DecoderModel
from ..parts import Runtime
from ..weights import load_weights
from .step import StepContext, StepEntry, StepError

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0", page_size: int = 16,
                 max_tokens: int = 8192, max_seqs: int = 8, max_batch_tokens: int = 2048,
                 max_context: int = None):
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
        if not torch.cuda.is_available():
            raise RuntimeError("lia_rs_b200 needs a CUDA device: there is no CPU execution path")
        ops.lib()                                            # build/load the kernels now, loudly
        raw = read_config_json(model_dir)
        self.architecture = resolve_architecture(raw)
        self.config = self.architecture.config_class.from_dict(raw)
        self.spec = self.architecture.build(self.config)
        self.dtype_name = "bfloat16" if _DTYPES[dtype] == torch.bfloat16 else "float32"
        self.runtime = Runtime(device, _DTYPES[dtype])
        self.device = self.runtime.device
        torch.cuda.set_device(self.device)
        tensors = load_weights(model_dir, self.spec.tensor_specs())
        self.model = DecoderModel(self.spec, tensors, self.runtime)
        del tensors
        self.page_size = int(page_size)
        self.max_seqs = int(max_seqs)
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_context = int(max_context or self.spec.max_positions)
        if self.max_context > self.spec.max_positions:
            raise ValueError(f"max_context {self.max_context} exceeds the model's {self.spec.max_positions} positions")
        num_pages = max(1, (int(max_tokens) + self.page_size - 1) // self.page_size)
        self.cache = CacheManager(self.spec.cache_requests(), self.spec.state_requests(), num_pages,
                                  self.page_size, self.max_seqs, self.max_context, self.runtime.compute_dtype,
                                  self.device)
        cap = self.max_batch_tokens
        self._meta_host = torch.zeros(4 * cap, dtype=torch.int32, pin_memory=True)
        self._meta_device = torch.zeros(4 * cap, dtype=torch.int32, device=self.device)
        self._error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._error_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._copy_event = torch.cuda.Event()
        self._buffers = {}
        self._logits_buffer = None
        self.stats = {"steps": 0, "tokens": 0}

    # ---- requests and pages (thin faces of the cache manager) ----
    def admit(self) -> int:
        return self.cache.admit()

    def reserve(self, slot: int, start: int, end: int) -> bool:
        return self.cache.ensure(slot, start, end)

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # ---- memory ----
    def _workspace(self, name, shape, dtype):
        rows, width = shape
        key = (name, width, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            buf = torch.empty((max(rows, self.max_batch_tokens), width), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def _logits(self, rows, vocab):
        buf = self._logits_buffer
        if buf is None or buf.shape[0] < rows:
            buf = torch.empty((max(rows, self.max_seqs), vocab), dtype=torch.float32, device=self.device)
            self._logits_buffer = buf
        return buf[:rows]

    # ---- the step ----
    def step(self, entries) -> torch.Tensor:
        """Run one batch.  Returns 32-bit logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's `want`.  The pages for every position must have been reserved."""
        tokens, positions, slots, out_rows, segments = [], [], [], [], []
        seen = set()
        vocab = self.spec.vocab_size
        for entry in entries:
            count = len(entry.tokens)
            if count == 0:
                raise StepError("a step entry brings no tokens")
            if entry.slot in seen:
                raise StepError(f"request slot {entry.slot} appears twice in one step")
            seen.add(entry.slot)
            if entry.slot not in self.cache._live:
                raise StepError(f"request slot {entry.slot} is not live")
            if entry.start < 0 or entry.start + count > self.cache.length[entry.slot]:
                raise StepError(f"slot {entry.slot}: positions [{entry.start}, {entry.start + count}) have no "
                                f"reserved pages (reserved up to {self.cache.length[entry.slot]})")
            low, high = min(entry.tokens), max(entry.tokens)
            if low < 0 or high >= vocab:
                raise StepError(f"token id {low if low < 0 else high} is outside the vocabulary of {vocab}")
            offset = len(tokens)
            for w in entry.want:
                if not 0 <= w < count:
                    raise StepError(f"wanted index {w} is outside the entry's {count} tokens")
                out_rows.append(offset + w)
            segments.append((entry.slot, entry.start, count, offset))
            tokens.extend(entry.tokens)
            positions.extend(range(entry.start, entry.start + count))
            slots.extend([entry.slot] * count)
        n, n_out, cap = len(tokens), len(out_rows), self.max_batch_tokens
        if n == 0:
            return self._logits(0, vocab)
        if n > cap:
            raise StepError(f"{n} tokens in one step exceed max_batch_tokens={cap}")
        self._copy_event.synchronize()               # the staging buffer of the last step is free again
        self._raise_device_errors()
        host = self._meta_host
        host[0:n] = torch.tensor(tokens, dtype=torch.int32)
        host[cap:cap + n] = torch.tensor(positions, dtype=torch.int32)
        host[2 * cap:2 * cap + n] = torch.tensor(slots, dtype=torch.int32)
        if n_out:
            host[3 * cap:3 * cap + n_out] = torch.tensor(out_rows, dtype=torch.int32)
        with torch.cuda.device(self.device):
            self._meta_device.copy_(host, non_blocking=True)
            self.cache.flush()
            self._copy_event.record()
            ctx = StepContext(self, n, n_out, segments)
            logits = self.model.forward(ctx)
            self._error_host.copy_(self._error_flag, non_blocking=True)
        self.stats["steps"] += 1
        self.stats["tokens"] += n
        return logits

    def synchronize(self) -> None:
        """Wait for the device and raise if a kernel flagged an error."""
        torch.cuda.synchronize(self.device)
        self._raise_device_errors()

    def _raise_device_errors(self):
        code = int(self._error_host[0])
        if code:
            self._error_host[0] = 0
            self._error_flag.zero_()
            raise StepError({1: "a token id outside the vocabulary reached the embedding kernel",
                             2: "a token's block table entry has no page"}.get(code, f"device error {code}"))

    def _attention(self, ctx, q, kv, out, nq, nkv, d, window, scale):
        ops.attention_generic(q, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table, out,
                              nq, nkv, d, window, scale)
