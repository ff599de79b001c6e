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
from ..weights import adopt_tensors, load_weights, random_weights
from .step import StepRuntime

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class PendingTokens:
    """Tokens that have been selected on the device and are on their way to the host."""

    def __init__(self, engine, device_tokens, host_tokens, event):
        self.engine, self.device_tokens, self.host_tokens, self.event = engine, device_tokens, host_tokens, event

    def tokens(self) -> list:
        self.event.synchronize()
        tokens = self.host_tokens.tolist()
        self.engine._raise_device_errors()
        return tokens


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0", page_size: int = 16,
                 max_tokens: int = 8192, max_seqs: int = 8, max_batch_tokens: int = 2048,
                 max_context: int = None, cuda_graphs: bool = True, profile: bool = False, _tensors=None):
        """`model_dir`: a folder with config.json and model.safetensors (or a sharded index).
        `max_tokens`: tokens the page pool of each cache group holds; `max_seqs`: request slots;
        `max_batch_tokens`: most tokens one step may bring; `max_context`: most positions of one
        request (default: the model's max_position_embeddings);
        `profile`: time every kernel class with CUDA events (`profile_summary()`); steps then run launch by launch,
        never as graphs (the reference's LIA_PROFILE likewise: src/inference/huggingface/minicpm5.rs:14-17).  It can
        be switched at any time by setting `engine.profile`;
        `cuda_graphs`: capture steps (decoded tokens, prompt portions, both) in CUDA graphs, one per
        shape of a step, when a shape comes a second time, and replay them."""
        if dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
        if not torch.cuda.is_available():
            raise RuntimeError("lia_rs_b200 needs a CUDA device: there is no CPU execution path")
        ops.lib()                                            # build/load the kernels now, loudly
        raw = _tensors[0].to_dict() if _tensors else read_config_json(model_dir)
        self.architecture = resolve_architecture(raw)
        self.config = _tensors[0] if _tensors else self.architecture.config_class.from_dict(raw)
        self.spec = self.architecture.build(self.config)
        self.dtype_name = "bfloat16" if _DTYPES[dtype] == torch.bfloat16 else "float32"
        self.runtime = Runtime(device, _DTYPES[dtype])
        self.device = self.runtime.device
        torch.cuda.set_device(self.device)
        if _tensors:
            tensors = adopt_tensors(_tensors[1], self.spec.tensor_specs())
        else:
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
        self.runtime_step = StepRuntime(self.cache, self.spec.vocab_size, self.max_batch_tokens, self.device)
        self.stats = {"steps": 0, "tokens": 0, "kernels": 0, "graph_replays": 0}
        self.cuda_graphs = bool(cuda_graphs) and self.model.graph_safe
        self.profile = bool(profile)
        self.profiler = ops.Profiler()
        # (tokens, wanted, context bucket, tokens of each entry) -> None (seen once) | (graph, logits, kernels, generation),
        # least recently used first
        self._graphs = {}
        self._capture_stream = None

    @classmethod
    def from_tensors(cls, config, tensors: dict, **options) -> "Engine":
        """An engine over tensors that are already in memory, by checkpoint name (they pass the loader's checks:
        missing, unexpected, wrong shapes, non-finite values), for a typed configuration."""
        return cls(None, _tensors=(config, tensors), **options)

    @classmethod
    def random(cls, config, seed: int = 0, **options) -> "Engine":
        """An engine with the weights that `weights.write_random_model(config, folder, seed)` would write (the
        same generator, the same values, through the loader's checks), without the folder: for sizes whose
        file would take long to write and read back."""
        return cls.from_tensors(config, random_weights(config, seed), **options)

    # ---- requests and pages (thin faces of the cache manager) ----
    def admit(self) -> int:
        return self.cache.admit()

    def reserve(self, slot: int, start: int, end: int) -> bool:
        return self.cache.ensure(slot, start, end)

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # ---- the step ----
    def step(self, entries, feed: "PendingTokens" = None) -> torch.Tensor:
        """Run one batch.  Returns 32-bit logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's `want`.  The pages for every position must have been reserved.
        With `feed` (tokens selected for the step before, perhaps not read by the host yet) every entry
        is one token, and entry i's token is row i of `feed`, taken on the device: the ids in the
        entries only stand in."""
        entries = list(entries)
        if not entries:
            return self.runtime_step.logits(0, self.spec.vocab_size)
        with torch.cuda.device(self.device):
            ctx = self.runtime_step.begin(entries, feed=None if feed is None else feed.device_tokens)
            if self.profile:
                ops.set_profiler(self.profiler)
                try:
                    logits = self._launch(ctx)
                finally:
                    ops.set_profiler(None)
            elif self.cuda_graphs:
                logits = self._replay(ctx)
            else:
                logits = self._launch(ctx)
            self.runtime_step.finish()
        self.stats["steps"] += 1
        self.stats["tokens"] += ctx.n_tokens - ctx.padding
        return logits[:ctx.n_out - ctx.padding] if ctx.padding else logits

    def _launch(self, ctx) -> torch.Tensor:
        before = ops.kernel_launches()
        logits = self.model.forward(ctx)
        self.stats["kernels"] += ops.kernel_launches() - before
        return logits

    MAX_GRAPHS = 64

    def _replay(self, ctx) -> torch.Tensor:
        """A step through its CUDA graph.  The step's metadata (token ids, positions, slots, wanted rows,
        the portions' starts) and the block tables lie in fixed device buffers, and what the host decides about
        a step's launches follows from the step's numbers of tokens, of wanted rows, of single-token entries and of
        portions, the context bucket and what the parts add (`Part.graph_key`: the attention's number of tiles); so
        a graph captured for these serves every later step that agrees in them, however its tokens are divided
        among its entries: every decode step of a batch, the portions of a long prompt that a scheduler cuts under
        one budget, and the full-budget steps of a mixed load whose portions differ in length.  The first
        step of a shape runs launch by launch (it allocates the workspace); the second is captured; a
        reallocation of any buffer makes the captured graphs stale.  The least recently used graphs go when
        there are more than MAX_GRAPHS shapes."""
        key = self.model.graph_key(ctx)
        entry = self._graphs.pop(key, False)
        if entry is False:
            self._graphs[key] = None
            while len(self._graphs) > self.MAX_GRAPHS:
                del self._graphs[next(iter(self._graphs))]
            return self._launch(ctx)
        if entry is None or entry[3] != self.runtime_step.generation:
            graph = torch.cuda.CUDAGraph()
            before = ops.kernel_launches()
            # Captured on a stream of the engine's own between capture_begin and capture_end, not through
            # `torch.cuda.graph`: that context synchronises the device, collects garbage and empties the
            # allocator's cache at every entry (15 ms a capture; a third of a mixed workload's 0.83 s went there).
            # Nothing is allocated during a capture: the shape's first step, launched kernel by kernel, has made the
            # workspace.
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(device=self.device)
            current = torch.cuda.current_stream(self.device)
            self._capture_stream.wait_stream(current)
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin()
                try:
                    logits = self.model.forward(ctx)
                finally:
                    graph.capture_end()
            current.wait_stream(self._capture_stream)
            entry = (graph, logits, ops.kernel_launches() - before, self.runtime_step.generation)
        self._graphs[key] = entry                        # most recently used last
        graph, logits, kernels, _ = entry
        graph.replay()
        self.stats["kernels"] += kernels
        self.stats["graph_replays"] += 1
        return logits

    # ---- token selection ----
    def select_tokens(self, logits: torch.Tensor, samplings, positions) -> list:
        """One token per row of `logits` on the device (greedy, or Gumbel-max keyed by seed and
        position); returns host integers.  This is the step's device-to-host read."""
        return self.select_tokens_start(logits, samplings, positions).tokens()

    def select_tokens_start(self, logits: torch.Tensor, samplings, positions) -> "PendingTokens":
        """The same, without waiting: the tokens are selected on the device and copied to pinned host
        memory behind the step; `PendingTokens.tokens()` waits for that copy.  Meanwhile the next step may
        be launched with the tokens fed on the device (`step(..., feed=)`)."""
        rows = logits.shape[0]
        out = self._workspace("select.out", (1, max(rows, self.max_seqs)), torch.int32)[0, :rows]
        if all(s.greedy for s in samplings):
            ops.select_tokens(logits, out)
        else:
            temperature = torch.tensor([s.temperature for s in samplings], dtype=torch.float32)
            seeds = torch.tensor([s.seed & 0x7FFFFFFFFFFFFFFF for s in samplings], dtype=torch.int64)
            where = torch.tensor(list(positions), dtype=torch.int64)
            ops.select_tokens(logits, out, temperature.to(self.device), seeds.to(self.device),
                              where.to(self.device))
        if not hasattr(self, "_select_host"):
            self._select_host = [torch.empty(self.max_seqs, dtype=torch.int32, pin_memory=True) for _ in range(2)]
            self._select_events = [torch.cuda.Event() for _ in range(2)]
            self._select_turn = 0
        self._select_turn ^= 1                      # two buffers: a copy may be in flight while the one before is read
        host, event = self._select_host[self._select_turn], self._select_events[self._select_turn]
        if rows > host.numel():
            host = self._select_host[self._select_turn] = torch.empty(rows, dtype=torch.int32, pin_memory=True)
        host[:rows].copy_(out, non_blocking=True)
        event.record()
        return PendingTokens(self, out, host[:rows], event)

    def select_candidates(self, logits: torch.Tensor, k: int, temperatures=None):
        """The best `k` logits of every row and their token ids on the host (float32 [rows, k], int32 [rows, k],
        best first, ids of -1 where a row has fewer): all that a sampling rule which keeps at most k tokens needs
        of a row, instead of the row.  With `temperatures` (one a row, 0 where none is needed) a third result,
        float64 [rows, 2]: each row's largest logit and the 64-bit sum of exp((x - largest) / temperature) over the
        whole row, by which a rule without top_k can tell whether its kept tokens lie within the candidates.
        Raises if a logit is not finite, as the host's rule would."""
        rows = logits.shape[0]
        most = max(rows, self.max_seqs)
        values = self._workspace("select.candidate_values", (most, k), torch.float32)[:rows]
        ids = self._workspace("select.candidate_ids", (most, k), torch.int32)[:rows]
        odd = self._workspace("select.nonfinite", (1, 1), torch.int32)
        odd.zero_()
        if temperatures is None:
            ops.select_candidates(logits, k, values, ids, odd[0])
            host_mass = None
        else:
            wanted = self._workspace("select.temperatures", (1, most), torch.float64)[0, :rows]
            wanted.copy_(torch.tensor([float(t) for t in temperatures], dtype=torch.float64))
            mass = self._workspace("select.mass", (most, 2), torch.float64)[:rows]
            ops.select_candidates(logits, k, values, ids, odd[0], wanted, mass)
            host_mass = mass.cpu().numpy()
        host_values, host_ids, count = values.cpu().numpy(), ids.cpu().numpy(), int(odd.item())
        self._raise_device_errors()
        if count:
            raise ValueError("nonfinite output logits")
        return (host_values, host_ids) if temperatures is None else (host_values, host_ids, host_mass)

    def logits_to_host(self, logits: torch.Tensor):
        rows = logits.float().cpu().numpy()
        self._raise_device_errors()
        return rows

    def profile_summary(self) -> dict:
        """kernel class -> {calls, ms, bytes, flops} of the steps run with `profile` on since the last call.
        Classes are the library's kernels, products further told apart by what they are to the layer
        ("gemm_skinny:qkv"); bytes and flops are what a roofline counts (every operand once; for attention
        the cache of the single-token rows, or the flops of the prompt portions)."""
        return self.profiler.summary()

    def synchronize(self) -> None:
        """Wait for the device and raise if a kernel flagged an error."""
        torch.cuda.synchronize(self.device)
        self._raise_device_errors()

    def _raise_device_errors(self):
        self.runtime_step.raise_device_errors()

    def _workspace(self, name, shape, dtype):
        return self.runtime_step.workspace(name, shape, dtype)
