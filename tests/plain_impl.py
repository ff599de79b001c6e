"""Plain, slow implementation of the MiniCPM5 Llama decoder: whole sequences, no cache.

This file is the oracle of the test-suite.  It shares no code with the package: it takes a
plain dict (the parsed config.json) and a dict of tensors by checkpoint name, and computes
everything with dense torch operations on the CPU, one function per part.

Anchoring.  The reference project's model code exists only as Rust device code behind its
`cuda` feature (src/lib.rs:6-11), it accepts one fixed 42-layer geometry
(src/models/minicpm5.rs:7-31) and no Rust toolchain is available where these tests run, so
the reference cannot be executed on a tiny random model.  This implementation therefore
rests on the reference's formulas, each cited by file:line below, plus MiniCPM's three
scalars (scale_emb, scale_depth, dim_model_base) and tied embeddings, which the reference
does not have and which reduce to the reference's plain Llama when the keys are absent.
"""
from __future__ import annotations

import math

import torch


def _f(cfg, key, default):
    v = cfg.get(key, default)
    return default if v is None else v


def head_dim_of(cfg) -> int:
    return int(_f(cfg, "head_dim", cfg["hidden_size"] // cfg["num_attention_heads"]))


def layer_windows(cfg) -> list:
    """Per layer: None (all keys) or the window length (keys pos-w+1 .. pos are visible)."""
    n = cfg["num_hidden_layers"]
    window = cfg.get("sliding_window")
    kinds = cfg.get("layer_types") or ["full_attention"] * n
    out = []
    for kind in kinds:
        if kind == "sliding_attention":
            out.append(int(window))
        else:
            out.append(None)
    return out


def embedding(tokens: torch.Tensor, table: torch.Tensor, scale_emb: float, dtype) -> torch.Tensor:
    """h0[t,:] = E[token_t,:] (src/gpu/kernels/basic.rs:51-73: bf16 row widened to f32),
    times MiniCPM's scale_emb."""
    return table[tokens.long()].to(dtype) * scale_emb


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * 1/sqrt(mean(x^2) + eps) * w, the weight used as stored (no +1)
    (src/gpu/kernels/normalization.rs:46-112)."""
    mean_square = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(mean_square + eps)) * weight.to(x.dtype)


def rotary(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE over the whole head: inv_i = 1/theta^(2i/d), a = pos*inv_i,
    out[i] = x[i] cos a - x[i+d/2] sin a, out[i+d/2] = x[i+d/2] cos a + x[i] sin a
    (src/gpu/kernels/llama.rs:44-55, src/gpu/kernels/llama_position.rs:35-46,78-105).
    x: [T, heads, d]."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (2.0 * i / d))
    angle = positions.to(torch.float64)[:, None] * inv[None, :]
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    left, right = x[..., :half], x[..., half:]
    return torch.cat([left * cos - right * sin, right * cos + left * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window, store=None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.  q-head h reads kv-head
    h div g; s_j = (q.k_j)/sqrt(d) for keys j <= pos (src/gpu/kernels/llama.rs:62-159,
    GQA map src/gpu/kernels/llama_flash_math.rs:152); with a window w only keys
    j > pos - w are visible.  q: [T, nq, d], k, v: [T, nkv, d] -> [T, nq, d]."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    pos = torch.arange(T)
    out = torch.empty_like(q)
    rows_at_a_time = 1024          # of a long sequence the score matrix is made a band of query rows at a time (memory only)
    for begin in range(0, T, rows_at_a_time):
        rows = pos[begin:begin + rows_at_a_time]
        visible = pos[None, :] <= rows[:, None]
        if window is not None:
            visible &= pos[None, :] > (rows[:, None] - window)
        for h in range(nq):
            kh = h // g
            scores = (q[rows, h, :] @ k[:, kh, :].T) * (1.0 / math.sqrt(d))
            scores = scores.masked_fill(~visible, float("-inf"))
            if store is None:
                out[rows, h, :] = torch.softmax(scores, dim=-1) @ v[:, kh, :]
            else:
                # the serving path feeds 16-bit probabilities to the tensor cores and divides by the
                # 32-bit sum afterwards; it takes the exponentials in base 2 against a whole-number
                # reference point, so that the 16-bit mantissas do not depend on how the keys are tiled
                log2_scores = scores * math.log2(math.e)
                p = torch.exp2(log2_scores - torch.ceil(log2_scores.max(dim=-1, keepdim=True).values))
                out[rows, h, :] = (store(p) @ v[:, kh, :]) / p.sum(dim=-1, keepdim=True)
    return out


def _identity(x):
    return x


def round_to_bfloat16(x: torch.Tensor) -> torch.Tensor:
    """The values that survive a store in bfloat16 (round to nearest even), kept in x's type."""
    return x.to(torch.float32).to(torch.bfloat16).to(x.dtype)


def attention_mixer(x, w, prefix, cfg, positions, window, dtype, store=_identity, store_p=None, kv=None,
                    keep=None):
    """q,k,v projections without bias (src/inference/llama.rs:92-112), RoPE on q and k,
    attention, output projection (src/inference/llama.rs:290-298).  `kv` = (k, v) of another layer
    replaces this layer's own keys and values (a layer that reads another layer's cache); `keep`
    (a list) receives this layer's (k, v)."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    T = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].to(dtype).T).view(T, nq, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].to(dtype).T).view(T, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].to(dtype).T).view(T, nkv, d)
    theta = float(_f(cfg, "rope_theta", 10000.0))
    q = store(rotary(q, positions, theta))
    k = store(rotary(k, positions, theta))
    v = store(v)
    if kv is not None:
        k, v = kv
    if keep is not None:
        keep.append((k, v))
    o = store(attention(q, k, v, window, store_p).reshape(T, nq * d))
    return o @ w[prefix + "self_attn.o_proj.weight"].to(dtype).T


def swiglu_feed_forward(x, w, prefix, dtype, store=_identity):
    """act = up * gate/(1+exp(-gate)); f = act W_down^T (src/inference/moe.rs:31-61,
    src/gpu/kernels/basic.rs:150-157)."""
    gate = x @ w[prefix + "mlp.gate_proj.weight"].to(dtype).T
    up = x @ w[prefix + "mlp.up_proj.weight"].to(dtype).T
    act = store(up * (gate / (1.0 + torch.exp(-gate))))
    return act @ w[prefix + "mlp.down_proj.weight"].to(dtype).T


def decoder_block(h, w, layer, cfg, positions, window, dtype, store=_identity, store_p=None, kv=None,
                  keep=None):
    """Pre-norm block: r = h + s*attn(norm(h)); h' = r + s*ffn(norm(r))
    (src/inference/llama_fusion.rs:41-117), s = scale_depth/sqrt(num_layers) (MiniCPM) or 1."""
    prefix = f"model.layers.{layer}."
    eps = float(cfg["rms_norm_eps"])
    scale_depth = cfg.get("scale_depth")
    s = 1.0 if scale_depth is None else float(scale_depth) / math.sqrt(cfg["num_hidden_layers"])
    a = attention_mixer(store(rms_norm(h, w[prefix + "input_layernorm.weight"], eps)), w, prefix, cfg,
                        positions, window, dtype, store, store_p, kv, keep)
    r = h + a * s
    f = swiglu_feed_forward(store(rms_norm(r, w[prefix + "post_attention_layernorm.weight"], eps)), w,
                            prefix, dtype, store)
    return r + f * s


def lm_head(h, w, cfg, dtype, store=_identity):
    """Final RMSNorm (src/inference/paging.rs:310-315), division by hidden_size/dim_model_base
    (MiniCPM), product with the output matrix, which is the embedding table when tied
    (src/inference/paging.rs:316)."""
    y = rms_norm(h, w["model.norm.weight"], float(cfg["rms_norm_eps"]))
    y = store(y)
    base = cfg.get("dim_model_base")
    if base is not None:
        y = y / (cfg["hidden_size"] / float(base))
    if cfg.get("tie_word_embeddings", False):
        out = w["model.embed_tokens.weight"]
    else:
        out = w["lm_head.weight"]
    return y @ out.to(dtype).T


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, order=None, store=_identity,
            store_p=None, reads=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence.  `order` is the list of layer
    indices to run (default 0..L-1).  `store` is applied wherever the serving path keeps a value
    in 16 bits between kernels (normalised activations, rotated q and k, v, attention output,
    the SwiGLU product, the final normalised row): the identity gives the exact model,
    `round_to_bfloat16` the model that the bfloat16 path computes, up to the order of sums.
    `store_p` (None or a rounding) is applied to the unnormalised softmax probabilities, which the
    tensor-core attention kernels feed to the tensor cores in 16 bits.  `reads` maps a place in
    `order` to an earlier place whose keys and values that entry uses instead of its own."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    h = embedding(tokens, weights["model.embed_tokens.weight"], float(_f(cfg, "scale_emb", 1.0)), dtype)
    windows = layer_windows(cfg)
    kept = []
    for place, layer in enumerate(order if order is not None else range(cfg["num_hidden_layers"])):
        source = (reads or {}).get(place)
        h = decoder_block(h, weights, layer, cfg, positions, windows[layer], dtype, store, store_p,
                          kv=None if source is None else kept[source], keep=kept)
    return lm_head(h, weights, cfg, dtype, store)


def greedy(cfg, weights, prompt, steps: int, dtype=torch.float64) -> list:
    """Greedy continuation by whole-sequence recomputation.  Ties go to the larger token id,
    as the reference's max_by over total_cmp keeps the last maximum
    (src/server/paged/request.rs:117-124)."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        row = forward(cfg, weights, tokens, dtype)[-1]
        best = row.max()
        token = int(torch.nonzero(row == best).max())
        out.append(token)
        tokens.append(token)
    return out


# ---------------------------------------------------------------------------------------
# Sampling (the reference samples on the CPU in f64).

class MT19937:
    """Mersenne twister with the reference's two-word double (src/sampling/random.rs:8-46)."""

    def __init__(self, seed: int):
        self.words = [0] * 624
        self.words[0] = seed & 0xFFFFFFFF
        for i in range(1, 624):
            prev = self.words[i - 1]
            self.words[i] = (1812433253 * (prev ^ (prev >> 30)) + i) & 0xFFFFFFFF
        self.index = 624

    def next(self) -> int:
        if self.index == 624:
            for i in range(624):
                mixed = (self.words[i] & 0x80000000) | (self.words[(i + 1) % 624] & 0x7FFFFFFF)
                self.words[i] = self.words[(i + 397) % 624] ^ (mixed >> 1) ^ (0x9908B0DF if mixed & 1 else 0)
            self.index = 0
        value = self.words[self.index]
        self.index += 1
        value ^= value >> 11
        value ^= (value << 7) & 0x9D2C5680
        value ^= (value << 15) & 0xEFC60000
        return (value ^ (value >> 18)) & 0xFFFFFFFF

    def uniform(self) -> float:
        low = float(self.next())
        high = float(self.next())
        return min((low + high * 4294967296.0) / 18446744073709551616.0, 1.0 - 2.0 ** -53)


def distribution(logits, temperature: float, top_k: int, top_p: float) -> list:
    """Sorted (token, probability) entries: descending logit, ties to the larger id; keep
    top_k (0 = all); weights exp((x-max)/T) in f64; keep the shortest prefix whose mass
    reaches top_p * total; renormalise (src/sampling.rs:82-131)."""
    items = [(i, float(x)) for i, x in enumerate(logits) if x != float("-inf")]
    items.sort(key=lambda e: (-e[1], -e[0]))
    if top_k and len(items) > top_k:
        items = items[:top_k]
    top = items[0][1]
    entries = [(i, math.exp((x - top) / temperature)) for i, x in items]
    total = sum(p for _, p in entries)
    mass = 0.0
    keep = len(entries)
    for n, (_, p) in enumerate(entries):
        mass += p
        if mass >= top_p * total:
            keep = n + 1
            break
    entries = entries[:keep]
    total = sum(p for _, p in entries)
    return [(i, p / total) for i, p in entries]


def draw(entries, rng: MT19937) -> int:
    """Inverse CDF over the sorted entries; a single entry consumes no random number
    (src/sampling.rs:134-186)."""
    if len(entries) == 1:
        return entries[0][0]
    sample = rng.uniform()
    cumulative = 0.0
    for token, p in entries:
        cumulative += p
        if sample < cumulative:
            return token
    return entries[-1][0]
