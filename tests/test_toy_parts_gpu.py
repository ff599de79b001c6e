"""A toy feed-forward with routing and a toy position encoding, defined here, registered, built and
stepped without a change to the framework's files: they prove the interfaces for a new feed-forward and
a new position encoding (the toy mixer with state of its own is in test_toy_mixer_gpu.py).  Neither is a
model of anyone's."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

EXPERTS = 3


def define_toys():
    from lia_rs_b200 import LlamaConfig, register_architecture
    from lia_rs_b200.models.minicpm5_llama import build_llama
    from lia_rs_b200.parts import FeedForward, PartSpec, register_feed_forward
    from lia_rs_b200.parts.base import PositionEncoding, register_position_encoding
    from lia_rs_b200.parts.block import LayerSpec
    from lia_rs_b200.weights import TensorSpec

    @register_feed_forward("toy_routed")
    class Routed(FeedForward):
        """Each token goes to the ONE expert with the largest router logit (32-bit logits and softmax);
        out = p_e * tanh(x We^T), p_e the router's probability of that expert."""

        @staticmethod
        def tensor_specs(params, prefix):
            h = params["hidden"]
            return [TensorSpec(prefix + "router.weight", (EXPERTS, h))] + \
                   [TensorSpec(prefix + f"experts.{e}.weight", (h, h)) for e in range(EXPERTS)]

        def __init__(self, params, tensors, prefix, runtime):
            super().__init__(params, tensors, prefix, runtime)
            self.router = tensors[prefix + "router.weight"].float()
            self.experts = torch.stack([tensors[prefix + f"experts.{e}.weight"].float() for e in range(EXPERTS)])

        def forward(self, ctx, x, residual, scale):
            rows = x.float()
            probabilities = torch.softmax(rows @ self.router.T, dim=-1)
            weight, chosen = probabilities.max(dim=-1)
            outputs = torch.tanh(torch.einsum("th,tkh->tk", rows, self.experts[chosen]))
            residual.add_(outputs * weight[:, None], alpha=scale)

    @register_position_encoding("toy_decay")
    class Decay(PositionEncoding):
        """No rotation: the first half of every query and key head is multiplied by cos(position / period),
        the second half by sin(position / period + 1).  It uses the framework's append of keys and values."""

        def __init__(self, params, tensors, prefix, runtime):
            super().__init__(params, tensors, prefix, runtime)
            self.period = float(params["period"])

        def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d):
            positions = ctx.positions.float() / self.period
            factor = torch.cat([torch.cos(positions)[:, None].expand(-1, d // 2),
                                torch.sin(positions + 1.0)[:, None].expand(-1, d - d // 2)], dim=1)
            heads = qkv.view(qkv.shape[0], nq + 2 * nkv, d)
            heads[:, :nq + nkv] *= factor[:, None, :]                    # q and k; v stays
            self.runtime.ops.rope_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                           kv.v_pages, nq, nkv, d, 0, None, write_kv=kv.writes,
                                           error_flag=ctx.error_flag)

    def build_toys(config):
        spec = build_llama(config)
        first, second = spec.layers[0], spec.layers[1]
        spec.layers[0] = LayerSpec(mixer=first.mixer, feed_forward=PartSpec("toy_routed", {"hidden": config.hidden_size}),
                                   norm=first.norm, residual_scale=first.residual_scale)
        params = dict(second.mixer.params, position=PartSpec("toy_decay", {"period": 7.0}))
        spec.layers[1] = LayerSpec(mixer=PartSpec(second.mixer.kind, params), feed_forward=second.feed_forward,
                                   norm=second.norm, residual_scale=second.residual_scale)
        spec.schedule = []
        spec.__post_init__()
        return spec

    register_architecture("ToyPartsForTest", LlamaConfig, build_toys)


def plain_toys(raw, weights, tokens):
    """The same model with dense torch operations, whole sequence, 64-bit."""
    import plain_impl
    dtype = torch.float64
    t = torch.as_tensor(tokens)
    positions = torch.arange(len(tokens))
    eps = raw["rms_norm_eps"]
    h = plain_impl.embedding(t, weights["model.embed_tokens.weight"], 1.0, dtype)
    # layer 0: the framework's attention, then the routed feed-forward
    prefix = "model.layers.0."
    x = plain_impl.rms_norm(h, weights[prefix + "input_layernorm.weight"], eps)
    h = h + plain_impl.attention_mixer(x, weights, prefix, raw, positions, None, dtype)
    x = plain_impl.rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], eps)
    probabilities = torch.softmax(x @ weights[prefix + "mlp.router.weight"].double().T, dim=-1)
    weight, chosen = probabilities.max(dim=-1)
    experts = torch.stack([weights[prefix + f"mlp.experts.{e}.weight"].double() for e in range(EXPERTS)])
    h = h + torch.tanh(torch.einsum("th,tkh->tk", x, experts[chosen])) * weight[:, None]
    # layer 1: attention with the toy position encoding, then the framework's feed-forward
    prefix = "model.layers.1."
    x = plain_impl.rms_norm(h, weights[prefix + "input_layernorm.weight"], eps)
    nq, nkv, d = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    q = (x @ weights[prefix + "self_attn.q_proj.weight"].double().T).view(-1, nq, d)
    k = (x @ weights[prefix + "self_attn.k_proj.weight"].double().T).view(-1, nkv, d)
    v = (x @ weights[prefix + "self_attn.v_proj.weight"].double().T).view(-1, nkv, d)
    where = positions.double() / 7.0
    factor = torch.cat([torch.cos(where)[:, None].expand(-1, d // 2),
                        torch.sin(where + 1.0)[:, None].expand(-1, d - d // 2)], dim=1)[:, None, :]
    a = plain_impl.attention(q * factor, k * factor, v, None).reshape(len(tokens), nq * d)
    h = h + a @ weights[prefix + "self_attn.o_proj.weight"].double().T
    x = plain_impl.rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], eps)
    h = h + plain_impl.swiglu_feed_forward(x, weights, prefix, dtype)
    return plain_impl.lm_head(h, weights, raw, dtype), chosen


def test_toy_routed_feed_forward_and_toy_position_encoding_register_build_and_step(tmp_path):
    from safetensors.torch import load_file
    from lia_rs_b200 import LlamaConfig, write_random_model
    from lia_rs_b200.engine import Engine
    define_toys()
    raw = dict(architectures=["ToyPartsForTest"], model_type="toy", hidden_size=40, intermediate_size=56,
               num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=53,
               max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=50.0, tie_word_embeddings=False,
               initializer_range=0.4, hidden_act="silu")
    folder = write_random_model(LlamaConfig.from_dict(raw), str(tmp_path / "toys"), seed=11)
    weights = load_file(folder + "/model.safetensors")
    assert "model.layers.0.mlp.router.weight" in weights and "model.layers.0.mlp.gate_proj.weight" not in weights
    assert "model.layers.1.mlp.gate_proj.weight" in weights
    engine = Engine(folder, dtype="float32", page_size=4, max_tokens=96, max_seqs=3, max_batch_tokens=64)
    assert not engine.model.graph_safe               # the toys say nothing about graphs: the model runs launch by launch
    a, b = helpers.random_tokens(53, 29, 1), helpers.random_tokens(53, 13, 2)
    want_a, chosen_a = plain_toys(raw, weights, a)
    want_b, _ = plain_toys(raw, weights, b)
    assert len(set(chosen_a.tolist())) > 1            # the router does choose different experts
    replay = helpers.Replayer(engine)
    got_a, got_b = [], []
    got_a.append(replay.step([("a", a[:7], range(7))]))
    both = replay.step([("a", a[7:10], range(3)), ("b", b[:6], range(6))])
    got_a.append(both[:3]); got_b.append(both[3:])
    for i in range(10, 29):
        entries = [("a", [a[i]], [0])]
        if i - 4 < 13:
            entries.append(("b", [b[i - 4]], [0]))
        out = replay.step(entries, end=["b"] if i - 4 == 12 else [])
        got_a.append(out[:1])
        if len(entries) == 2:
            got_b.append(out[1:])
    helpers.assert_close(np.concatenate(got_a), want_a, "float32", "toy parts a")
    helpers.assert_close(np.concatenate(got_b), want_b, "float32", "toy parts b")
