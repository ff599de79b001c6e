"""A toy mixer with state of its own, defined here, registered, built and stepped without a change
to the framework's files: it proves the interfaces for a new mixer and a new architecture."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def define_toy():
    from lia_rs_b200 import LlamaConfig, register_architecture
    from lia_rs_b200.models.minicpm5_llama import build_llama
    from lia_rs_b200.parts import Mixer, PartSpec, StateRequest, register_mixer
    from lia_rs_b200.parts.block import LayerSpec
    from lia_rs_b200.weights import TensorSpec

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """out_t = W . mean(x_0 .. x_t).  Per-request state: the running sum and the count, carried
        from step to step in a slot of fixed size; no pages."""

        @staticmethod
        def tensor_specs(params, prefix):
            return [TensorSpec(prefix + "mix.weight", (params["hidden"], params["hidden"]))]

        @staticmethod
        def state_request(params):
            return StateRequest((params["hidden"] + 1,), torch.float32)

        def __init__(self, params, tensors, prefix, runtime):
            super().__init__(params, tensors, prefix, runtime)
            self.weight = tensors[prefix + "mix.weight"].float()

        def forward(self, ctx, x, residual, scale, kv=None, state=None):
            for slot, start, count, offset in ctx.segments:
                if start == 0:
                    state[slot].zero_()
                rows = x[offset:offset + count].float()
                sums = state[slot, :-1] + torch.cumsum(rows, dim=0)
                counts = state[slot, -1] + torch.arange(1, count + 1, device=x.device, dtype=torch.float32)
                residual[offset:offset + count].add_((sums / counts[:, None]) @ self.weight.T, alpha=scale)
                state[slot, :-1] = sums[-1]
                state[slot, -1] = counts[-1]

    def build_toy(config):
        spec = build_llama(config)
        first = spec.layers[0]
        spec.layers[0] = LayerSpec(mixer=PartSpec("toy_running_mean", {"hidden": config.hidden_size}),
                                   feed_forward=first.feed_forward, norm=first.norm,
                                   residual_scale=first.residual_scale)
        spec.schedule = []
        spec.__post_init__()
        return spec

    register_architecture("ToyStateForTest", LlamaConfig, build_toy)


def plain_toy(raw, weights, tokens):
    """The same model with dense torch operations, whole sequence, 64-bit."""
    import plain_impl
    t = torch.as_tensor(tokens)
    h = plain_impl.embedding(t, weights["model.embed_tokens.weight"], 1.0, torch.float64)
    positions = torch.arange(len(tokens))
    eps = raw["rms_norm_eps"]
    x = plain_impl.rms_norm(h, weights["model.layers.0.input_layernorm.weight"], eps)
    mean = torch.cumsum(x, dim=0) / torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
    h = h + mean @ weights["model.layers.0.self_attn.mix.weight"].double().T
    x = plain_impl.rms_norm(h, weights["model.layers.0.post_attention_layernorm.weight"], eps)
    h = h + plain_impl.swiglu_feed_forward(x, weights, "model.layers.0.", torch.float64)
    h = plain_impl.decoder_block(h, weights, 1, raw, positions, None, torch.float64)
    return plain_impl.lm_head(h, weights, raw, torch.float64)


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from safetensors.torch import load_file
    from lia_rs_b200 import LlamaConfig, write_random_model
    from lia_rs_b200.engine import Engine
    define_toy()
    raw = dict(architectures=["ToyStateForTest"], model_type="toy", hidden_size=32, intermediate_size=48,
               num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=16, vocab_size=61,
               max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=100.0, tie_word_embeddings=True,
               initializer_range=0.3, hidden_act="silu")
    folder = write_random_model(LlamaConfig.from_dict(raw), str(tmp_path / "toy"), seed=5)
    weights = load_file(folder + "/model.safetensors")
    assert "model.layers.0.self_attn.mix.weight" in weights and "model.layers.0.self_attn.q_proj.weight" not in weights
    engine = Engine(folder, dtype="float32", page_size=4, max_tokens=64, max_seqs=3, max_batch_tokens=64)
    assert list(engine.cache.states) == [0] and engine.cache.states[0].shape == (3, 33)
    assert [g.cache_ids for g in engine.cache.groups] == [[1]]        # only the attention layer has pages
    a, b = helpers.random_tokens(61, 23, 1), helpers.random_tokens(61, 11, 2)
    replay = helpers.Replayer(engine)
    got_a, got_b = [], []
    got_a.append(replay.step([("a", a[:6], range(6))]))
    both = replay.step([("a", a[6:8], range(2)), ("b", b[:5], range(5))])
    got_a.append(both[:2]); got_b.append(both[2:])
    for i in range(8, 23):
        entries = [("a", [a[i]], [0])]
        if i - 3 < 11:
            entries.append(("b", [b[i - 3]], [0]))
        out = replay.step(entries, end=["b"] if i - 3 == 10 else [])
        got_a.append(out[:1])
        if len(entries) == 2:
            got_b.append(out[1:])
    helpers.assert_close(np.concatenate(got_a), plain_toy(raw, weights, a), "float32", "toy a")
    helpers.assert_close(np.concatenate(got_b), plain_toy(raw, weights, b), "float32", "toy b")
    # the freed slot is used again by a new request and its state starts from zero
    c = helpers.random_tokens(61, 9, 3)
    helpers.assert_close(replay.step([("c", c, range(9))]), plain_toy(raw, weights, c), "float32", "toy c")
