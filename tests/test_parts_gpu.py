"""Each part alone, built from a PartSpec at sizes of its own, against the plain implementation's
function for that part; and the order of layers as data (a layer run twice, a layer that reads
another layer's cache)."""
import math

import pytest
import torch

import helpers
import plain_impl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def harness(dtype, cache_requests=None, page_size=4, max_tokens=256, max_slots=2):
    from lia_rs_b200.cache import CacheManager
    from lia_rs_b200.engine import StepRuntime
    from lia_rs_b200.parts import Runtime
    rt = Runtime(DEV, TORCH[dtype])
    cache = CacheManager(cache_requests or {}, {}, max_tokens // page_size, page_size, max_slots, 512,
                         TORCH[dtype], DEV)
    return rt, StepRuntime(cache, 1000, 256, DEV)


def weights_for(specs, scale=1.0):
    torch.manual_seed(len(specs))
    out = {}
    for spec in specs:
        if spec.kind == "norm":
            out[spec.name] = (torch.rand(spec.shape) + 0.5).to(torch.bfloat16)
        else:
            out[spec.name] = (torch.randn(spec.shape) * scale / math.sqrt(spec.shape[-1])).to(torch.bfloat16)
    return out


def run_in_portions(step_runtime, portions, call):
    """Feed `portions` (token counts) of one request through `call(ctx, lo, hi)`."""
    from lia_rs_b200.engine import StepEntry
    slot = step_runtime.cache.admit()
    at = 0
    for count in portions:
        assert step_runtime.cache.ensure(slot, at, at + count)
        ctx = step_runtime.begin([StepEntry(slot, [1] * count, at, [])])
        call(ctx, at, at + count)
        at += count
    torch.cuda.synchronize()
    step_runtime.raise_device_errors()


def limit(dtype, reference):
    return (1e-4 if dtype == "float32" else 1e-2) * max(1.0, float(reference.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from lia_rs_b200.parts import NORMS
    rt, step = harness(dtype)
    params = {"hidden": 200, "eps": 1e-4}
    w = weights_for(NORMS["rmsnorm"].tensor_specs(params, "n."))
    part = NORMS["rmsnorm"](params, {k: v.to(DEV) for k, v in w.items()}, "n.", rt)
    x = torch.randn(9, 200, device=DEV)
    out = torch.empty(9, 200, device=DEV, dtype=TORCH[dtype])
    part.forward(None, x, out)
    want = plain_impl.rms_norm(x.double().cpu(), w["n.weight"], 1e-4)
    assert float((out.double().cpu() - want).abs().max()) <= limit(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 7])
def test_attention_mixer_part_in_portions(dtype, window):
    from lia_rs_b200.parts import MIXERS, PartSpec
    hidden, heads, kv_heads, d, theta = 80, 5, 1, 32, 1234.0
    params = {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": d, "window": window,
              "position": PartSpec("rotary", {"theta": theta, "rotary_dim": d})}
    cls = MIXERS["gqa_attention"]
    rt, step = harness(dtype, {0: cls.cache_request(params)})
    w = weights_for(cls.tensor_specs(params, "L.self_attn."), scale=3.0)
    part = cls(params, {k: v.to(DEV) for k, v in w.items()}, "L.self_attn.", rt)
    T = 37
    x = torch.randn(T, hidden).to(torch.bfloat16)
    residual = torch.zeros(T, hidden, device=DEV)

    def call(ctx, lo, hi):
        part.forward(ctx, x[lo:hi].to(DEV).to(TORCH[dtype]).contiguous(), residual[lo:hi], 0.5,
                     kv=ctx.kv_view(0, True))

    run_in_portions(step, [5, 2, 1, 1, 13, 3, 12], call)
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": d, "hidden_size": hidden,
           "rope_theta": theta}
    store = plain_impl._identity if dtype == "float32" else plain_impl.round_to_bfloat16
    want = 0.5 * plain_impl.attention_mixer(x.double(), w, "L.", cfg, torch.arange(T), window, torch.float64, store)
    assert float((residual.double().cpu() - want).abs().max()) <= limit(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part_adds_into_the_residual(dtype):
    from lia_rs_b200.parts import FEED_FORWARDS
    params = {"hidden": 72, "intermediate": 200}
    cls = FEED_FORWARDS["swiglu"]
    rt, step = harness(dtype)
    w = weights_for(cls.tensor_specs(params, "L.mlp."), scale=2.0)
    part = cls(params, {k: v.to(DEV) for k, v in w.items()}, "L.mlp.", rt)
    x = torch.randn(11, 72).to(torch.bfloat16)
    base = torch.randn(11, 72)
    residual = base.clone().to(DEV)
    run_in_portions(step, [11], lambda ctx, lo, hi: part.forward(ctx, x.to(DEV).to(TORCH[dtype]), residual, 0.7))
    store = plain_impl._identity if dtype == "float32" else plain_impl.round_to_bfloat16
    want = base.double() + 0.7 * plain_impl.swiglu_feed_forward(x.double(), w, "L.", torch.float64, store)
    assert float((residual.double().cpu() - want).abs().max()) <= limit(dtype, want)


def small_config(layers=2):
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=48, intermediate_size=80,
                num_hidden_layers=layers, num_attention_heads=3, num_key_value_heads=3, head_dim=16, vocab_size=97,
                max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=100.0, tie_word_embeddings=False,
                scale_depth=2.0, initializer_range=0.2, hidden_act="silu")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_part(dtype):
    from lia_rs_b200 import LlamaConfig
    from lia_rs_b200.models.minicpm5_llama import build_llama
    from lia_rs_b200.parts import build_layer, layer_tensor_specs
    raw = small_config()
    spec = build_llama(LlamaConfig.from_dict(raw))
    layer = spec.layers[1]
    prefix = "model.layers.1."
    w = weights_for(layer_tensor_specs(layer, prefix), scale=1.5)
    rt, step = harness(dtype, {0: spec.cache_requests()[1]})
    block = build_layer(layer, {k: v.to(DEV) for k, v in w.items()}, prefix, rt)
    T = 21
    h0 = torch.randn(T, 48)
    h = h0.clone().to(DEV)
    run_in_portions(step, [8, 1, 12], lambda ctx, lo, hi: block.forward(ctx, h[lo:hi], kv=ctx.kv_view(0, True)))
    store = plain_impl._identity if dtype == "float32" else plain_impl.round_to_bfloat16
    want = plain_impl.decoder_block(h0.double(), w, 1, raw, torch.arange(T), None, torch.float64, store)
    assert float((h.double().cpu() - want).abs().max()) <= limit(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_order_of_layers_is_data(tmp_path, dtype):
    """A model whose list runs layer 0 twice (with a second cache) and lets the last entry read the
    cache that the first wrote, registered from the test."""
    from safetensors.torch import load_file
    from lia_rs_b200 import LlamaConfig, register_architecture, write_random_model
    from lia_rs_b200.engine import Engine
    from lia_rs_b200.models import ScheduleEntry
    from lia_rs_b200.models.minicpm5_llama import build_llama

    def build_looped(config):
        spec = build_llama(config)
        spec.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                         ScheduleEntry(1, 0, writes=False)]
        spec.__post_init__()
        return spec

    register_architecture("LoopedLlamaForTest", LlamaConfig, build_looped)
    raw = dict(small_config(), architectures=["LoopedLlamaForTest"])
    folder = write_random_model(LlamaConfig.from_dict(raw), str(tmp_path / "looped"), seed=1)
    weights = load_file(folder + "/model.safetensors")
    tokens = helpers.random_tokens(97, 26, 4)
    store = plain_impl._identity if dtype == "float32" else plain_impl.round_to_bfloat16
    want = plain_impl.forward(raw, weights, tokens, order=[0, 1, 0, 1], reads={3: 0}, store=store)
    engine = Engine(folder, dtype=dtype, page_size=4, max_tokens=64, max_seqs=2, max_batch_tokens=64)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].cache_ids == [0, 1, 2]
    replay = helpers.Replayer(engine)
    got = [replay.step([("a", tokens[:9], range(9))]), replay.step([("a", tokens[9:11], range(2))])]
    got += [replay.step([("a", [t], [0])]) for t in tokens[11:]]
    import numpy as np
    helpers.assert_close(np.concatenate(got), want, dtype, "looped order")


@pytest.mark.parametrize("M,N,K", [(1, 16384, 512), (8, 16384, 512), (24, 16384, 264), (8, 2048, 512), (16, 2048, 1024),
                                   (24, 2048, 512), (40, 1024, 2048), (300, 1024, 512), (8, 1000, 100), (5, 333, 72)])
def test_linear_gives_the_product_whichever_kernel_it_chooses(M, N, K):
    """`linear` sends a bfloat16 product to one of four kernels by its shape (many output tiles: the tcgen05
    kernel at any number of tokens; few tokens: the streaming kernel; more: the cluster kernel; what TMA cannot
    address: the streaming kernel or the 32-bit pipes): every choice gives the product, with every epilogue."""
    from lia_rs_b200.parts import Runtime
    from lia_rs_b200.parts.linear import ACCUM, STORE, SWIGLU, linear
    rt = Runtime(DEV, torch.bfloat16)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    out = torch.empty(M, N, device=DEV)
    linear(rt, STORE, a, w[:N], out, 0.5)
    assert float((out.double() - 0.5 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(max(K, 64) / 64)
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    linear(rt, ACCUM, a, w[:N], acc, 1.5)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(max(K, 64) / 64)
    act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    linear(rt, SWIGLU, a, w, act)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
