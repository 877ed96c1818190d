"""Gifudra through the framework's step function, cache manager and engine on a CPU (stand-in kernels), against the
plain implementation of `plain_gifudra.py`: every way of cutting the same requests gives the same logits."""

from __future__ import annotations

import json

import pytest
import torch

import gifudra_configs as gc
import plain_gifudra
import replay_harness as rh


@pytest.fixture(scope="module")
def gifudra_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("gifudra")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in gc.ALL.items()}


def expected_logits(model_dir, requests):
    config, tensors = plain_gifudra.read_model(model_dir)
    return {name: plain_gifudra.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


def full_trace(requests):
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda name: len(requests[name]))
    for i, token in enumerate(requests[longest]):            # every token a step of its own, from the first one on
        trace.add([(f"o-{longest}", [token], [0])], end=[f"o-{longest}"] if i == len(requests[longest]) - 1 else [])
    return trace


def test_config_round_trip_names_and_schedule(gifudra_dirs):
    from liteinfer_b200.config.gifudra_config import GifudraConfig
    from liteinfer_b200.config.model_config import ConfigError
    from liteinfer_b200.config.registry import resolve

    for name, (raw, _, _) in gc.ALL.items():
        arch, config = resolve(raw)
        assert arch.name == "Gifudra" and GifudraConfig.from_dict(config.to_dict()) == config
        assert GifudraConfig.from_dict(json.loads((gifudra_dirs[name] / "config.json").read_text())) == config
    arch, config = resolve(gc.GIF_A)
    spec = arch.build_spec(config)
    assert [(e.layer, e.cache_of) for e in spec.schedule] == [(0, None), (1, 0), (2, None), (3, 0), (4, 2)]
    assert spec.stream_copies == 2 and resolve(gc.GIF_C)[0].build_spec(resolve(gc.GIF_C)[1]).stream_copies == 1
    _, tensors = plain_gifudra.read_model(gifudra_dirs["gif_a"])
    assert "l1.mix.dkv" not in tensors and "l0.mix.dkv.norm" in tensors and "l2.norm2" not in tensors
    assert tensors["l0.hc1.mix"].shape == (2, 2) and tensors["l4.ls2"].shape == (96,) and "head" not in tensors
    _, plain = plain_gifudra.read_model(gifudra_dirs["gif_c"])
    assert "l0.hc1.in" not in plain and "l0.ls1" in plain
    bad = json.loads(json.dumps(gc.GIF_A))
    bad["layers"][1]["mixer"]["kv_from"] = 3                 # a later layer
    with pytest.raises(ConfigError):
        resolve(bad)
    bad["layers"][1]["mixer"]["kv_from"] = 0
    bad["layers"][3]["mixer"]["kv_from"] = 1                 # a layer that makes no entries itself
    with pytest.raises(ConfigError):
        resolve(bad)
    bad["layers"][3]["mixer"].update(kv_from=2)              # an owner of another latent size
    with pytest.raises(ConfigError):
        resolve(bad)


def test_readers_keep_no_pages_of_their_own(gifudra_dirs):
    """A layer that reads another layer's entries adds nothing to what a token costs the cache."""
    from liteinfer_b200.weights.loader import load_model

    model, _ = load_model(gifudra_dirs["gif_a"], torch.float32, "cpu")
    from liteinfer_b200.cache.manager import CacheManager

    cache = CacheManager(model.cache_needs(), model.schedule, 16, 8, 2, torch.float32, "cpu")
    assert sorted(len(g.holders) for g in cache.groups) == [1, 1]          # layers 0 and 2; 1, 3 and 4 hold nothing
    assert cache.bytes_per_page() == 4 * 16 * ((48 + 8) + (24 + 16))
    caches = cache.layer_caches()
    assert caches[3].kvs["latent"].k_pool.data_ptr() == caches[0].kvs["latent"].k_pool.data_ptr() and caches[3].read_only
    assert caches[4].kvs["latent"].k_pool.data_ptr() == caches[2].kvs["latent"].k_pool.data_ptr()
    assert caches[0].kvs["latent"].v_pool.numel() == 0                     # the entries are keys and values at once


@pytest.mark.parametrize("name,lengths", [("gif_a", (1, 7, 61, 90)), ("gif_b", (2, 30, 45)), ("gif_c", (5, 52, 80, 18, 70)),
                                           ("gif_d", (3, 150, 97, 130))])
def test_all_cuts_match_plain_on_cpu(cpu_kernels, gifudra_dirs, name, lengths):
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = gc.ALL[name]
    requests = {f"r{i}": gc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = expected_logits(gifudra_dirs[name], requests)
    trace = full_trace(requests)
    assert trace.max_live <= 4
    runner = build_runner(gifudra_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < gc.FLOAT32_TOLERANCE[name], f"worst difference {worst} at step {where}"
    assert not runner.cache.live_requests
    for group in runner.cache.groups:
        assert group.allocator.num_held == 0


def test_layers_one_by_one_against_plain_on_cpu(cpu_kernels, gifudra_dirs):
    """The residual (the sum of the streams) after every layer: which layer differs first, if one does."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("gif_a", "gif_b", "gif_c"):
        config, tensors = plain_gifudra.read_model(gifudra_dirs[name])
        tokens = gc.prompt(config["vocab"], 37, 3)
        want: list = []
        plain_gifudra.forward(config, tensors, tokens, want)
        runner = build_runner(gifudra_dirs[name], torch.float32, "cpu", 8, 8, 2)
        runner.cache.reserve(["a"], [37])
        context = runner.build_context([StepEntry("a", tokens, [36])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(config["layers"])
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.double() - plain).abs().max()) < 1e-4, f"{name}: layer {stop}"


def test_greedy_generation_through_the_engine(cpu_kernels, gifudra_dirs):
    """`LLM.generate` (scheduler, sampler, engine loop) on a Gifudra folder picks the plain implementation's tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_gifudra.read_model(gifudra_dirs["gif_a"])
    prompts = [gc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9)]
    llm = LLM(str(gifudra_dirs["gif_a"]), dtype="float32", device="cpu", block_size=16, num_gpu_blocks=32, max_num_seqs=2,
              max_model_len=64, max_num_batched_tokens=16, enable_cuda_graphs=False)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain_gifudra.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]


def test_plain_pieces_agree_with_their_definitions():
    """The plain implementation's own mechanisms on inputs where the answer is known."""
    torch.manual_seed(0)
    # One stream, read 1, mix 1, write 1 is the ordinary residual sum.
    x, y = torch.randn(1, 5, 7, dtype=torch.float64), torch.randn(5, 7, dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.equal(plain_gifudra.streams_read(x, one), x[0])
    assert torch.allclose(plain_gifudra.streams_write(x, one[None], one, y)[0], x[0] + y)
    # The mixing matrix is indexed [from, to]: a matrix that only feeds stream 0 into stream 1.
    two = torch.randn(2, 3, 4, dtype=torch.float64)
    mix = torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=torch.float64)
    moved = plain_gifudra.streams_write(two, mix, torch.zeros(2, dtype=torch.float64), torch.zeros(3, 4, dtype=torch.float64))
    assert torch.equal(moved[1], two[0]) and not moved[0].any()
    # A sink far above every score takes all the weight; far below, none.
    q, k, v = (torch.randn(2, 6, 8, dtype=torch.float64) for _ in range(3))
    none = plain_gifudra.sink_softmax_attention(q, k, v, 0.3, None)
    low = plain_gifudra.sink_softmax_attention(q, k, v, 0.3, torch.full((2,), -80.0, dtype=torch.float64))
    high = plain_gifudra.sink_softmax_attention(q, k, v, 0.3, torch.full((2,), 80.0, dtype=torch.float64))
    assert torch.allclose(none, low) and float(high.abs().max()) < 1e-20
    assert torch.allclose(none[:, 0], v[:, 0])               # the first token sees only itself
    # The rotation turns pairs (i, i + dims / 2) and leaves the rest; position 0 changes nothing.
    z = torch.randn(3, 2, 10, dtype=torch.float64)
    turned = plain_gifudra.rotate_half_split(z, torch.tensor([0, 1, 5]), 6, 100.0)
    assert torch.equal(turned[0], z[0]) and torch.equal(turned[..., 6:], z[..., 6:])
    assert torch.allclose(turned[1, :, 0], z[1, :, 0] * torch.cos(torch.tensor(1.0, dtype=torch.float64))
                          - z[1, :, 3] * torch.sin(torch.tensor(1.0, dtype=torch.float64)))
    assert torch.allclose(turned[..., :6].pow(2).sum(-1), z[..., :6].pow(2).sum(-1))
