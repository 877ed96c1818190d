"""Kegizen through the framework's step function, cache manager and engine on a CPU (stand-in kernels), against the
plain implementation of `plain_kegizen.py`: every way of cutting the same requests gives the same logits."""

from __future__ import annotations

import json

import pytest
import torch

import kegizen_configs as kc
import plain_kegizen
import replay_harness as rh


@pytest.fixture(scope="module")
def kegizen_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("kegizen")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items()}


def expected_logits(model_dir, requests):
    config, tensors = plain_kegizen.read_model(model_dir)
    return {name: plain_kegizen.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


def one_by_one(trace, requests, tag="o"):
    """Every token a step of its own, from the first one on (the first tokens of a sequence, and long decoding)."""
    for name, tokens in requests.items():
        rid = f"{tag}-{name}"
        for i, token in enumerate(tokens):
            trace.add([(rid, [token], [0])], end=[rid] if i == len(tokens) - 1 else [])


def full_trace(requests):
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda name: len(requests[name]))
    one_by_one(trace, {longest: requests[longest]})
    return trace


def test_config_round_trip_and_names(kegizen_dirs):
    from liteinfer_b200.config.kegizen_config import KegizenConfig
    from liteinfer_b200.config.registry import resolve

    for name, (raw, _, _) in kc.ALL.items():
        arch, config = resolve(raw)
        assert arch.name == "Kegizen" and KegizenConfig.from_dict(config.to_dict()) == config
        written = json.loads((kegizen_dirs[name] / "config.json").read_text())
        assert KegizenConfig.from_dict(written) == config
    arch, config = resolve(kc.KEG_A)
    spec = arch.build_spec(config)
    assert [(e.layer, e.reenter) for e in spec.schedule] == [(0, True), (1, False), (0, True), (1, False), (2, False), (3, False)]
    _, tensors = plain_kegizen.read_model(kegizen_dirs["keg_a"])
    assert "l3.norm2" not in tensors and "l0.mix.q.norm" in tensors and "l1.mix.q.conv" in tensors and "loop.in" in tensors
    assert "loop.in" not in plain_kegizen.read_model(kegizen_dirs["keg_b"])[1]


@pytest.mark.parametrize("name,lengths", [("keg_a", (1, 7, 61, 90)), ("keg_b", (2, 30, 45)), ("keg_c", (5, 52, 80, 18, 70)),
                                           ("keg_d", (3, 150, 97, 260))])
def test_all_cuts_match_plain_on_cpu(cpu_kernels, kegizen_dirs, name, lengths):
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = expected_logits(kegizen_dirs[name], requests)
    trace = full_trace(requests)
    assert trace.max_live <= 4
    runner = build_runner(kegizen_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = rh.run_in_process(runner, trace)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    assert worst < kc.FLOAT32_TOLERANCE[name], f"worst difference {worst} at step {where}"
    assert not runner.cache.live_requests
    for group in runner.cache.groups:
        assert group.allocator.num_held == 0


def test_window_pages_are_given_back_but_kept_tokens_stay(cpu_kernels, kegizen_dirs):
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, _, page = kc.ALL["keg_c"]                    # window 33, 17 kept tokens, pages of 8
    runner = build_runner(kegizen_dirs["keg_c"], torch.float32, "cpu", page, 40, 4)
    tokens = kc.prompt(config["vocab"], 120, 5)
    runner.step([StepEntry("a", tokens[:100], [])])
    windowed = [g for g in runner.cache.groups if g.need.window is not None]
    assert len(windowed) == 1 and windowed[0].need.keep_first == 17
    table = windowed[0].tables["a"]
    kept, first = 3, (100 - 33 + 1) // page               # ceil(17 / 8) leading blocks stay; the window starts in block 8
    assert all(p >= 0 for p in table[:kept]) and all(p < 0 for p in table[kept:first]) and all(p >= 0 for p in table[first:])
    full = [g for g in runner.cache.groups if g.need.window is None]
    assert all(p >= 0 for p in full[0].tables["a"])
    expected = expected_logits(kegizen_dirs["keg_c"], {"a": tokens})["a"]
    got = runner.step([StepEntry("a", tokens[100:], list(range(20)))])
    assert float((got - expected[100:]).abs().max()) < 5e-5
    runner.release("a")
    runner.cache.check_invariants()
    assert all(g.allocator.num_held == 0 for g in runner.cache.groups)


def test_greedy_generation_through_the_engine(cpu_kernels, kegizen_dirs):
    """`LLM.generate` (scheduler, sampler, engine loop) on a Kegizen folder picks the plain implementation's tokens."""
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_kegizen.read_model(kegizen_dirs["keg_a"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9)]
    llm = LLM(str(kegizen_dirs["keg_a"]), dtype="float32", device="cpu", block_size=16, num_gpu_blocks=32, max_num_seqs=2,
              max_model_len=64, max_num_batched_tokens=16, enable_cuda_graphs=False)
    outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(6):
            tokens.append(int(plain_kegizen.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]


def test_cache_manager_kept_tokens_and_value_size():
    """A window that keeps first tokens costs their pages on top of the window's; values of another size than keys
    get a pool of their own; such needs group apart from plain ones."""
    from liteinfer_b200.cache.manager import CacheManager
    from liteinfer_b200.parts.context import KVNeed
    from liteinfer_b200.parts.spec import ScheduleEntry

    needs = [(KVNeed(2, 16, 24, v_head_dim=40, keep_first=9),), (KVNeed(2, 16, 24),), (KVNeed(2, 16, 24, v_head_dim=40, keep_first=9),)]
    m = CacheManager(needs, tuple(ScheduleEntry(i) for i in range(3)), 8, 32, 4, torch.float32, "cpu")
    assert len(m.groups) == 2
    kept, plain = m.groups
    assert kept.pool.shape == (2, 1, 32, 2, 8, 16) and kept.v_pool.shape == (2, 32, 2, 8, 40) and plain.v_pool is None
    caches = m.layer_caches()
    assert caches[0].kv.v_pool.shape == (32, 2, 8, 40) and caches[1].kv.v_pool.shape == (32, 2, 8, 16)
    assert caches[2].kv.k_pool.data_ptr() != caches[0].kv.k_pool.data_ptr()
    assert kept.kept_blocks == 2 and plain.kept_blocks == 0
    assert kept.pages_at(200, 1) == plain.pages_at(200, 1) + 2 and kept.pages_at(10, 10) == 2
    m.reserve(["a"], [100])
    m.commit("a", 100)
    first = (100 - 24 + 1) // 8
    assert [p >= 0 for p in kept.tables["a"]] == [True, True] + [False] * (first - 2) + [True] * (13 - first)
    assert [p >= 0 for p in plain.tables["a"]] == [False] * first + [True] * (13 - first)
    assert m.bytes_per_page() == 4 * 8 * 2 * (2 * (16 + 40) + (16 + 16))
    m.release("a")
    m.check_invariants()
    assert kept.allocator.num_held == 0 and plain.allocator.num_held == 0


def test_yarn_frequencies_are_the_plain_ones():
    from liteinfer_b200.parts.position import yarn_inverse_frequencies

    for dims, base, factor, original, fast, slow in ((16, 10000.0, 4.0, 32, 8.0, 1.0), (12, 1000.0, 8.0, 16, 4.0, 0.5),
                                                      (64, 5000.0, 3.0, 64, 16.0, 2.0), (8, 100.0, 1.5, 4096, 32.0, 1.0)):
        got, stretch = yarn_inverse_frequencies(dims, base, factor, float(original), fast, slow)
        want, want_stretch = plain_kegizen.yarn_frequencies(dims, base, {"factor": factor, "original": original,
                                                                         "fast": fast, "slow": slow})
        assert torch.equal(got, want.to(torch.float32)) and stretch == want_stretch
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        assert bool((want <= plain + 1e-12).all()) and bool((want >= plain / factor - 1e-12).all())


def test_layers_one_by_one_against_plain_on_cpu(cpu_kernels, kegizen_dirs):
    """The residual stream after every stop of the schedule: which layer differs first, if one does."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("keg_a", "keg_c"):
        config, tensors = plain_kegizen.read_model(kegizen_dirs[name])
        tokens = kc.prompt(config["vocab"], 37, 3)
        want: list = []
        plain_kegizen.forward(config, tensors, tokens, want)
        runner = build_runner(kegizen_dirs[name], torch.float32, "cpu", 8, 8, 2)
        runner.cache.reserve(["a"], [37])
        context = runner.build_context([StepEntry("a", tokens, [36])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want) == len(plain_kegizen.layer_runs(config))
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.double() - plain).abs().max()) < 1e-4, f"{name}: stop {stop}"
