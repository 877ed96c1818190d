"""Gifudra's kernels each against the plain torch function of the same name (`torch_kernels.py`) and against the
mechanisms of `plain_gifudra.py`, and the whole model through `bin/trace_run` in float32 and bfloat16."""

from __future__ import annotations

import pytest
import torch

import gifudra_configs as gc
import plain_gifudra
import replay_harness as rh
import torch_kernels as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2 ** -6, atol=2 ** -6)


def _randn(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ residual streams
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("copies", [1, 3])
def test_embedding_streams(dtype, copies):
    from liteinfer_b200 import ops

    table = _randn(50, 72, dtype=dtype)
    ids = _ints([3, 49, 0, 17, 50, -1])
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops.embedding_streams(ids, table, torch.empty(6, copies * 72, device=DEV), 3.7, flag)
    want = table[ids[:4].long()].float() * 3.7
    for s in range(copies):
        assert torch.equal(out[:4, s * 72:(s + 1) * 72], want)
    assert not out[4:].any() and int(flag) == 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,S", [(48, 1), (72, 2), (257, 3), (2048, 4), (5000, 8)])
def test_stream_rmsnorm_rewrite_read_and_rows(dtype, width, S):
    from liteinfer_b200 import ops

    T = 7
    x = _randn(T, S * width, seed=1, scale=3.0) + 0.5
    y = _randn(T, width, seed=2, scale=0.3, dtype=dtype)
    weight, gain = 1 + 0.2 * _randn(width, seed=3), 0.5 + torch.rand(width, device=DEV)
    read, write, mix = _randn(S, seed=4), 1 + 0.3 * _randn(S, seed=5), torch.eye(S, device=DEV) + 0.2 * _randn(S, S, seed=6)
    update = ops.StreamUpdate(y, gain, write, mix)
    # Against the plain mechanisms in 64-bit: the rewrite, the read, the norm.
    streams = x.view(T, S, width).transpose(0, 1).double()
    new = plain_gifudra.streams_write(streams, mix.double(), write.double(), gain.double() * y.double())
    normed = plain_gifudra.rms_norm(plain_gifudra.streams_read(new, read.double()), weight.double(), 1e-5) * 1.7
    got_x, out = x.clone(), torch.empty(T, width, dtype=dtype, device=DEV)
    ops.stream_rmsnorm(got_x, weight, 1e-5, out, read=read, update=update, out_scale=1.7)
    torch.testing.assert_close(got_x.view(T, S, width).transpose(0, 1).double(), new, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(out.double(), normed, rtol=_tol(dtype)["rtol"], atol=_tol(dtype)["atol"])
    # Against the stand-in: no rewrite pending; the plain sum of the streams; gathered rows leave the streams alone.
    for kwargs in (dict(read=read), dict(read=None), dict(read=None, update=update, rows=_ints([6, 0, 3])),
                   dict(read=read, update=ops.StreamUpdate(y, None, write, mix))):
        n = 3 if "rows" in kwargs else T
        a, b = x.clone(), x.clone()
        got = ops.stream_rmsnorm(a, weight, 1e-5, torch.empty(n, width, dtype=dtype, device=DEV), **kwargs)
        want = ref.stream_rmsnorm(b, weight, 1e-5, torch.empty(n, width, dtype=dtype, device=DEV), **kwargs)
        torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
        if "rows" in kwargs or "update" not in kwargs:
            assert torch.equal(a, x)
    # The rewrite alone (no norm behind it).
    a, b = x.clone(), x.clone()
    ops.stream_rmsnorm(a, None, 0.0, None, update=update)
    ref.stream_rmsnorm(b, None, 0.0, None, update=update)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)


def test_streams_stay_32_bit():
    """A sublayer output far below the streams' bfloat16 spacing still arrives."""
    from liteinfer_b200 import ops

    x = torch.full((2, 2 * 64), 100.0, device=DEV)
    y = _randn(2, 64, seed=1, dtype=torch.bfloat16) * 0.01
    one, eye = torch.ones(2, device=DEV), torch.eye(2, device=DEV)
    ops.stream_rmsnorm(x, None, 0.0, None, update=ops.StreamUpdate(y, None, one, eye))
    assert torch.equal(x[:, :64], 100.0 + y.float()) and torch.equal(x[:, 64:], 100.0 + y.float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_squared_relu_and_gate(dtype):
    from liteinfer_b200 import ops

    x = _randn(5, 203, dtype=dtype)
    got = ops.activation(x.clone(), torch.empty_like(x), "relu_squared")
    torch.testing.assert_close(got.float(), torch.relu(x.float()) ** 2, **_tol(dtype))
    same = x.clone()
    ops.activation(same, same, "relu_squared")
    assert torch.equal(same, got)
    v, wide = _randn(3, 9, 20, seed=1, dtype=dtype), _randn(9, 100, seed=2, dtype=dtype)
    gate = wide[:, 17:77]
    got = ops.gate_heads(v, gate, torch.empty(9, 60, dtype=dtype, device=DEV))
    want = v.float().transpose(0, 1).reshape(9, 60) * torch.sigmoid(gate.float())
    torch.testing.assert_close(got.float(), want, **_tol(dtype))
    plain = ops.gate_heads(v, None, torch.empty(9, 60, dtype=dtype, device=DEV))
    assert torch.equal(plain, v.transpose(0, 1).reshape(9, 60))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 264, 96), (5, 4096, 512), (8, 200, 1024), (12, 328, 96), (16, 8192, 256), (40, 264, 96)])
@pytest.mark.parametrize("name", ["relu_squared", "silu", "gelu_tanh"])
def test_linear_with_activation(dtype, M, N, K, name):
    """The product with the activation on its way out (a few rows of x: the weight-streaming kernels; more: the
    product, then the elementwise kernel) equals the two steps apart, and the plain formula."""
    from liteinfer_b200 import ops

    x, w = _randn(M, K, seed=1, dtype=dtype), _randn(N, K, seed=2, scale=0.1, dtype=dtype)
    got = ops.linear(x, w, None, activation=name)
    apart = ops.linear(x, w, None)
    product = apart.float().clone()
    ops.activation(apart, apart, name)
    torch.testing.assert_close(got.float(), apart.float(), rtol=2 ** -7 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)
    want = {"relu_squared": lambda v: torch.relu(v) ** 2, "silu": lambda v: v * torch.sigmoid(v),
            "gelu_tanh": lambda v: torch.nn.functional.gelu(v, approximate="tanh")}[name](product)
    torch.testing.assert_close(got.float(), want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,M,N,K", [(3, 5, 40, 12), (1, 70, 33, 100), (6, 1, 24, 48), (4, 130, 64, 32)])
def test_batched_linear_on_column_slices(dtype, B, M, N, K):
    from liteinfer_b200 import ops

    wide = _randn(M, B * (K + 5), seed=1, dtype=dtype)
    x = wide.view(M, B, K + 5)[:, :, :K].transpose(0, 1)                # a head's first K columns of a projection
    w = _randn(B, N, K, seed=2, dtype=dtype)
    got = ops.batched_linear(x, w, torch.empty(B, M, N, dtype=dtype, device=DEV))
    want = torch.einsum("bmk,bnk->bmn", x.double(), w.double())
    torch.testing.assert_close(got.double(), want, rtol=_tol(dtype)["rtol"], atol=_tol(dtype)["atol"] * K ** 0.5)


# ------------------------------------------------------------------ latent attention
def _batch(query_lens, context_lens, page_size, pages, seed=0):
    """Block tables over shuffled pages, and the step's index arrays, for sequences that bring `query_lens` tokens
    and then hold `context_lens`."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(pages, generator=g).tolist()
    width = max(-(-c // page_size) for c in context_lens)
    table, positions, seq_of, qsl = [], [], [], [0]
    for i, (n, c) in enumerate(zip(query_lens, context_lens)):
        need = -(-c // page_size)
        table.append([order.pop() for _ in range(need)] + [-1] * (width - need))
        positions += list(range(c - n, c))
        seq_of += [i] * n
        qsl.append(qsl[-1] + n)
    return _ints(table), _ints(positions), _ints(seq_of), _ints(qsl), _ints(list(context_lens))


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_prep_writes_entries_and_skips_padding(dtype):
    from liteinfer_b200 import ops

    q_rank, c, r, dims, page = 24, 40, 10, 6, 4
    table, positions, seq_of, _, _ = _batch([5, 1, 3], [9, 14, 3], page, 12)
    seq_of[6] = -1                                                       # a row of padding in the middle
    proj = _randn(9, 100, seed=1, dtype=dtype)
    wq, wkv = 1 + 0.2 * _randn(q_rank, seed=2), 1 + 0.2 * _randn(c, seed=3)
    inv_freq = (100.0 ** (-torch.arange(dims // 2, dtype=torch.float64) * 2 / dims)).float().to(DEV)
    pools = [torch.full((12, 1, page, c + r), 7.0, dtype=dtype, device=DEV) for _ in range(3)]
    outs = [torch.empty(9, q_rank, dtype=dtype, device=DEV) for _ in range(3)]
    args = (0, q_rank, q_rank + 3, c, r, dims, wq, wkv, 1e-5, inv_freq, positions, seq_of, table)
    ops.latent_prep(proj, *args, pools[0], outs[0])
    ref.latent_prep(proj, *args, pools[1], outs[1])
    torch.testing.assert_close(outs[0].float(), outs[1].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0].float(), pools[1].float(), **_tol(dtype))
    untouched = (pools[1] == 7.0).all(-1)
    assert int((~untouched).sum()) == 8 and torch.equal((pools[0] == 7.0).all(-1), untouched)
    # Against the plain mechanism: the entry of sequence 1's newest token (position 13, token row 5).
    kv = proj[5:6, q_rank + 3:q_rank + 3 + c + r].double().cpu()
    latent, shared = plain_gifudra.latent_and_rotated_key(
        kv, {"dkv": torch.eye(c + r, dtype=torch.float64), "dkv.norm": wkv.double().cpu()},
        {"kv_rank": c, "rot_dim": r, "rot": {"dims": dims, "base": 100.0}}, 1e-5, torch.tensor([13]))
    entry = pools[0][int(table[1, 13 // page]), 0, 13 % page].double().cpu()
    torch.testing.assert_close(entry, torch.cat([latent[0], shared[0]]), rtol=_tol(dtype)["rtol"], atol=_tol(dtype)["atol"])
    # A layer that reads another layer's entries stores nothing, and still normalises its query latent.
    ops.latent_prep(proj, 0, q_rank, None, c, r, dims, wq, None, 1e-5, inv_freq, positions, seq_of, table, pools[2], outs[2])
    assert bool((pools[2] == 7.0).all()) and torch.equal(outs[2], outs[0])


def _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, seed):
    table, positions, seq_of, qsl, ctxl = _batch(query_lens, context_lens, page, pages, seed)
    tokens = int(qsl[-1])
    pool = _randn(pages, 1, page, c + r, seed=seed + 1, dtype=dtype)
    q_lat = _randn(heads, tokens, c, seed=seed + 2, scale=0.5, dtype=dtype)
    q_raw = _randn(tokens, heads * (d + r) + 3, seed=seed + 3, dtype=dtype)
    return table, qsl, ctxl, pool, q_lat, q_raw


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,c,r,dims,d,page", [(3, 40, 10, 6, 12, 4), (1, 24, 2, 2, 5, 8), (6, 96, 32, 32, 16, 16),
                                                   (16, 64, 32, 32, 32, 32), (9, 128, 64, 64, 8, 64), (2, 512, 64, 64, 4, 16), (2, 640, 16, 16, 4, 16)])
@pytest.mark.parametrize("sink", [True, False])
def test_latent_attention_portions_and_single_tokens(dtype, heads, c, r, dims, d, page, sink):
    from liteinfer_b200 import ops

    query_lens, context_lens = [17, 1, 2, 1, 40], [17, 70, 2 * page + 2, 1, 40 + 3 * page]
    pages = sum(-(-n // page) for n in context_lens) + 3
    table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, 5)
    inv_freq = (1000.0 ** (-torch.arange(dims // 2, dtype=torch.float64) * 2 / dims)).float().to(DEV)
    sinks = _randn(heads, seed=9) if sink else None
    got = ops.latent_attention(q_lat, q_raw, d + r, d, torch.empty_like(q_lat), pool, table, qsl, ctxl, inv_freq, sinks,
                               5, 40, heads, c, r, dims, 0.11)
    want = ref.latent_attention(q_lat, q_raw, d + r, d, torch.empty_like(q_lat), pool, table, qsl, ctxl, inv_freq, sinks,
                                5, 40, heads, c, r, dims, 0.11)
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


def _plan(query_lens, context_lens):
    from liteinfer_b200.parts.context import AttentionPlan

    decode = [i for i, n in enumerate(query_lens) if n == 1]
    prefill = [i for i, n in enumerate(query_lens) if n > 1]
    starts = [sum(query_lens[:i]) for i in range(len(query_lens))]
    return AttentionPlan(num_decode=len(decode) + 1, decode_seqs=_ints(decode + [-1]),          # one place of padding each
                         decode_tokens=_ints([starts[i] for i in decode] + [0]), num_prefill=len(prefill) + 1,
                         prefill_seqs=_ints(prefill + [-1]), max_prefill_query_len=max([query_lens[i] for i in prefill], default=0),
                         max_decode_context_len=max([context_lens[i] for i in decode], default=0))


@pytest.mark.parametrize("heads,c,r,page", [(16, 64, 32, 16), (8, 128, 32, 32), (20, 128, 64, 16), (5, 256, 64, 64),
                                            (16, 512, 64, 16), (33, 512, 64, 32)])
@pytest.mark.parametrize("sink", [True, False])
def test_latent_attention_on_tensor_cores_with_a_plan(heads, c, r, page, sink):
    """Sizes the tensor-core kernel takes: portions (four queries a block) beside single tokens whose keys several
    blocks share, places of padding in both lists, against the plain twin and against the SIMT kernel."""
    from liteinfer_b200 import ops

    dtype, d = torch.bfloat16, 8
    assert ops.latent_mma_supports(dtype, c, r, r)
    query_lens, context_lens = [1, 37, 1, 6, 1, 130], [900, 37, 1, 70, 65, 130 + 2 * page + 3]
    pages = sum(-(-n // page) for n in context_lens) + 3
    table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, 7)
    inv_freq = (1000.0 ** (-torch.arange(r // 2, dtype=torch.float64) * 2 / r)).float().to(DEV)
    sinks = _randn(heads, seed=9) if sink else None
    common = (q_lat, q_raw, d + r, d)
    rest = (pool, table, qsl, ctxl, inv_freq, sinks, 6, 130, heads, c, r, r, 0.09)
    want = ref.latent_attention(*common, torch.empty_like(q_lat), *rest)
    planned = ops.latent_attention(*common, torch.zeros_like(q_lat), *rest, plan=_plan(query_lens, context_lens))
    unplanned = ops.latent_attention(*common, torch.zeros_like(q_lat), *rest)
    torch.testing.assert_close(planned.float(), want.float(), **_tol(dtype))
    torch.testing.assert_close(unplanned.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("heads,c,r", [(16, 64, 32), (5, 512, 64), (20, 128, 32)])
def test_latent_attention_wide_batch_of_single_tokens(heads, c, r):
    """More than sixteen single-token sequences at once (the launch then runs two blocks per SM, rounds of 32 keys):
    contexts of one token, on both sides of a round's and a stage's edge, and long enough for several splits."""
    from liteinfer_b200 import ops

    dtype, d, page = torch.bfloat16, 8, 16
    context_lens = [1, 2, 31, 32, 33, 63, 64, 65, 96, 97, 100, 257, 500, 511, 512, 513, 700, 1000, 1024, 1500]
    query_lens = [1] * len(context_lens)
    pages = sum(-(-n // page) for n in context_lens) + 3
    table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, query_lens, context_lens, page, pages, 3)
    inv_freq = (1000.0 ** (-torch.arange(r // 2, dtype=torch.float64) * 2 / r)).float().to(DEV)
    sinks = _randn(heads, seed=9)
    common = (q_lat, q_raw, d + r, d)
    rest = (pool, table, qsl, ctxl, inv_freq, sinks, len(context_lens), 1, heads, c, r, r, 0.09)
    want = ref.latent_attention(*common, torch.empty_like(q_lat), *rest)
    got = ops.latent_attention(*common, torch.zeros_like(q_lat), *rest, plan=_plan(query_lens, context_lens))
    torch.testing.assert_close(got.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype,c,r", [(torch.float32, 48, 8), (torch.bfloat16, 48, 8), (torch.bfloat16, 64, 32)])
@pytest.mark.parametrize("decode", [False, True])
def test_latent_attention_one_key_stands_out(dtype, c, r, decode):
    """One key's score is lifted far above all others, wherever it lies: at position 0, on both sides of page
    borders, hundreds of tokens back, the query's own position.  The query then reads that entry's latent.  A key
    just behind the query's position is never seen, whatever it holds; a sink as large as the lifted score halves
    the result."""
    from liteinfer_b200 import ops

    heads, d, page, ctx = 3, 6, 16, 700
    n = 1 if decode else 9
    plan = _plan([n], [ctx]) if c == 64 else None          # the tensor-core kernel: split keys for the single token
    pages = -(-ctx // page) + 2
    inv_freq = (1000.0 ** (-torch.arange(r // 2, dtype=torch.float64) * 2 / r)).float().to(DEV)
    qpos = ctx - 1
    for target in (0, 15, 16, 17, 255, 256, 400, qpos - 1, qpos, qpos + 1):
        table, qsl, ctxl, pool, q_lat, q_raw = _attention_inputs(dtype, heads, c, r, d, [n], [ctx], page, pages, 11)
        pool.mul_(0.05)
        entry_page, slot = int(table[0, target // page]) if target < ctx else int(table[0, (ctx - 1) // page]), target % page
        if target >= ctx:            # the slot right behind the sequence's newest token (same page, or a free one)
            if target // page < table.shape[1] and int(table[0, target // page]) >= 0:
                entry_page = int(table[0, target // page])
            else:
                continue
        lifted = torch.zeros(c + r, device=DEV)
        lifted[:c] = _randn(c, seed=3)
        pool[entry_page, 0, slot] = lifted.to(dtype)
        q_lat[:, -1] = (lifted[:c] * 3.0).to(dtype)                   # the last query looks for exactly that latent
        sink = torch.full((heads,), -50.0, device=DEV)
        out = ops.latent_attention(q_lat, q_raw, d + r, d, torch.empty_like(q_lat), pool, table, qsl, ctxl, inv_freq,
                                   sink, 1, n, heads, c, r, r, 1.0, plan=plan)
        found = pool[entry_page, 0, slot, :c].float()
        if target <= qpos:
            torch.testing.assert_close(out[:, -1].float(), found.expand(heads, c), rtol=2e-2, atol=2e-2)
            score = float((q_lat[0, -1].float() * found).sum())
            sink = torch.full((heads,), score, device=DEV)
            halved = ops.latent_attention(q_lat, q_raw, d + r, d, torch.empty_like(q_lat), pool, table, qsl, ctxl,
                                          inv_freq, sink, 1, n, heads, c, r, r, 1.0, plan=plan)
            torch.testing.assert_close(halved[:, -1].float(), 0.5 * found.expand(heads, c), rtol=3e-2, atol=3e-2)
        else:
            assert float(out[:, -1].float().abs().max()) < 0.2      # an average of small entries: the lifted one is not in it


# ------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module")
def gifudra_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("gifudra")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in gc.ALL.items()}


def _expected(model_dir, requests):
    config, tensors = plain_gifudra.read_model(model_dir)
    return {name: plain_gifudra.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


@pytest.mark.parametrize("name,lengths", [("gif_a", (1, 7, 61, 90)), ("gif_b", (2, 30, 45)), ("gif_c", (5, 52, 80, 18, 70)),
                                           ("gif_d", (3, 150, 97, 260))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_all_cuts(gifudra_dirs, tmp_path, name, lengths, dtype):
    config, _, page = gc.ALL[name]
    requests = {f"r{i}": gc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = _expected(gifudra_dirs[name], requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda r: len(requests[r]))
    for i, token in enumerate(requests[longest]):            # every token a step of its own, from the first one on
        trace.add([(f"o-{longest}", [token], [0])], end=[f"o-{longest}"] if i == len(requests[longest]) - 1 else [])
    results = rh.run_program(trace, gifudra_dirs[name], dtype, tmp_path / "out", config["vocab"], page_size=page)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    limit = 2 * gc.FLOAT32_TOLERANCE[name] if dtype == "float32" else gc.BFLOAT16_TOLERANCE[name]
    assert worst < limit, f"worst difference {worst} at step {where}"


def test_layers_one_by_one_against_plain(gifudra_dirs):
    """The sum of the residual streams after every layer (32-bit engine) equals the plain implementation's."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    for name in ("gif_a", "gif_c"):
        config, tensors = plain_gifudra.read_model(gifudra_dirs[name])
        tokens = gc.prompt(config["vocab"], 45, 3)
        want: list = []
        plain_gifudra.forward(config, tensors, tokens, want)
        runner = build_runner(gifudra_dirs[name], torch.float32, DEV, 16, 8, 2)
        runner.cache.reserve(["a"], [45])
        context = runner.build_context([StepEntry("a", tokens, [44])])
        context.layer_trace = []
        runner.model.forward(context, runner.layer_caches)
        assert len(context.layer_trace) == len(want)
        for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
            assert float((got.cpu().double() - plain).abs().max()) < 2e-4, f"{name}: layer {stop}"


def test_greedy_generation_through_the_engine_on_gpu(gifudra_dirs):
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_gifudra.read_model(gifudra_dirs["gif_b"])
    prompts = [gc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9, 14, 2)]
    with LLM(str(gifudra_dirs["gif_b"]), dtype="float32", block_size=4, num_gpu_blocks=64, max_num_seqs=3,
             max_model_len=64, max_num_batched_tokens=16) as llm:
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(12):
            tokens.append(int(plain_gifudra.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]
