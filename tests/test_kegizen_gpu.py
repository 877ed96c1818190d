"""Kegizen's kernels each against the plain torch function of the same name (`torch_kernels.py`), and the whole
model through `bin/trace_run` in float32 and bfloat16 against `plain_kegizen.py`."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import kegizen_configs as kc
import plain_kegizen
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


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                      (torch.float32, torch.float32)])
def test_convert_between_column_slices(src, dst):
    from liteinfer_b200 import ops

    wide_src, wide_dst = _randn(37, 150, dtype=src), torch.zeros(37, 200, dtype=dst, device=DEV)
    ops.convert(wide_src[:, 20:131], wide_dst[:, 7:118])
    assert torch.equal(wide_dst[:, 7:118], wide_src[:, 20:131].to(dst))
    assert not wide_dst[:, :7].any() and not wide_dst[:, 118:].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 257, 2048, 8192, 12288, 20000])
def test_layernorm_alone_with_delta_and_rows(dtype, width):
    from liteinfer_b200 import ops

    w, wd = (1 + 0.2 * _randn(width, seed=1)).to(dtype), (1 + 0.2 * _randn(width, seed=2)).to(dtype)
    x = _randn(9, width, seed=3, scale=3.0) + 1.5                      # the stream is 32-bit; a mean far from zero
    value = _randn(9, width, seed=4, scale=0.3, dtype=dtype) - 0.4
    for stream in (x, x.to(dtype)):
        out, want = torch.empty(9, width, dtype=dtype, device=DEV), torch.empty(9, width, dtype=dtype, device=DEV)
        ops.layernorm(stream.clone(), w, 1e-5, out)
        ref.layernorm(stream.clone(), w, 1e-5, want)
        torch.testing.assert_close(out.float(), want.float(), **_tol(dtype))
        delta = ops.NormedDelta(value, wd, 1e-3)
        got_stream, want_stream = stream.clone(), stream.clone()
        ops.layernorm(got_stream, w, 1e-5, out, delta=delta, write_stream=True)
        ref.layernorm(want_stream, w, 1e-5, want, delta=delta, write_stream=True)
        torch.testing.assert_close(got_stream.float(), want_stream.float(), **_tol(stream.dtype))
        torch.testing.assert_close(out.float(), want.float(), **_tol(dtype))
        rows = _ints([8, 0, 3])
        got_stream = stream.clone()
        picked = ops.layernorm(got_stream, w, 1e-5, torch.empty(3, width, dtype=dtype, device=DEV), delta=delta, rows=rows)
        assert torch.equal(got_stream, stream)                          # gathered rows leave the stream alone
        torch.testing.assert_close(picked.float(), want[[8, 0, 3]].float(), **_tol(dtype))
        added = stream.clone()
        ops.layernorm_add(added, value, wd, 1e-3)
        torch.testing.assert_close(added.float(), want_stream.float(), **_tol(stream.dtype))


def test_layernorm_keeps_the_stream_32_bit():
    """A delta far below the stream's bfloat16 spacing still arrives in a 32-bit stream."""
    from liteinfer_b200 import ops

    stream = torch.full((2, 64), 100.0, device=DEV)
    value = _randn(2, 64, seed=1, dtype=torch.bfloat16)
    weight = torch.full((64,), 0.01, dtype=torch.bfloat16, device=DEV)
    before = stream.clone()
    ops.layernorm_add(stream, value, weight, 1e-5)
    moved = (stream - before).abs()
    assert float(moved.max()) < 0.05 and float(moved.mean()) > 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_rmsnorm_on_two_slices(dtype):
    from liteinfer_b200 import ops

    qkv = _randn(11, 96 + 40 + 30, seed=1, dtype=dtype)
    wq, wk = (1 + 0.3 * _randn(96, seed=2)).to(dtype), (1 + 0.3 * _randn(40, seed=3)).to(dtype)
    want = qkv.clone()
    ref.qk_projection_rmsnorm_(want[:, :96], wq, want[:, 96:136], wk, 1e-4)
    ops.qk_projection_rmsnorm_(qkv[:, :96], wq, qkv[:, 96:136], wk, 1e-4)
    torch.testing.assert_close(qkv.float(), want.float(), **_tol(dtype))
    assert torch.equal(qkv[:, 136:], want[:, 136:])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,size", [(3, 20), (2, 128), (5, 1)])
def test_gated_rmsnorm(dtype, heads, size):
    from liteinfer_b200 import ops

    x = _randn(13, heads * size, seed=1, scale=2.0)
    wide = _randn(13, heads * size + 9, seed=2, dtype=dtype)
    weight = 1 + 0.2 * _randn(size, seed=3)
    out, want = (torch.empty(13, heads * size, dtype=dtype, device=DEV) for _ in range(2))
    ops.gated_rmsnorm(x, wide[:, 4:4 + heads * size], weight, 1e-5, out, heads)
    ref.gated_rmsnorm(x, wide[:, 4:4 + heads * size], weight, 1e-5, want, heads)
    torch.testing.assert_close(out.float(), want.float(), **_tol(dtype))


def _cut(lengths, cuts):
    """query_start_loc of one step per entry of `cuts`: every sequence brings its next cuts[k][i] tokens."""
    steps, at = [], [0] * len(lengths)
    for counts in cuts:
        steps.append([(a, min(a + c, n)) for a, c, n in zip(at, counts, lengths)])
        at = [b for _, b in steps[-1]]
    assert at == list(lengths)
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_conv_in_portions_equals_whole(dtype, taps):
    """Portions of 1, 2 and more tokens (shorter than the tail too) give what the whole sequence gives, through
    slots that are not in order; the twin agrees."""
    from liteinfer_b200 import ops

    channels, lengths, slots = (72 if taps != 2 else 70), (23, 9), _ints([5, 2])       # 72: the vector kernels' sizes
    x = [_randn(n, channels + 8, seed=10 + i, dtype=dtype) for i, n in enumerate(lengths)]
    w = _randn(taps, channels, seed=3, scale=0.5, dtype=dtype)

    def run(impl, cuts):
        tail = torch.zeros(8, taps - 1, channels, dtype=dtype, device=DEV)
        outs = [[] for _ in lengths]
        for step in _cut(lengths, cuts):
            rows = torch.cat([x[i][a:b] for i, (a, b) in enumerate(step)])[:, 8:8 + channels]
            counts = [b - a for a, b in step]
            qsl = _ints([0, counts[0], counts[0] + counts[1]])
            seq_of = _ints([0] * counts[0] + [1] * counts[1])
            out = torch.empty(rows.shape[0], channels, dtype=dtype, device=DEV)
            if max(counts) == 1 and min(counts) == 1:      # the step function's call: one launch where the kernel can
                impl.short_conv_step(rows, w, tail, seq_of, qsl, slots, 2, out, "silu", single_tokens=True)
            else:
                impl.short_conv(rows, w, tail, seq_of, qsl, slots, out, "silu")
                impl.short_conv_update(rows, tail, qsl, slots, 2)
            outs[0].append(out[:counts[0]]); outs[1].append(out[counts[0]:])
        return [torch.cat(o) for o in outs], tail

    whole, tail_whole = run(ops, [lengths])
    cuts = [(1, 2), (2, 1), (1, 1), (1, 1), (1, 1), (3, 1), (2, 1), (12, 1)]
    parts, tail_parts = run(ops, cuts)
    want, tail_want = run(ref, cuts)
    for a, b, c in zip(whole, parts, want):
        assert torch.equal(a, b)
        torch.testing.assert_close(a.float(), c.float(), **_tol(dtype))
    assert torch.equal(tail_whole, tail_parts) and torch.equal(tail_parts, tail_want)
    assert not tail_parts[[0, 1, 3, 4, 6, 7]].any()


def test_short_conv_skips_padding():
    from liteinfer_b200 import ops

    x, w = _randn(6, 16, seed=1), _randn(3, 16, seed=2)
    tail = _randn(4, 2, 16, seed=3)
    before = tail.clone()
    out = torch.full((6, 16), 7.0, device=DEV)
    qsl, slots = _ints([0, 0, 4, 4]), _ints([1, 2, 1])         # sequences 0 and 2 bring nothing (and name live slots)
    ops.short_conv(x, w, tail, _ints([1, 1, 1, 1, -1, -1]), qsl, slots, out, "silu")
    ops.short_conv_update(x, tail, qsl, slots, 3)
    assert not out[4:].any() and torch.equal(tail[[0, 1, 3]], before[[0, 1, 3]])
    assert torch.equal(tail[2], x[2:4])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 24, 16), (3, 3, 48, 20), (2, 1, 128, 40), (6, 2, 8, 72), (1, 1, 200, 33),
                                                      (2, 2, 64, 32), (1, 1, 256, 8), (2, 1, 32, 36), (2, 1, 128, 64),
                                                      (1, 1, 256, 32), (4, 2, 32, 32)])
def test_gated_delta_rule_in_portions_equals_whole(dtype, heads, kv_heads, dim, vdim):
    from liteinfer_b200 import ops

    lengths, slots = (19, 6), _ints([3, 0])
    width = 2 * kv_heads * dim + heads * vdim
    qkv = [_randn(n, width, seed=20 + i, dtype=dtype) for i, n in enumerate(lengths)]
    ab = [_randn(n, 2 * heads + 3, seed=30 + i, scale=2.0, dtype=dtype) for i, n in enumerate(lengths)]
    a_log, dt_bias = torch.log(1 + 3 * torch.rand(heads, device=DEV)), _randn(heads, seed=5)

    def run(impl, cuts):
        state = torch.zeros(4, heads, vdim, dim, device=DEV)
        outs = [[] for _ in lengths]
        for step in _cut(lengths, cuts):
            rows = torch.cat([qkv[i][a:b] for i, (a, b) in enumerate(step)])
            gates = torch.cat([ab[i][a:b] for i, (a, b) in enumerate(step)])[:, 1:1 + 2 * heads]
            counts = [b - a for a, b in step]
            qsl = _ints([0, counts[0], counts[0] + counts[1]])
            out = torch.zeros(rows.shape[0], heads * vdim, device=DEV)
            impl.gated_delta_rule(rows, gates, a_log, dt_bias, state, qsl, slots, 2, heads, kv_heads, dim, vdim, out,
                                  max(counts))
            outs[0].append(out[:counts[0]]); outs[1].append(out[counts[0]:])
        return [torch.cat(o) for o in outs], state

    whole, state_whole = run(ops, [lengths])
    cuts = [(2, 1), (1, 1), (1, 0), (1, 1), (6, 0), (8, 3)]      # steps of single tokens take the kernel's other variant
    parts, state_parts = run(ops, cuts)
    want, state_want = run(ref, cuts)
    for a, b, c in zip(whole, parts, want):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)            # the same chain however it is cut
        torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(state_whole, state_parts, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(state_parts, state_want, rtol=1e-4, atol=1e-5)
    assert not state_parts[[1, 2]].any()


def test_gated_delta_rule_recalls_a_far_key():
    """One key written 300 tokens back with decay 1 is read out exactly; with a decay below 1 it has faded."""
    from liteinfer_b200 import ops

    dim, vdim, n = 32, 16, 301
    qkv = torch.zeros(n, 2 * dim + vdim, device=DEV)
    for t in range(n):
        qkv[t, dim + (t % (dim - 1)) + 1] = 1.0                # keys along the axes 1..dim-1, never axis 0 again
    qkv[0, dim:2 * dim] = 0; qkv[0, dim] = 1.0                 # token 0 writes along axis 0 ...
    qkv[0, 2 * dim:] = torch.arange(1, vdim + 1, device=DEV)   # ... these values
    qkv[-1, 0] = 1.0                                           # the last query asks for axis 0
    ab = torch.zeros(n, 2, device=DEV)
    ab[:, 0] = 30.0                                            # beta = 1
    for decay_raw, factor in ((-60.0, 1.0), (0.0, None)):
        ab[:, 1] = decay_raw
        state = torch.zeros(1, 1, vdim, dim, device=DEV)
        out = torch.zeros(n, vdim, device=DEV)
        ops.gated_delta_rule(qkv, ab, torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), state, _ints([0, n]),
                             _ints([0]), 1, 1, 1, dim, vdim, out)
        want = torch.arange(1, vdim + 1, device=DEV) * dim ** -0.5
        if factor is not None:
            torch.testing.assert_close(out[-1], want * factor, rtol=1e-5, atol=1e-6)
        else:
            assert float(out[-1].abs().max()) < 1e-20


# ------------------------------------------------------------------ attention options
def _paged_case(lengths, queries, kv_heads, head_dim, v_dim, page, dtype, seed=0):
    """Sequences of `lengths` tokens whose last `queries` are this step's; pages dealt out in a shuffled order."""
    g = torch.Generator().manual_seed(seed)
    pages_of = [-(-n // page) for n in lengths]
    order = torch.randperm(sum(pages_of) + 3, generator=g).tolist()
    table = torch.full((len(lengths), max(pages_of)), -1, dtype=torch.int32)
    for i, n in enumerate(pages_of):
        table[i, :n] = torch.tensor([order.pop() for _ in range(n)], dtype=torch.int32)
    k_pool = _randn(sum(pages_of) + 3, kv_heads, page, head_dim, seed=seed + 1, dtype=dtype)
    v_pool = _randn(sum(pages_of) + 3, kv_heads, page, v_dim, seed=seed + 2, dtype=dtype)
    qsl = [0]
    for n in queries:
        qsl.append(qsl[-1] + n)
    return SimpleNamespace(table=table.to(DEV), k_pool=k_pool, v_pool=v_pool, qsl=_ints(qsl), ctx=_ints(list(lengths)),
                           tokens=qsl[-1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep_first,softcap,head_dim,v_dim", [
    (20, 3, 10.0, 32, 24), (9, 0, 5.0, 40, 48), (33, 17, 0.0, 16, 16), (0, 0, 2.0, 64, 80), (5, 40, 30.0, 8, 130)])
def test_attention_window_kept_tokens_softcap_value_size(dtype, window, keep_first, softcap, head_dim, v_dim):
    from liteinfer_b200 import ops

    heads, kv_heads, page = 4, 2, 8
    case = _paged_case((70, 1, 37, 26), (70, 1, 5, 1), kv_heads, head_dim, v_dim, page, dtype)
    q = _randn(case.tokens, heads * head_dim + 11, seed=9, dtype=dtype)
    out, want = (torch.zeros(case.tokens, heads * v_dim, dtype=dtype, device=DEV) for _ in range(2))
    args = (case.k_pool, case.v_pool, case.table, case.qsl, case.ctx, 4, 70, heads, kv_heads, head_dim, 0.3, window)
    ops.paged_attention(q, q.shape[1], out, *args, keep_first=keep_first, softcap=softcap)
    ref.paged_attention(q, q.shape[1], want, *args, keep_first=keep_first, softcap=softcap)
    torch.testing.assert_close(out.float(), want.float(), **_tol(dtype))


@pytest.mark.parametrize("decode", [False, True])
def test_attention_edges_of_window_and_kept_tokens_stand_out(decode):
    """One key gets a score far above the rest; the output is its value exactly when the key is visible: just
    inside and just outside the window, the last kept token and the first one that is not kept."""
    from liteinfer_b200 import ops

    head_dim, v_dim, page, n = 16, 24, 8, 90
    case = _paged_case((n,), (1 if decode else n,), 1, head_dim, v_dim, page, torch.float32, seed=4)
    case.k_pool.mul_(0.01)
    pos = n - 1                                                # the query looked at
    cases = [(21, 5, key, seen) for key, seen in ((pos - 20, True), (pos - 21, False), (4, True), (5, False), (0, True), (pos, True))]
    cases += [(26, 8, 64, True), (26, 8, 63, False), (26, 8, 7, True), (26, 8, 8, False)]     # both edges on page borders
    cases += [(0, 0, 0, True), (0, 3, 40, True), (1, 0, pos, True), (1, 0, pos - 1, False)]   # no window: a far key; a window of one
    for window, keep, key, seen in cases:
        k_pool = case.k_pool.clone()
        slot = int(case.table[0, key // page]) 
        k_pool[slot, 0, key % page] = 0.0
        k_pool[slot, 0, key % page, 2] = 50.0
        q = torch.zeros(case.tokens, head_dim, device=DEV)
        q[:, 2] = 1.0
        out = torch.zeros(case.tokens, v_dim, device=DEV)
        ops.paged_attention(q, head_dim, out, k_pool, case.v_pool, case.table, case.qsl, case.ctx, 1, case.tokens, 1, 1,
                            head_dim, 1.0, window, keep_first=keep, softcap=0.0)
        value = case.v_pool[slot, 0, key % page]
        close = float((out[-1] - value).abs().max()) < 1e-4
        assert close == seen, f"key {key} for the query at {pos}: expected {'visible' if seen else 'hidden'}"


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("window,keep_first,softcap", [(100, 4, 20.0), (70, 0, 8.0), (64, 130, 0.0), (0, 0, 15.0), (200, 65, 30.0)])
def test_tensor_core_attention_with_kept_tokens_and_softcap(head_dim, window, keep_first, softcap):
    """The mma.sync kernel's options (prompts, portions and split single tokens) against the plain function."""
    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    heads, kv_heads, page, dtype = 4, 2, 16, torch.bfloat16
    lengths, queries = (333, 700, 1, 260, 515), (333, 1, 1, 7, 1)
    case = _paged_case(lengths, queries, kv_heads, head_dim, head_dim, page, dtype, seed=3)
    q = _randn(case.tokens, heads * head_dim, seed=9, dtype=dtype)
    out, want = (torch.zeros(case.tokens, heads * head_dim, dtype=dtype, device=DEV) for _ in range(2))
    args = (case.k_pool, case.v_pool, case.table, case.qsl, case.ctx, 5, 333, heads, kv_heads, head_dim, head_dim ** -0.5, window)
    ref.paged_attention(q, q.shape[1], want, *args, keep_first=keep_first, softcap=softcap)
    ops.paged_attention(q, q.shape[1], out, *args, keep_first=keep_first, softcap=softcap)
    torch.testing.assert_close(out.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)
    plan = AttentionPlan(num_decode=3, decode_seqs=_ints([1, 2, 4]), decode_tokens=_ints([333, 334, 342]), num_prefill=2,
                         prefill_seqs=_ints([0, 3]), max_prefill_query_len=333, max_decode_context_len=700)
    for splits in (None, 3):
        out.zero_()
        ops.paged_attention(q, q.shape[1], out, *args, plan=plan, decode_splits=splits, keep_first=keep_first, softcap=softcap)
        torch.testing.assert_close(out.float(), want.float(), rtol=2 ** -6, atol=2 ** -6)


@pytest.mark.parametrize("kernel", ["mma", "tcgen05", "decode"])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_tensor_core_attention_edges_stand_out(kernel, head_dim):
    """As `test_attention_edges_of_window_and_kept_tokens_stand_out`, on the tensor-core kernels (bfloat16): the
    mma.sync kernel on a prompt and on a split single token, the tcgen05 kernel on a prompt; edges inside a key
    tile and on a tile's border."""
    from liteinfer_b200 import ops
    from liteinfer_b200.parts.context import AttentionPlan

    page, n, dtype = 16, 400, torch.bfloat16
    decode = kernel == "decode"
    for window, keep in ((143, 5), (128, 64), (208, 70)):
        case = _paged_case((n,), (1 if decode else n,), 1, head_dim, head_dim, page, dtype, seed=4)
        case.k_pool.mul_(0.01)
        pos = n - 1
        plan = None
        if decode:
            plan = AttentionPlan(num_decode=1, decode_seqs=_ints([0]), decode_tokens=_ints([0]), max_decode_context_len=n)
        elif kernel == "tcgen05":
            plan = AttentionPlan(num_prefill=1, prefill_seqs=_ints([0]), max_prefill_query_len=n)
        for key, seen in ((pos - window + 1, True), (pos - window, False), (keep - 1, True), (keep, False), (0, True)):
            k_pool = case.k_pool.clone()
            slot = int(case.table[0, key // page])
            k_pool[slot, 0, key % page] = 0.0
            k_pool[slot, 0, key % page, 2] = 60.0
            q = torch.zeros(case.tokens, head_dim, dtype=dtype, device=DEV)
            q[:, 2] = 1.0
            out = torch.zeros(case.tokens, head_dim, dtype=dtype, device=DEV)
            ops.paged_attention(q, head_dim, out, k_pool, case.v_pool, case.table, case.qsl, case.ctx, 1, case.tokens, 1, 1,
                                head_dim, 1.0, window, plan=plan, decode_splits=2 if decode else None, keep_first=keep,
                                softcap=0.0)
            value = case.v_pool[slot, 0, key % page]
            close = float((out[-1].float() - value.float()).abs().max()) < 2e-2
            assert close == seen, f"window {window}, kept {keep}: key {key} for the query at {pos}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_kv_write_partial_rotation_scaled_and_wide_values(dtype):
    from liteinfer_b200 import ops
    from liteinfer_b200.parts.position import yarn_inverse_frequencies

    heads, kv_heads, head_dim, v_dim, rot, page = 3, 1, 40, 56, 12, 8
    inv_freq, scale = yarn_inverse_frequencies(rot, 1000.0, 8.0, 16.0, 4.0, 0.5)
    inv_freq = inv_freq.to(DEV)
    assert scale > 1.2
    tokens = 21
    qkv = _randn(tokens, (heads + kv_heads) * head_dim + kv_heads * v_dim, seed=1, dtype=dtype)
    positions, seq_of = _ints(list(range(30, 30 + tokens - 1)) + [0]), _ints([0] * (tokens - 1) + [-1])
    table = _ints([[4, 2, 9, 0, 7, 1, 3]])
    pools = [(torch.zeros(10, kv_heads, page, head_dim, dtype=dtype, device=DEV),
              torch.zeros(10, kv_heads, page, v_dim, dtype=dtype, device=DEV)) for _ in range(2)]
    got, want = qkv.clone(), qkv.clone()
    ops.rope_kv_write(got, positions, seq_of, table, *pools[0], inv_freq, heads, kv_heads, head_dim, rot,
                      v_head_dim=v_dim, cos_sin_scale=scale)
    ref.rope_kv_write(want, positions, seq_of, table, *pools[1], inv_freq, heads, kv_heads, head_dim, rot,
                      v_head_dim=v_dim, cos_sin_scale=scale)
    torch.testing.assert_close(got[:-1].float(), want[:-1].float(), **_tol(dtype))
    torch.testing.assert_close(pools[0][0].float(), pools[1][0].float(), **_tol(dtype))
    assert torch.equal(pools[0][1], pools[1][1])
    assert torch.equal(got[:, heads * head_dim + rot:], qkv[:, heads * head_dim + rot:])     # k's tail, v: untouched in the row


# ------------------------------------------------------------------ the whole model
@pytest.fixture(scope="module")
def kegizen_dirs(tmp_path_factory):
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("kegizen")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in kc.ALL.items()}


def _expected(model_dir, requests):
    config, tensors = plain_kegizen.read_model(model_dir)
    return {name: plain_kegizen.forward(config, tensors, tokens).float() for name, tokens in requests.items()}


@pytest.mark.parametrize("name,lengths", [("keg_a", (1, 7, 61, 90)), ("keg_b", (2, 30, 45)), ("keg_c", (5, 52, 80, 18, 70)),
                                           ("keg_d", (3, 150, 97, 260))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_all_cuts(kegizen_dirs, tmp_path, name, lengths, dtype):
    config, _, page = kc.ALL[name]
    requests = {f"r{i}": kc.prompt(config["vocab"], n, 100 + i) for i, n in enumerate(lengths)}
    expected = _expected(kegizen_dirs[name], requests)
    trace = rh.Trace()
    rh.whole(trace, requests)
    rh.tail_decoded(trace, requests, tail=40)
    rh.portions(trace, requests)
    rh.mixed(trace, requests)
    longest = max(requests, key=lambda r: len(requests[r]))
    for i, token in enumerate(requests[longest]):            # every token a step of its own, from the first one on
        trace.add([(f"o-{longest}", [token], [0])], end=[f"o-{longest}"] if i == len(requests[longest]) - 1 else [])
    results = rh.run_program(trace, kegizen_dirs[name], dtype, tmp_path / "out", config["vocab"], page_size=page)
    worst, where = rh.worst_error(results, rh.gather_expected(trace, expected))
    limit = 2 * kc.FLOAT32_TOLERANCE[name] if dtype == "float32" else kc.BFLOAT16_TOLERANCE[name]
    assert worst < limit, f"worst difference {worst} at step {where}"


def test_layers_one_by_one_against_plain(kegizen_dirs):
    """The residual stream after every stop of the schedule (32-bit engine) equals the plain implementation's."""
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    config, tensors = plain_kegizen.read_model(kegizen_dirs["keg_a"])
    tokens = kc.prompt(config["vocab"], 45, 3)
    want: list = []
    plain_kegizen.forward(config, tensors, tokens, want)
    runner = build_runner(kegizen_dirs["keg_a"], torch.float32, DEV, 16, 8, 2)
    runner.cache.reserve(["a"], [45])
    context = runner.build_context([StepEntry("a", tokens, [44])])
    context.layer_trace = []
    runner.model.forward(context, runner.layer_caches)
    assert len(context.layer_trace) == len(want)
    for stop, (got, plain) in enumerate(zip(context.layer_trace, want)):
        assert float((got.cpu().double() - plain).abs().max()) < 2e-4, f"stop {stop}"


def test_greedy_generation_through_the_engine_on_gpu(kegizen_dirs):
    from liteinfer_b200.engine.llm import LLM
    from liteinfer_b200.sampling.params import SamplingParams

    config, tensors = plain_kegizen.read_model(kegizen_dirs["keg_b"])
    prompts = [kc.prompt(config["vocab"], n, 40 + n) for n in (3, 26, 9, 14, 2)]
    with LLM(str(kegizen_dirs["keg_b"]), dtype="float32", block_size=4, num_gpu_blocks=64, max_num_seqs=3,
             max_model_len=64, max_num_batched_tokens=16) as llm:
        outputs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for prompt, output in zip(prompts, outputs):
        tokens = list(prompt)
        for _ in range(12):
            tokens.append(int(plain_kegizen.forward(config, tensors, tokens)[-1].argmax()))
        assert list(output.token_ids) == tokens[len(prompt):]
