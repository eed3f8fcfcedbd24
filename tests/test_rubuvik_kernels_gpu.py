"""The kernels of the Rubuvik mechanisms, each alone against its plain PyTorch statement (tests/plain_kernels.py)
at sizes of their own: the scan with one fixed decay a head, the norm over all heads with a sigmoid gate, attention
with a slope per head on the distance (general kernel, tensor-core tiles, few-row form, keys in chunks) beside a
sink and a window, the query temperature and the value mixing of the cache write, the router with a choice
correction and groups, the sum that also leaves the stream in the activation type, the gated token input."""
from __future__ import annotations

import math

import pytest
import torch

import plain_kernels as P
from test_dutivik_kernels_gpu import _HostBatch, _states
from test_kernels_gpu import DEV, DTYPES, K, _cache_case, randn, tol
from test_pipesun_kernels_gpu import _Batch

pytestmark = pytest.mark.gpu
F32 = dict(rtol=3e-5, atol=3e-5)

SCAN_SIZES = [(3, 6, 10), (2, 16, 24), (1, 40, 200), (2, 64, 32), (2, 128, 48), (1, 200, 20), (1, 256, 36), (1, 512, 12)]
SCAN_LENS = [(0, 1), (0, 19), (0, 2), (0, 9)]


def _decays(heads):
    return torch.tensor([0.0, 1.0, 0.9, 0.5, 0.999][:heads] if heads > 1 else [0.97], dtype=torch.float32, device=DEV)


# ---- the scan with one fixed decay a head ---------------------------------------------------------------
@pytest.mark.parametrize("front", [3, 8])      # the state begins `front` floats into its row: off and on a 16-byte boundary
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", SCAN_SIZES)
def test_fixed_decay_scan(dtype, heads, dim, vdim, front):
    batch = _Batch(SCAN_LENS, slots=[4, 0, 2, 5])
    tokens = batch.num_tokens
    rows = randn(tokens, 2 * heads * dim + heads * vdim + 8, dtype=dtype, seed=1, scale=2.0)
    q, k = rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim]
    v = rows[:, 2 * heads * dim:2 * heads * dim + heads * vdim]
    decay = _decays(heads)
    state, host_state = _states(6, front + heads * dim * vdim + (5 if front % 4 else 4), seed=3)
    sizes = dict(heads=heads, dim=dim, value_dim=vdim, q_scale=0.7, state_offset=front)
    got = K().lightning_scan(q, k, v, decay, state, batch, **sizes)
    want = P.lightning_scan(q.cpu(), k.cpu(), v.cpu(), decay.cpu(), host_state, _HostBatch(batch), **sizes)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(state.cpu(), host_state, rtol=1e-4, atol=1e-4)       # also the slots and floats nobody owns


def test_fixed_decay_scan_does_not_depend_on_the_cut():
    """A request in one portion, in portions of 1, 2, 5 and 17 tokens beside other slots, and token by token: the
    same bits out, the same bits in the state."""
    heads, dim, vdim, tokens = 2, 40, 24, 31
    rows = randn(tokens, 2 * heads * dim + heads * vdim, seed=6, dtype=torch.float32)
    q, k, v = rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim], rows[:, 2 * heads * dim:]
    decay = torch.tensor([0.8, 0.995], dtype=torch.float32, device=DEV)

    def run(lo, hi, state, batch):
        return K().lightning_scan(q[lo:hi], k[lo:hi], v[lo:hi], decay, state, batch, heads=heads, dim=dim, value_dim=vdim)
    whole_state = torch.zeros(3, heads * dim * vdim, dtype=torch.float32, device=DEV)
    whole = run(0, tokens, whole_state, _Batch([(0, tokens)], slots=[1]))
    for cuts in ([1, 2, 5, 17, 6], [1] * tokens):
        state = torch.zeros(3, heads * dim * vdim, dtype=torch.float32, device=DEV)
        outs, at = [], 0
        for n in cuts:
            outs.append(run(at, at + n, state, _Batch([(at, n)], slots=[2])))
            at += n
        assert torch.equal(torch.cat(outs), whole)
        assert torch.equal(state[2], whole_state[1])
        assert not state[:2].any()


@pytest.mark.parametrize("dim,vdim", [(40, 24), (128, 40), (128, 13), (512, 8)])
def test_fixed_decay_scan_does_not_depend_on_the_rows_a_thread_holds(dim, vdim, monkeypatch):
    heads, lens = 2, [(0, 21), (0, 1), (0, 6)]
    batch = _Batch(lens, slots=[2, 0, 1])
    rows = randn(batch.num_tokens, 2 * heads * dim + heads * vdim, seed=7, dtype=torch.float32)
    q, k, v = rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim], rows[:, 2 * heads * dim:]
    decay = torch.tensor([0.9, 0.99], dtype=torch.float32, device=DEV)
    results = []
    for shape in ({}, {"KVCORE_SCAN_ROWS": "4"}, {"KVCORE_SCAN_ROWS": "8"}, {"KVCORE_SCAN_ROWS": "16"},
                  {"KVCORE_SCAN_COLS": "4"}, {"KVCORE_SCAN_COLS": "1"}):
        for name in ("KVCORE_SCAN_ROWS", "KVCORE_SCAN_COLS"):
            monkeypatch.delenv(name, raising=False)
        for name, value in shape.items():
            monkeypatch.setenv(name, value)
        state = torch.zeros(3, heads * dim * vdim, dtype=torch.float32, device=DEV)
        results.append((K().lightning_scan(q, k, v, decay, state, batch, heads=heads, dim=dim, value_dim=vdim), state))
    for out, state in results[1:]:
        assert torch.equal(out, results[0][0]) and torch.equal(state, results[0][1])


def test_a_far_token_is_read_through_the_fixed_decay_state():
    """One token writes a value under a key that no other token's key touches; 300 tokens on, with a decay of one,
    the query that points along that key reads the value back (through SiLU on all three) and no other query sees
    it; with a decay below one the same read-out has shrunk by decay^300."""
    dim, vdim, tokens = 32, 16, 301
    silu = lambda x: x / (1.0 + math.exp(-x))
    big = 6.0                                       # silu(6) = 5.985; silu(-20) is zero in 32-bit
    k = torch.full((tokens, dim), -20.0)
    k[:, 1:] = torch.randn(tokens, dim - 1, generator=torch.Generator().manual_seed(11)) * 0.3
    k[:, 0] = -20.0
    k[0] = -20.0
    k[0, 0] = big
    v = torch.randn(tokens, vdim, generator=torch.Generator().manual_seed(12))
    q = k.clone()
    q[-1] = -20.0
    q[-1, 0] = big
    rows = torch.cat([q, k, v], dim=1).to(DEV)
    want = silu(big) ** 2 * torch.nn.functional.silu(v[0])
    for a in (1.0, 0.99):
        state = torch.zeros(1, dim * vdim, dtype=torch.float32, device=DEV)
        out = K().lightning_scan(rows[:, :dim], rows[:, dim:2 * dim], rows[:, 2 * dim:],
                                 torch.tensor([a], dtype=torch.float32, device=DEV), state, _Batch([(0, tokens)]),
                                 heads=1, dim=dim, value_dim=vdim)
        torch.testing.assert_close(out[-1, 0].cpu(), want * a ** 300, rtol=1e-3, atol=1e-4)
        if a == 1.0:
            assert (out[1:-1, 0].cpu() - want).abs().max() > 0.1
        # the same with the last 40 tokens decoded one by one, in a slot that another request has used
        state = torch.full((3, dim * vdim), 7.0, dtype=torch.float32, device=DEV)
        state[1] = 0.0                                      # the runner zeroes a slot before its request's first step
        at, last = 0, None
        for n in [tokens - 40] + [1] * 40:
            last = K().lightning_scan(rows[at:at + n, :dim], rows[at:at + n, dim:2 * dim], rows[at:at + n, 2 * dim:],
                                      torch.tensor([a], dtype=torch.float32, device=DEV), state,
                                      _Batch([(at, n)], slots=[1]), heads=1, dim=dim, value_dim=vdim)
            at += n
        assert torch.equal(last[-1], out[-1])
        assert bool((state[0] == 7.0).all()) and bool((state[2] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,vdim", [(1, 10), (1, 200), (1, 4096 + 8), (3, 24)])
def test_norm_over_all_heads_with_a_sigmoid_gate(dtype, heads, vdim):
    tokens = 7
    o = randn(tokens, heads, vdim, dtype=torch.float32, seed=18, scale=4.0)
    rows = randn(tokens, heads * vdim + 16, dtype=dtype, seed=19)
    weight = randn(heads * vdim, dtype=dtype, seed=20)[:vdim] + 1.0
    got = torch.zeros(tokens, 2 * heads * vdim, dtype=dtype, device=DEV)
    want = got.cpu().clone()
    K().gated_rms_norm(o, rows[:, 8:8 + heads * vdim], weight, 1e-5, got[:, heads * vdim:], 0.7, gate_act="sigmoid")
    P.gated_rms_norm(o.cpu(), rows.cpu()[:, 8:8 + heads * vdim], weight.cpu(), 1e-5, want[:, heads * vdim:], 0.7,
                     gate_act="sigmoid")
    torch.testing.assert_close(got.cpu(), want, **(F32 if dtype == torch.float32 else tol(dtype)))


# ---- attention with a slope per head on the distance ------------------------------------------------------
def _slopes(heads, exponent=8.0):
    return torch.exp2(-exponent * torch.arange(1, heads + 1, dtype=torch.float64) / heads).to(torch.float32).to(DEV)


# dtype, heads, kv heads, key width, value width, page, requests (cached, new), window, sink
SLOPE_CASES = [
    (torch.float32, 4, 2, 20, 12, 4, [(0, 40), (13, 1), (5, 9)], 9, False),
    (torch.float32, 3, 1, 56, 40, 16, [(70, 3), (0, 1)], None, True),
    (torch.bfloat16, 4, 2, 64, 128, 16, [(100, 201), (0, 77)], 50, True),        # tiles of 64 rows
    (torch.bfloat16, 8, 2, 112, 40, 16, [(300, 5), (17, 3)], 130, False),         # the few-row form
    (torch.bfloat16, 4, 1, 128, 64, 16, [(640, 1), (1000, 1), (3, 1)], 100, True),  # decoded, keys in chunks
    (torch.bfloat16, 6, 3, 80, 48, 16, [(90, 1), (0, 300), (200, 1)], 40, False),  # portions beside single tokens
    (torch.bfloat16, 2, 2, 24, 20, 8, [(30, 4)], 7, True),                          # widths only the general kernel takes
]


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,vdim,page,lens,window,sink", SLOPE_CASES)
def test_attention_with_slopes(dtype, heads, kv_heads, dim, vdim, page, lens, window, sink):
    width = kv_heads * (dim + vdim)
    case = _cache_case(dtype, 1, 1, width, page, lens, seed=31)
    plane, batch = case["k_cache"], _Batch(lens)
    q = randn(batch.num_tokens, heads, dim, dtype=dtype, seed=32, scale=0.5)
    slopes = _slopes(heads, 6.0)
    sinks = randn(heads, dtype=torch.float32, seed=33) if sink else None
    args = dict(scale=dim ** -0.5, window=window, out_dtype=torch.float32, value_heads=kv_heads, group=heads // kv_heads,
                maps=1, key_width=dim, value_width=vdim, key_strides=(page * width, dim, width),
                value_strides=(page * width, vdim, width), page_size=page, num_pages=plane.shape[0])
    want = P.attention_dims(q.cpu(), plane.cpu(), plane.cpu().view(-1)[kv_heads * dim:], case["table"].cpu(),
                            _HostBatch(batch), sink=None if sinks is None else sinks.cpu(), slopes=slopes.cpu(), **args)
    flat = P.attention_dims(q.cpu(), plane.cpu(), plane.cpu().view(-1)[kv_heads * dim:], case["table"].cpu(),
                            _HostBatch(batch), sink=None if sinks is None else sinks.cpu(), **args)
    assert (want - flat).abs().max() > 1e-2, "the slopes move nothing in this case"
    close = F32 if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for force in (False, True):
        got = K().attention_dims(q, plane, plane.view(-1)[kv_heads * dim:], case["table"], batch, sink=sinks,
                                 slopes=slopes, force_general=force, **args)
        assert K().read_status() == 0
        torch.testing.assert_close(got.cpu(), want, **close)
    if dtype == torch.bfloat16 and batch.max_query_len == 1:
        for splits in (1, 3):
            got = K().attention_dims(q, plane, plane.view(-1)[kv_heads * dim:], case["table"], batch, sink=sinks,
                                     slopes=slopes, num_splits=splits, **args)
            torch.testing.assert_close(got.cpu(), want, **close)


SLOPE_EDGES = [
    (torch.float32, 20, 12, 4, (0, 40), 9),
    (torch.float32, 20, 12, 4, (39, 1), 8),
    (torch.bfloat16, 64, 128, 16, (100, 201), 50),
    (torch.bfloat16, 112, 40, 16, (300, 5), 130),
    (torch.bfloat16, 128, 64, 16, (640, 1), 100),
    (torch.bfloat16, 128, 64, 16, (1000, 1), 513),
    (torch.bfloat16, 80, 48, 16, (90, 1), 1),
]


@pytest.mark.parametrize("dtype,dim,vdim,page,lens,window", SLOPE_EDGES)
@pytest.mark.parametrize("place", ["inside", "outside"])
def test_the_window_s_edge_under_slopes_and_a_sink(dtype, dim, vdim, page, lens, window, place):
    """A row at position p sees positions p - window + 1 .. p.  One key is made to dominate the last row's scores
    (a score of 60 beats the slope's bias over the whole window, a slope of at most 2^-2 a position here, and the
    sink): at p - window + 1 the output is that key's value; at p - window, with a huge value, it leaves no trace."""
    heads, kv_heads = 4, 2
    context, query = lens
    last = context + query - 1
    position = last - window + (1 if place == "inside" else 0)
    if position < 0:
        pytest.skip("nothing lies in front of the first position")
    width = kv_heads * (dim + vdim)
    case = _cache_case(dtype, 1, 1, width, page, [lens], seed=23)
    plane, batch = case["k_cache"], _Batch([lens])
    q = randn(batch.num_tokens, heads * dim, dtype=dtype, seed=29).view(batch.num_tokens, heads, dim) * 0.05
    for h in range(1, heads):
        q[-1, h] = q[-1, 0]
    # a slope of 2^-2 .. 2^-8 a position: over a window of 513 the bias reaches 128 for the first head; the dominating
    # score exceeds it by 60
    slopes = _slopes(heads)
    reach = float(slopes.max()) * window + 60.0
    page_id, slot = int(case["table"][0, position // page]), position % page
    for g in range(kv_heads):
        plane[page_id, 0, slot, g * dim:(g + 1) * dim] = (q[-1, 0].float() * (reach / q[-1, 0].float().pow(2).sum())).to(dtype)
    value = plane[page_id, 0, slot, kv_heads * dim:].view(kv_heads, vdim)
    if place == "outside":
        value.fill_(3.0e4)
    sinks = torch.full((heads,), 2.0, dtype=torch.float32, device=DEV)
    out = K().attention_dims(q, plane, plane.view(-1)[kv_heads * dim:], case["table"], batch, scale=1.0, window=window,
                             out_dtype=torch.float32, value_heads=kv_heads, group=heads // kv_heads, maps=1,
                             key_width=dim, value_width=vdim, key_strides=(page * width, dim, width),
                             value_strides=(page * width, vdim, width), page_size=page, num_pages=plane.shape[0],
                             sink=sinks, slopes=slopes)
    assert K().read_status() == 0
    if place == "outside":
        assert out[-1].abs().max() < 50.0, "a key one position behind the window reached the row's output"
    else:
        want = value.float().repeat_interleave(heads // kv_heads, dim=0)
        torch.testing.assert_close(out[-1], want, rtol=2e-2, atol=3e-2)


def test_a_sink_that_dominates_leaves_nothing():
    """A sink far above every score takes the whole weight: the output vanishes; far below, it changes nothing."""
    dtype, heads, kv_heads, dim, vdim, page, lens = torch.bfloat16, 4, 2, 64, 32, 16, [(50, 3), (20, 1)]
    width = kv_heads * (dim + vdim)
    case = _cache_case(dtype, 1, 1, width, page, lens, seed=41)
    plane, batch = case["k_cache"], _Batch(lens)
    q = randn(batch.num_tokens, heads, dim, dtype=dtype, seed=42, scale=0.3)
    args = dict(scale=0.2, window=24, out_dtype=torch.float32, value_heads=kv_heads, group=2, maps=1, key_width=dim,
                value_width=vdim, key_strides=(page * width, dim, width), value_strides=(page * width, vdim, width),
                page_size=page, num_pages=plane.shape[0], slopes=_slopes(heads))
    run = lambda sink: K().attention_dims(q, plane, plane.view(-1)[kv_heads * dim:], case["table"], batch,
                                          sink=None if sink is None else torch.full((heads,), sink, dtype=torch.float32, device=DEV),
                                          **args)
    plain = run(None)
    assert run(80.0).abs().max() < 1e-6
    torch.testing.assert_close(run(-80.0), plain, rtol=1e-5, atol=1e-5)


# ---- what the cache write does to q and to the values ----------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,k_heads,dim,vwidth,norm,q_temp,mixed", [
    (4, 2, 16, 48, False, (0.4, 3), True), (2, 2, 10, 20, True, (1.5, 1), False), (8, 2, 64, 256, True, None, True),
    (3, 1, 24, 8, False, (0.5, 128), False)])
def test_query_temperature_and_value_mixing(dtype, q_heads, k_heads, dim, vwidth, norm, q_temp, mixed):
    """Positions across a page's border and across the temperature's periods, a request that begins in the middle
    of a page; q comes back in place and scaled, k and the (mixed) values go to the cached row."""
    page, pages = 4, 12
    lens = [(0, 6), (5, 1), (3, 7)]
    batch = _Batch(lens)
    table = torch.tensor([[3, 9, 0, 0], [7, 1, 0, 0], [11, 2, 5, 0]], dtype=torch.int32, device=DEV)
    qc, kc = q_heads * dim, k_heads * dim
    rows = randn(batch.num_tokens, (qc + kc + vwidth + q_heads + 7) & ~7, dtype=dtype, seed=24)
    first = randn(batch.num_tokens, vwidth + 8, dtype=dtype, seed=25)[:, 8:] if mixed else None
    lam = torch.tensor(0.3125, dtype=torch.float32, device=DEV) if mixed else None
    cache = torch.zeros(pages, 1, page, kc + vwidth, dtype=dtype, device=DEV)
    host_rows, host_cache = rows.cpu().clone(), cache.cpu().clone()
    sizes = dict(q_heads=q_heads, k_heads=k_heads, dim=dim, value_width=vwidth, norm=norm, eps=1e-5, q_temp=q_temp)
    K().turn_norm_kv_write(rows, None, 0, batch, table, cache, mix_values=first, mix_weight=lam, **sizes)
    P.turn_norm_kv_write(host_rows, None, 0, _HostBatch(batch), table.cpu(), host_cache,
                         mix_values=None if first is None else first.cpu(), mix_weight=None if lam is None else lam.cpu(),
                         **sizes)
    close = F32 if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(rows.cpu()[:, :qc], host_rows[:, :qc], **close)
    torch.testing.assert_close(rows.cpu()[:, qc:], host_rows[:, qc:], rtol=0, atol=0)      # k, v, gates: untouched
    torch.testing.assert_close(cache.cpu(), host_cache, **close)
    if q_temp is not None and not norm:
        # the factor steps up exactly where floor((p + 1) / every) does
        coef, every = q_temp
        before = randn(batch.num_tokens, rows.shape[1], dtype=dtype, seed=24).float().cpu()[:, :qc]
        factor = (rows.cpu()[:, :qc].float() / before).median(dim=1).values
        steps = torch.div(batch.positions.cpu() + 1, every, rounding_mode="floor") + 1
        torch.testing.assert_close(factor, 1.0 + coef * torch.log(steps.float()), rtol=2e-2, atol=2e-2)


# ---- the router -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [5, 300])
@pytest.mark.parametrize("experts,top,groups,keep,corrected", [(12, 3, 4, 2, True), (8, 2, 4, 1, True), (6, 6, 2, 2, False),
                                                               (64, 6, 8, 3, True), (5, 1, 1, 1, True), (40, 3, 40, 3, False)])
def test_router_with_a_correction_and_groups(dtype, tokens, experts, top, groups, keep, corrected):
    width = 72
    x = randn(tokens, width, dtype=dtype, seed=51)
    router = randn(experts, width, dtype=torch.float32, seed=52, scale=0.5)
    correction = randn(experts, dtype=torch.float32, seed=53, scale=0.2) if corrected else None
    args = dict(score="softmax", correction=correction, group_count=groups, group_keep=keep, weight_scale=1.75)
    ids, weights, _ = K().moe_route(x, router, top, **args)
    want_ids, want_weights, _ = P.moe_route(x.cpu(), router.cpu(), top,
                                            **dict(args, correction=None if correction is None else correction.cpu()))
    per = experts // groups
    assert all(len({int(e) // per for e in row}) <= keep for row in ids.cpu()), "experts of too many groups"
    same = (ids.cpu() == want_ids).all(dim=1)
    assert same.float().mean() > 0.97          # a choice may hang on the last bit of a sum taken in another order
    torch.testing.assert_close(weights.cpu()[same], want_weights[same], rtol=1e-4, atol=1e-6)
    if corrected and groups > 1:
        free, _, _ = P.moe_route(x.cpu(), router.cpu(), top, score="softmax")
        assert (free != want_ids).any(), "correction and groups change no choice in this case"


def test_router_groups_that_decide():
    """A correction that lifts one group's expert above everything keeps that group, although another group holds
    the largest plain score; choice scores may be negative, and experts outside the kept groups are never chosen
    even when fewer than `top` experts inside have a positive choice score."""
    experts, width = 8, 16
    router = torch.zeros(experts, width, dtype=torch.float32, device=DEV)
    router[5, 0] = 4.0                                     # expert 5 (group 2 of four pairs) has the largest score
    correction = torch.full((experts,), -2.0, dtype=torch.float32, device=DEV)
    correction[0] = 3.0                                    # expert 0 (group 0) is lifted above it
    x = torch.zeros(3, width, dtype=torch.float32, device=DEV)
    x[:, 0] = 1.0
    ids, weights, _ = K().moe_route(x, router, 2, score="softmax", correction=correction, group_count=4, group_keep=1)
    assert ids.cpu().tolist() == [[0, 1]] * 3              # both of group 0, expert 1 with a negative choice score
    scores = torch.softmax(x.cpu() @ router.cpu().T, -1)
    torch.testing.assert_close(weights.cpu(), scores[:, :2], rtol=1e-5, atol=1e-7)


# ---- the sum behind a sub-layer, the gated token input -------------------------------------------------------
@pytest.mark.parametrize("width", [40, 1000, 4096 + 24])
@pytest.mark.parametrize("weight_dtype", [torch.float32, torch.bfloat16])
def test_sum_that_also_leaves_the_stream_in_the_activation_type(width, weight_dtype):
    x = randn(9, width, dtype=torch.float32, seed=61, scale=3.0)
    a = randn(9, width, dtype=torch.bfloat16, seed=62)
    w = randn(width, dtype=weight_dtype, seed=63) + 1.0
    want, _ = P.stream_add_norm(x.cpu().clone(), a.cpu(), w.cpu(), 1e-5)
    got, avg, rounded = K().stream_add_norm(x, a, w, 1e-5, rounded=torch.bfloat16)
    assert avg is None and rounded.dtype == torch.bfloat16 and got.data_ptr() == x.data_ptr()
    torch.testing.assert_close(got.cpu(), want, **F32)
    assert torch.equal(rounded, got.to(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,column,total", [(6, 12, 30), (24, 0, 24), (256, 512, 1024), (7, 7, 21)])
def test_gated_token_input(dtype, dim, column, total):
    tokens = 11
    z = randn(tokens, dim, dtype=dtype, seed=71, scale=2.0)
    rows = randn(tokens, total + 8, dtype=dtype, seed=72)[:, 8:]
    got = K().gelu_mul(z, rows, column)
    torch.testing.assert_close(got.cpu(), P.gelu_mul(z.cpu(), rows.cpu(), column), **(F32 if dtype == torch.float32 else tol(dtype)))
