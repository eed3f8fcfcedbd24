"""The kernels of mixers with a matrix state (decay per key channel, delta rule behind a short convolution), of
sliding-window attention with turned and normed q and k and a gate per head, and of the scaled embedding: each
alone against its plain PyTorch statement (tests/plain_kernels.py), at sizes of their own."""
from __future__ import annotations

import pytest
import torch

import plain_kernels as P
from test_kernels_gpu import DEV, DTYPES, K, _cache_case, randn, tol
from test_pipesun_kernels_gpu import _Batch

pytestmark = pytest.mark.gpu
F32 = dict(rtol=3e-5, atol=3e-5)

# (heads, key width, value width): every split of a column over lanes (key widths up to 16, 32, 64, 128, 256,
# 512), widths no 16-byte copy fits, fewer columns than a block owns and more than one block of them
SCAN_SIZES = [(3, 6, 10), (2, 16, 24), (2, 24, 8), (1, 40, 200), (2, 64, 32), (2, 128, 48), (1, 200, 20),
              (1, 256, 36), (1, 512, 12)]
# requests of a step (cached tokens are irrelevant to a scan): none of a stage's sizes divides these
SCAN_LENS = [(0, 1), (0, 19), (0, 2), (0, 9)]


def _states(slots, floats, seed):
    state = randn(slots, floats, dtype=torch.float32, seed=seed, scale=0.3)
    return state, state.cpu().clone()


class _HostBatch:
    """The same batch with its tensors on the host, for the plain statements."""

    def __init__(self, batch):
        for name in ("positions", "req_index", "query_start", "state_slots"):
            setattr(self, name, getattr(batch, name).cpu())
        self.num_reqs = batch.num_reqs


@pytest.fixture(params=[None, "4"], ids=["columns-chosen", "columns-4"])
def columns_a_thread(request, monkeypatch):
    """The scans with the columns a thread holds left to the launch, and with four wherever the key width allows."""
    if request.param is None:
        monkeypatch.delenv("KVCORE_SCAN_COLS", raising=False)
    else:
        monkeypatch.setenv("KVCORE_SCAN_COLS", request.param)
    return request.param


@pytest.mark.parametrize("front", [3, 8])      # the state begins `front` floats into its row: off and on a 16-byte boundary
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", SCAN_SIZES)
def test_decay_per_channel_scan(dtype, heads, dim, vdim, front, columns_a_thread):
    batch = _Batch(SCAN_LENS, slots=[4, 0, 2, 5])
    tokens = batch.num_tokens
    rows = randn(tokens, 2 * heads * dim + heads * vdim + 8, dtype=dtype, seed=1)
    q, k = rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim]
    v = rows[:, 2 * heads * dim:2 * heads * dim + heads * vdim]
    z = randn(tokens, heads * dim, dtype=dtype, seed=2, scale=3.0)
    state, host_state = _states(6, front + heads * dim * vdim + (5 if front % 4 else 4), seed=3)
    sizes = dict(heads=heads, dim=dim, value_dim=vdim, q_scale=dim ** -0.5, tau=2.5, state_offset=front)
    got = K().gla_scan(q, k, v, z, state, batch, **sizes)
    want = P.gla_scan(q.cpu(), k.cpu(), v.cpu(), z.cpu(), host_state, _HostBatch(batch), **sizes)
    torch.testing.assert_close(got.cpu(), want, **F32)
    torch.testing.assert_close(state.cpu(), host_state, **F32)       # also the slots and floats nobody owns


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 6, 10), (2, 2, 16, 24), (6, 3, 32, 72), (2, 1, 64, 200),
                                                     (4, 1, 128, 40), (1, 1, 200, 20), (2, 2, 256, 12), (2, 1, 512, 8)])
@pytest.mark.parametrize("front", [7, 4])
def test_delta_rule_scan(heads, kv_heads, dim, vdim, front, columns_a_thread):
    batch = _Batch(SCAN_LENS, slots=[1, 3, 0, 2])
    tokens, qk = batch.num_tokens, kv_heads * dim
    prepared = randn(tokens, 2 * qk + heads * vdim + 2 * heads, dtype=torch.float32, seed=4)
    unit = lambda x: (x.reshape(tokens, kv_heads, dim) / x.reshape(tokens, kv_heads, dim).norm(dim=-1, keepdim=True)).reshape(tokens, qk)
    prepared[:, :qk] = unit(prepared[:, :qk]) * dim ** -0.5
    prepared[:, qk:2 * qk] = unit(prepared[:, qk:2 * qk])
    prepared[:, -2 * heads:] = torch.sigmoid(prepared[:, -2 * heads:])          # beta and the decay lie in (0, 1)
    state, host_state = _states(4, front + heads * dim * vdim + (1 if front % 4 else 0), seed=5)
    sizes = dict(heads=heads, kv_heads=kv_heads, dim=dim, value_dim=vdim, state_offset=front)
    got = K().delta_scan(prepared, state, batch, **sizes)
    want = P.delta_scan(prepared.cpu(), host_state, _HostBatch(batch), **sizes)
    torch.testing.assert_close(got.cpu(), want, **F32)
    torch.testing.assert_close(state.cpu(), host_state, **F32)


@pytest.mark.parametrize("kind", ["decay", "delta"])
def test_scans_do_not_depend_on_the_cut(kind):
    """A request in one portion, in portions of 1, 2, 5 and 17 tokens beside other requests in other slots, and
    token by token: the same bits out, the same bits in the state."""
    heads, kv_heads, dim, vdim, tokens = 2, 1, 40, 24, 31
    gen = dict(dtype=torch.float32)
    if kind == "decay":
        rows = randn(tokens, 2 * heads * dim + heads * vdim, seed=6, **gen)
        q, k, v = rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim], rows[:, 2 * heads * dim:]
        z = randn(tokens, heads * dim, seed=8, **gen)

        def run(lo, hi, state, batch):
            return K().gla_scan(q[lo:hi], k[lo:hi], v[lo:hi], z[lo:hi], state, batch, heads=heads, dim=dim,
                                value_dim=vdim, q_scale=0.3, tau=4.0)
    else:
        prepared = randn(tokens, 2 * kv_heads * dim + heads * vdim + 2 * heads, seed=10, **gen) * 0.2
        prepared[:, -2 * heads:] = torch.sigmoid(prepared[:, -2 * heads:])

        def run(lo, hi, state, batch):
            return K().delta_scan(prepared[lo:hi].contiguous(), state, batch, heads=heads, kv_heads=kv_heads,
                                  dim=dim, value_dim=vdim)
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


@pytest.mark.parametrize("dim,vdim", [(40, 24), (128, 40), (128, 13), (200, 12), (512, 8)])
@pytest.mark.parametrize("kind", ["decay", "delta"])
def test_scans_do_not_depend_on_the_rows_a_thread_holds(kind, dim, vdim, monkeypatch):
    """A launch picks how many rows of a column one thread holds, and of how many neighbouring columns, by the
    columns it has (a single prompt, or a batch of many requests): every choice gives the same bits, out and in
    the state.  The prompts hold full stages of tokens and a rest."""
    heads, kv_heads, lens = 2, 1, [(0, 29), (0, 1), (0, 6)]
    batch = _Batch(lens, slots=[2, 0, 1])
    tokens = batch.num_tokens
    seen = []
    for rows_a_thread, columns_a_thread in ((None, None), ("4", "1"), ("8", "1"), ("16", "1"), ("4", "4"), ("8", "4"),
                                            (None, "4"), (None, "1")):
        for name, value in (("KVCORE_SCAN_ROWS", rows_a_thread), ("KVCORE_SCAN_COLS", columns_a_thread)):
            if value is None:
                monkeypatch.delenv(name, raising=False)
            else:
                monkeypatch.setenv(name, value)
        state, _ = _states(3, heads * dim * vdim, seed=21)
        if kind == "decay":
            rows = randn(tokens, 2 * heads * dim + heads * vdim, seed=22, dtype=torch.float32)
            z = randn(tokens, heads * dim, seed=23, dtype=torch.float32)
            out = K().gla_scan(rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim], rows[:, 2 * heads * dim:], z,
                               state, batch, heads=heads, dim=dim, value_dim=vdim, q_scale=0.3, tau=4.0)
        else:
            prepared = randn(tokens, 2 * kv_heads * dim + heads * vdim + 2 * heads, seed=24, dtype=torch.float32) * 0.2
            prepared[:, -2 * heads:] = torch.sigmoid(prepared[:, -2 * heads:])
            out = K().delta_scan(prepared, state, batch, heads=heads, kv_heads=kv_heads, dim=dim, value_dim=vdim)
        seen.append((out.cpu(), state.cpu()))
    for out, state in seen[1:]:
        assert torch.equal(out, seen[0][0]) and torch.equal(state, seen[0][1])


@pytest.mark.parametrize("kind", ["decay", "delta"])
def test_a_far_token_is_read_through_the_state(kind):
    """One token writes a value under a key that no other token's key touches; 300 tokens on, with decays of one,
    the query that points along that key reads the value back and no other query sees it."""
    heads, dim, vdim, tokens, far = 1, 32, 16, 301, 0
    k = torch.zeros(tokens, dim)
    k[:, 1:] = torch.randn(tokens, dim - 1, generator=torch.Generator().manual_seed(11)) * 0.1
    k[far] = 0.0
    k[far, 0] = 1.0
    v = torch.randn(tokens, vdim, generator=torch.Generator().manual_seed(12))
    q = k.clone()
    q[-1] = 0.0
    q[-1, 0] = 1.0
    state = torch.zeros(1, dim * vdim, dtype=torch.float32, device=DEV)
    batch = _Batch([(0, tokens)])
    if kind == "decay":
        z = torch.full((tokens, dim), 40.0)                                  # sigmoid(40) is one in 32-bit
        rows = torch.cat([q, k, v], dim=1).to(DEV)                           # q, k and v are views of one tensor of rows
        out = K().gla_scan(rows[:, :dim], rows[:, dim:2 * dim], rows[:, 2 * dim:], z.to(DEV), state, batch,
                           heads=heads, dim=dim, value_dim=vdim, q_scale=1.0, tau=1.0)
    else:
        k = k / k.norm(dim=-1, keepdim=True)
        q[:-1] = k[:-1]
        extra = torch.ones(tokens, 2)                                        # beta one, decay one
        prepared = torch.cat([q, k, v, extra], dim=1).to(DEV)
        out = K().delta_scan(prepared, state, batch, heads=heads, kv_heads=1, dim=dim, value_dim=vdim)
    torch.testing.assert_close(out[-1, 0].cpu(), v[far], rtol=1e-4, atol=1e-4)
    assert (out[1:-1, 0].cpu() - v[far]).abs().max() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,heads,kv_heads,dim,vdim", [(1, 2, 1, 6, 10), (2, 4, 2, 16, 8), (4, 2, 2, 40, 72),
                                                          (9, 1, 1, 128, 64)])
def test_convolution_and_what_the_delta_rule_reads(dtype, taps, heads, kv_heads, dim, vdim):
    """Portions that are shorter and longer than the taps, beside single tokens, in two steps: the inputs in front
    of a portion come from the state, which the step brings up to date."""
    channels = 2 * kv_heads * dim + heads * vdim
    b_col = channels + heads * vdim
    a_col = b_col + heads
    width = (a_col + heads + 7) & ~7
    weights = randn(channels, taps, dtype=dtype, seed=13)
    a_log, dt_bias = randn(heads, dtype=dtype, seed=14), randn(heads, dtype=dtype, seed=15)
    keep = channels * (taps - 1)
    state, host_state = _states(5, 4 + keep + 3, seed=16)
    sizes = dict(heads=heads, kv_heads=kv_heads, dim=dim, value_dim=vdim, b_col=b_col, a_col=a_col,
                 q_scale=dim ** -0.5, unit_eps=1e-6, state_offset=4)
    for step, lens in enumerate(([(0, 1), (0, 2), (0, 13), (0, 5)], [(1, 1), (2, 11), (13, 1), (5, 3)])):
        batch = _Batch(lens, slots=[3, 0, 4, 1])
        rows = randn(batch.num_tokens, width, dtype=dtype, seed=17 + step)
        got = K().conv_prepare(rows, weights, state, batch, a_log, dt_bias, **sizes)
        want = P.conv_prepare(rows.cpu(), weights.cpu(), host_state, _HostBatch(batch), a_log.cpu(), dt_bias.cpu(), **sizes)
        torch.testing.assert_close(got.cpu(), want, **F32)
        torch.testing.assert_close(state.cpu(), host_state, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,vdim", [(3, 10), (2, 64), (1, 288)])
def test_norm_and_gate_behind_the_read_out(dtype, heads, vdim):
    tokens = 7
    o = randn(tokens, heads, vdim, dtype=torch.float32, seed=18, scale=4.0)
    rows = randn(tokens, heads * vdim + 16, dtype=dtype, seed=19)
    weight = randn(vdim, dtype=dtype, seed=20) + 1.0
    got = torch.zeros(tokens, 2 * heads * vdim, dtype=dtype, device=DEV)
    want = got.cpu().clone()
    K().gated_rms_norm(o, rows[:, 8:8 + heads * vdim], weight, 1e-5, got[:, heads * vdim:], 0.7)
    P.gated_rms_norm(o.cpu(), rows.cpu()[:, 8:8 + heads * vdim], weight.cpu(), 1e-5, want[:, heads * vdim:], 0.7)
    torch.testing.assert_close(got.cpu(), want, **(F32 if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("gated", [True, False])
def test_gate_per_head(dtype, gated):
    tokens, heads, vdim = 5, 3, 24
    o = randn(tokens, heads, vdim, dtype=torch.float32, seed=21)
    gate = randn(tokens, heads + 5, dtype=dtype, seed=22)[:, 2:2 + heads] if gated else None
    got = torch.zeros(tokens, heads * vdim + 8, dtype=dtype, device=DEV)
    want = got.cpu().clone()
    K().head_gate(o, gate, got[:, 8:], 1.2)
    P.head_gate(o.cpu(), None if gate is None else gate.cpu(), want[:, 8:], 1.2)
    torch.testing.assert_close(got.cpu(), want, **(F32 if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding(dtype):
    table = randn(50, 72, dtype=dtype, seed=23)
    ids = torch.tensor([0, 49, 7, 7, 13], dtype=torch.int32, device=DEV)
    got = K().embed_scaled(table, ids, 8.5)
    torch.testing.assert_close(got.float().cpu(), P.embed_scaled(table.cpu(), ids.cpu(), 8.5).to(got.dtype).float(),
                               **(F32 if got.dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_heads,k_heads,dim,rot,vwidth,norm", [(4, 2, 16, 8, 48, True), (2, 2, 10, 0, 20, True),
                                                                 (8, 2, 64, 64, 256, True), (3, 1, 24, 24, 8, False)])
def test_turn_norm_and_cache_write(dtype, q_heads, k_heads, dim, rot, vwidth, norm):
    """Positions across a page's border, a request that begins in the middle of a page, pages in an order of
    their own; q comes back in place, k and v go to the cached row."""
    page, pages = 4, 12
    lens = [(0, 6), (5, 1), (3, 7)]
    batch = _Batch(lens)
    table = torch.tensor([[3, 9, 0, 0], [7, 1, 0, 0], [11, 2, 5, 0]], dtype=torch.int32, device=DEV)
    qc, kc = q_heads * dim, k_heads * dim
    rows = randn(batch.num_tokens, (qc + kc + vwidth + q_heads + 7) & ~7, dtype=dtype, seed=24)
    inv_freq = None if rot == 0 else (100.0 ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot) / 2.0).to(DEV)
    cache = torch.zeros(pages, 1, page, kc + vwidth, dtype=dtype, device=DEV)
    host_rows, host_cache = rows.cpu().clone(), cache.cpu().clone()
    sizes = dict(q_heads=q_heads, k_heads=k_heads, dim=dim, value_width=vwidth, norm=norm, eps=1e-5)
    K().turn_norm_kv_write(rows, inv_freq, rot, batch, table, cache, **sizes)
    P.turn_norm_kv_write(host_rows, None if inv_freq is None else inv_freq.cpu(), rot, _HostBatch(batch), table.cpu(),
                         host_cache, **sizes)
    close = F32 if dtype == torch.float32 else tol(dtype)
    torch.testing.assert_close(rows.cpu()[:, :qc], host_rows[:, :qc], **close)
    torch.testing.assert_close(rows.cpu()[:, qc:], host_rows[:, qc:], rtol=0, atol=0)      # k, v, gates: untouched
    torch.testing.assert_close(cache.cpu(), host_cache, **close)


# dtype, key width, value width, page, (cached, new), window: the edge among the step's own tokens and in the cache,
# inside a page and on its border, in prompts (tiles and the general kernel) and decoded (keys in chunks too)
WINDOW_EDGES = [
    (torch.float32, 20, 12, 4, (0, 40), 9),
    (torch.float32, 20, 12, 4, (39, 1), 8),
    (torch.float32, 56, 40, 16, (70, 3), 37),
    (torch.bfloat16, 64, 128, 16, (100, 201), 50),
    (torch.bfloat16, 64, 128, 16, (300, 5), 48),
    (torch.bfloat16, 128, 64, 16, (640, 1), 100),
    (torch.bfloat16, 128, 64, 16, (1000, 1), 513),
    (torch.bfloat16, 80, 48, 16, (90, 1), 1),
]


@pytest.mark.parametrize("dtype,dim,vdim,page,lens,window", WINDOW_EDGES)
@pytest.mark.parametrize("place", ["inside", "outside"])
def test_the_window_s_edge(dtype, dim, vdim, page, lens, window, place):
    """A row at position p sees positions p - window + 1 .. p.  One key is made to dominate the last row's flat
    scores by scaling it along the query: at p - window + 1 the output is that key's value; at p - window, with a
    huge value, it leaves no trace.  The cached row is [k of all kv heads | v of all kv heads]."""
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
    page_id, slot = int(case["table"][0, position // page]), position % page
    for g in range(kv_heads):
        plane[page_id, 0, slot, g * dim:(g + 1) * dim] = (q[-1, 0].float() * (12.0 / q[-1, 0].float().pow(2).sum())).to(dtype)
    value = plane[page_id, 0, slot, kv_heads * dim:].view(kv_heads, vdim)
    if place == "outside":
        value.fill_(3.0e4)
    out = K().attention_dims(q, plane, plane.view(-1)[kv_heads * dim:], case["table"], batch, scale=1.0, window=window,
                             out_dtype=torch.float32, value_heads=kv_heads, group=heads // kv_heads, maps=1,
                             key_width=dim, value_width=vdim, key_strides=(page * width, dim, width),
                             value_strides=(page * width, vdim, width), page_size=page, num_pages=plane.shape[0])
    assert K().read_status() == 0
    if place == "outside":
        assert out[-1].abs().max() < 50.0, "a key one position behind the window reached the row's output"
    elif window > 1:
        want = value.float().repeat_interleave(heads // kv_heads, dim=0)
        torch.testing.assert_close(out[-1], want, rtol=2e-2, atol=3e-2)
    else:       # a window of one position: the row sees itself alone
        torch.testing.assert_close(out[-1], value.float().repeat_interleave(heads // kv_heads, dim=0), rtol=1e-2, atol=1e-2)

