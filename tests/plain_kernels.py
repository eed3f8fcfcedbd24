"""Plain PyTorch statement of every kernel op, with the signatures of ``kvcore_b200.kernels``.

Two uses, both in tests only: (1) each CUDA kernel is compared alone against the function
of the same name here; (2) ``install(monkeypatch)`` swaps these in for the CUDA wrappers so
that the host side (step function, cache manager, scheduler, entry point) can be exercised
on a machine without a GPU.  The product never imports this file.
"""
from __future__ import annotations


import numpy as np
import torch


def require_device(device) -> None:
    return None


def ensure_built(verbose: bool = False) -> str:
    return "plain"


def read_status(reset: bool = True) -> int:
    return 0


def peek_status() -> int:
    return 0


def raise_on_status() -> None:
    return None


def check_attention_shape(num_heads, num_kv_heads, head_dim, dtype) -> None:
    from kvcore_b200.kernels.api import check_attention_shape as real

    real(num_heads, num_kv_heads, head_dim, dtype)


def gather_rows(table, ids, out=None):
    return table[ids.long()]


def feed_tokens(token_ids, source, sampled):
    take = source >= 0
    token_ids[take] = sampled[source[take].long()]


def rmsnorm(x, weight, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * y).to(x.dtype)


def add_rmsnorm(h, residual, weight, eps):
    residual.copy_((h.float() + residual.float()).to(h.dtype))
    return rmsnorm(residual, weight, eps)


def silu_mul(gate_up, group=0):
    inter = gate_up.shape[1] // 2
    if group:
        runs = gate_up.reshape(gate_up.shape[0], inter // group, 2, group)
        gate, up = runs[:, :, 0].reshape(-1, inter).float(), runs[:, :, 1].reshape(-1, inter).float()
    else:
        gate, up = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    act = torch.nn.functional.silu(gate).to(gate_up.dtype).float()
    return (act * up).to(gate_up.dtype)


def _rotate(x, positions, inv_freq):
    half = x.shape[-1] // 2
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


def rope_inplace(q, k, positions, inv_freq):
    q.copy_(_rotate(q, positions, inv_freq))
    if k is not None:
        k.copy_(_rotate(k, positions, inv_freq))


def rope_table(positions, inv_freq):
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    return torch.stack((angles.cos(), angles.sin()), dim=-1)


def _rotate_with(x, cos_sin):
    half = x.shape[-1] // 2
    cos, sin = cos_sin[:, None, :, 0], cos_sin[:, None, :, 1]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


def rope_kv_write(qkv, positions, req_index, cos_sin, table, k_cache, v_cache,
                  num_heads, num_kv_heads, head_dim, *, write_kv=True):
    tokens = qkv.shape[0]
    q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :q_size].view(tokens, num_heads, head_dim)
    k = qkv[:, q_size:q_size + kv_size].view(tokens, num_kv_heads, head_dim)
    v = qkv[:, q_size + kv_size:].view(tokens, num_kv_heads, head_dim)
    if cos_sin is not None:
        q.copy_(_rotate_with(q, cos_sin))
        k.copy_(_rotate_with(k, cos_sin))
    if write_kv:
        page_size = k_cache.shape[2]
        for t in range(tokens):
            pos = int(positions[t])
            page = int(table[int(req_index[t]), pos // page_size])
            assert page > 0, "write through the null page"
            k_cache[page, :, pos % page_size, :] = k[t]
            v_cache[page, :, pos % page_size, :] = v[t]


def paged_attention(qkv, k_cache, v_cache, table, ctx, num_heads, num_kv_heads, head_dim, scale, window,
                    *, force_general=False, num_splits=None, use_tma=True, use_tc5=True, cos_sin=None,
                    write_kv=None, keep_first=0):
    if write_kv is not None:   # the call also rotates q, k and writes this step's k, v
        rope_kv_write(qkv, ctx.positions, ctx.req_index, cos_sin, table, k_cache, v_cache,
                      num_heads, num_kv_heads, head_dim, write_kv=write_kv)
    return paged_attention_plain(qkv, k_cache, v_cache, table, ctx.positions, ctx.req_index,
                                 num_heads, num_kv_heads, head_dim, scale, window, keep_first)


def paged_attention_plain(qkv, k_cache, v_cache, table, positions, req_index,
                          num_heads, num_kv_heads, head_dim, scale, window, keep_first=0):
    tokens = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    q = qkv[:, : num_heads * head_dim].view(tokens, num_heads, head_dim).float()
    for t in range(tokens):
        pos = int(positions[t])
        first = 0 if not window else max(0, pos - window + 1)
        keys = torch.arange(first, pos + 1, device=qkv.device)
        if keep_first and first > 0:     # the kept first positions that lie behind the window
            keys = torch.cat((torch.arange(0, min(keep_first, first), device=qkv.device), keys))
        pages = table[int(req_index[t])].long()[keys // page_size]
        assert bool((pages > 0).all()), "read through the null page"
        offsets = keys % page_size
        k = k_cache[pages, :, offsets, :].float()  # [n, KVH, D]
        v = v_cache[pages, :, offsets, :].float()
        for h in range(num_heads):
            g = h // group
            scores = (k[:, g, :] @ q[t, h]) * scale
            probs = torch.softmax(scores, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (probs @ v[:, g, :]).to(qkv.dtype)
    return out


def layer_norm(x, weight, bias, eps, out_dtype=None):
    xf = x.float()
    centred = xf - xf.mean(-1, keepdim=True)
    y = centred / torch.sqrt(centred.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def stream_add(base, a=None, b=None, out=None):
    if out is not None:
        out.copy_(base.float())
    else:
        out = base if base.dtype == torch.float32 else base.float()
    if a is not None:
        addend = a.float() if b is None else a.float() + b.float()
        out = out.add_(addend) if (out is base or out.data_ptr() != base.data_ptr()) else out + addend
    return out


def _rms(x, eps):
    xf = x.float()
    return xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm_shift(x, weight, eps, out_dtype=None, *, shift=None, state=None, ctx=None):
    y = _rms(x, eps) * weight.float()
    if shift is not None:
        before = torch.empty_like(y)
        starts = [int(v) for v in ctx.query_start]
        for r in range(ctx.num_reqs):
            lo, hi = starts[r], starts[r + 1]
            slot = int(ctx.state_slots[r])
            before[lo] = state[slot]
            before[lo + 1:hi] = y[lo:hi - 1]
            state[slot] = y[hi - 1]
        y = y + (before - y) * shift.float()
    return y.to(out_dtype or x.dtype)


def stream_add_norm(x, a, weight, eps, *, out=None, stack=None, depth=0, coeffs=None, rounded=None):
    result = x + _rms(a, eps) * weight.float()
    if out is None:
        out = x
    out.copy_(result)
    avg = None
    if coeffs is not None:
        avg = torch.zeros_like(result)
        for j in range(depth):
            avg = avg + coeffs[j].float() * stack[j]
        avg = avg + coeffs[depth].float() * result
    if rounded is not None:
        return out, avg, out.to(rounded)
    return out, avg


def gelu_mul(z, rows, column):
    zf = z.float()
    gelu = 0.5 * zf * (1.0 + torch.tanh(0.7978845608028654 * (zf + 0.044715 * zf ** 3)))
    return (gelu * rows[:, column:column + z.shape[1]].float()).to(z.dtype)


def _strided(tensor, page, slot, head, strides, width):
    """The ``width`` entries of (page, head, slot) inside the cache tensor ``tensor`` (a view into it)."""
    begin = page * strides[0] + head * strides[1] + slot * strides[2]
    return tensor.reshape(-1)[begin:begin + width] if tensor.is_contiguous() else \
        torch.as_strided(tensor, (width,), (1,), tensor.storage_offset() + begin)


def attention_dims(q, keys, values, table, ctx, *, value_heads, group, maps, key_width, value_width, page_size,
                   num_pages, key_strides, value_strides, scale, sink=None, window=None, out=None, out_dtype=None,
                   force_general=False, num_splits=None, slopes=None):
    tokens, hq, _ = q.shape
    if out is None:
        out = torch.empty((tokens, hq, value_width), dtype=out_dtype or q.dtype, device=q.device)
    flat_k = torch.as_strided(keys, (keys.untyped_storage().nbytes() // keys.element_size() - keys.storage_offset(),), (1,),
                              keys.storage_offset())
    flat_v = torch.as_strided(values, (values.untyped_storage().nbytes() // values.element_size() - values.storage_offset(),),
                              (1,), values.storage_offset())
    for t in range(tokens):
        pos = int(ctx.positions[t])
        first = 0 if not window else max(0, pos - window + 1)
        positions = torch.arange(first, pos + 1)
        pages = table[int(ctx.req_index[t])].long()[positions // page_size]
        assert bool((pages > 0).all()) and bool((pages < num_pages).all()), "read through a page that is not held"
        slots = positions % page_size
        for h in range(hq):
            vh = h // (group * maps)
            kh = vh * maps + h % maps
            k_begin = pages * key_strides[0] + kh * key_strides[1] + slots * key_strides[2]
            v_begin = pages * value_strides[0] + vh * value_strides[1] + slots * value_strides[2]
            k = flat_k[k_begin[:, None] + torch.arange(key_width)[None]].float()
            v = flat_v[v_begin[:, None] + torch.arange(value_width)[None]].float()
            scores = (k @ q[t, h].float()) * scale
            if slopes is not None:
                scores = scores - slopes[h] * (pos - positions).float()
            top = scores.max() if sink is None else torch.maximum(scores.max(), sink[h])
            weights = torch.exp(scores - top)
            total = weights.sum() + (0.0 if sink is None else torch.exp(sink[h] - top))
            out[t, h] = ((weights / total) @ v).to(out.dtype)
    return out


def latent_prepare(kv_rows, norm_weight, eps, inv_freq, dims, ctx, table, cache, q, q_width, q_out, *,
                   q_latent=None, write=True):
    tokens, heads, q_row = q_out.shape
    rank = norm_weight.numel()
    rot = cache.shape[3] - rank
    lead = q_row - rot                   # the entries of a q_out row in front of the turned part
    page_size = cache.shape[2]

    def turn(x, pos):          # [..., rot] float, interleaved pairs of the first ``dims`` entries
        x = x.clone()
        angle = torch.tensor(float(pos), dtype=torch.float32) * inv_freq[: dims // 2]
        c, s = torch.cos(angle), torch.sin(angle)
        u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
        x[..., 0:dims:2] = u * c - v * s
        x[..., 1:dims:2] = v * c + u * s
        return x

    for t in range(tokens):
        pos = int(ctx.positions[t])
        if write:
            page = int(table[int(ctx.req_index[t]), pos // page_size])
            assert page > 0
            latent = _rms(kv_rows[t, :rank], eps) * norm_weight.float()
            cache[page, 0, pos % page_size, :rank] = latent.to(cache.dtype)
            cache[page, 0, pos % page_size, rank:] = turn(kv_rows[t, rank:].float(), pos).to(cache.dtype)
        q_out[t, :, lead:] = turn(q[t, :, q_width:].float(), pos).to(q_out.dtype)
        if q_latent is not None:
            q_out[t, :, :lead] = q_latent[t]


def gather_cached_rows(cache, table, src_req, src_pos, col0, cols, out, *, copies=1, head_stride=0):
    page_size = cache.shape[2]
    for n in range(src_req.numel()):
        pos = int(src_pos[n])
        page = int(table[int(src_req[n]), pos // page_size])
        assert page > 0
        for h in range(copies):
            out[n, h * head_stride:h * head_stride + cols] = cache[page, 0, pos % page_size, col0:col0 + cols]


def head_norm_kv_write(rows, q_weight, k_weight, eps, ctx, table, cache, *, q_vectors, k_vectors, dim, value_width,
                       write=True):
    tokens = rows.shape[0]
    page_size = cache.shape[2]
    qc, kc = q_vectors * dim, k_vectors * dim
    q = rows[:, :qc].reshape(tokens, q_vectors, dim)
    rows[:, :qc] = (_rms(q, eps) * q_weight.float()).to(rows.dtype).reshape(tokens, qc)
    if not write:
        return
    k = (_rms(rows[:, qc:qc + kc].reshape(tokens, k_vectors, dim), eps) * k_weight.float()).to(rows.dtype)
    for t in range(tokens):
        pos = int(ctx.positions[t])
        page = int(table[int(ctx.req_index[t]), pos // page_size])
        assert page > 0
        cache[page, 0, pos % page_size, :kc] = k[t].reshape(kc)
        cache[page, 0, pos % page_size, kc:] = rows[t, qc + kc:qc + kc + value_width]


def maps_combine(a, lam, eps, out_scale, out_dtype):
    tokens, heads, _, width = a.shape
    o = a[:, :, 0] - lam * a[:, :, 1]
    return (_rms(o, eps) * out_scale).to(out_dtype).reshape(tokens, heads * width)


def sigmoid_gate_mul(o, gate):
    tokens, heads, width = o.shape
    return (o.float().reshape(tokens, heads * width) * torch.sigmoid(gate.float())).to(o.dtype)


def heads_linear(x, weight, out=None):
    result = torch.einsum("thk,hnk->thn", x.float(), weight.float()).to(x.dtype)
    if out is not None:
        out.copy_(result)
        return out
    return result


def qk_prepare(rows, positions, req_index, cos_sin, table, k_cache, v_cache, num_heads, num_kv_heads, head_dim, *,
               rotary_dim=None, norm=None, q_norm_weight=None, k_norm_weight=None, eps=0.0, value_from_key=False,
               write_kv=True):
    tokens = rows.shape[0]
    q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
    q, k = rows[:, :q_size].float(), rows[:, q_size:q_size + kv_size].float()
    v = (rows[:, q_size:q_size + kv_size] if value_from_key else rows[:, q_size + kv_size:]).clone()

    def rms(x, weight, heads):
        if norm is None:
            return x
        shaped = x if norm == "projection" else x.view(tokens, heads, head_dim)
        shaped = shaped * torch.rsqrt(shaped.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        return shaped.reshape(tokens, -1)

    def turn(x, heads):
        x = x.view(tokens, heads, head_dim)
        if cos_sin is None:
            return x
        rot = head_dim if rotary_dim is None else rotary_dim
        half = rot // 2
        cos, sin = cos_sin[:, None, :, 0], cos_sin[:, None, :, 1]
        a, b = x[..., :half], x[..., half:rot]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rot:]), dim=-1)

    q = turn(rms(q, q_norm_weight, num_heads), num_heads).to(rows.dtype)
    k = turn(rms(k, k_norm_weight, num_kv_heads), num_kv_heads).to(rows.dtype)
    rows[:, :q_size] = q.reshape(tokens, q_size)
    rows[:, q_size:q_size + kv_size] = k.reshape(tokens, kv_size)
    if write_kv:
        page_size = k_cache.shape[2]
        for t in range(tokens):
            pos = int(positions[t])
            page = int(table[int(req_index[t]), pos // page_size])
            assert page > 0, "write through the null page"
            k_cache[page, :, pos % page_size, :] = k[t]
            v_cache[page, :, pos % page_size, :] = v[t].view(num_kv_heads, head_dim)


def glu_clamped(gate_up, *, alpha, limit, shift):
    inter = gate_up.shape[1] // 2
    g = gate_up[:, :inter].float().clamp(max=limit)
    u = gate_up[:, inter:].float().clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + shift)).to(gate_up.dtype)


def moe_route(x, router, top, *, score="sigmoid", renormalize=False, gate_rows=None, correction=None,
              group_count=1, group_keep=1, weight_scale=1.0):
    z = x.float() @ router.float().T
    scores = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=-1)
    tokens, experts = scores.shape
    ids = torch.empty(tokens, top, dtype=torch.int32, device=x.device)
    weights = torch.empty(tokens, top, dtype=torch.float32, device=x.device)
    left = scores.clone() if correction is None else scores + correction.float()
    rows = torch.arange(tokens)
    if group_keep < group_count:
        best_of = left.reshape(tokens, group_count, experts // group_count).max(-1).values.clone()
        kept = torch.zeros(tokens, group_count, dtype=torch.bool)
        for _ in range(group_keep):  # the largest, the lowest index among equals
            best = best_of.max(dim=-1, keepdim=True).values
            index = (best_of == best).float().argmax(dim=-1)
            kept[rows, index] = True
            best_of[rows, index] = -float("inf")
        left = left.masked_fill(~kept.repeat_interleave(experts // group_count, 1), -float("inf"))
    for slot in range(top):          # the largest, the lowest index among equals
        best = left.max(dim=-1, keepdim=True).values
        index = (left == best).float().argmax(dim=-1)
        ids[:, slot] = index
        weights[:, slot] = scores[rows, index]
        left[rows, index] = -float("inf")
    if renormalize:
        weights = weights / weights.sum(-1, keepdim=True)
    weights = weights * weight_scale
    gates = None if gate_rows is None else torch.sigmoid(x.float() @ gate_rows.float().T)
    return ids, weights, gates


def moe_path(x, pairs, ff):
    return "tiles"


def moe_experts(x, ids, weights, gate_up, down, *, weight_on_input, path=None, grouping=None):
    tokens, top = ids.shape
    ff = gate_up.shape[1] // 2
    out = torch.empty(tokens * top, down.shape[1], dtype=x.dtype, device=x.device)
    for t in range(tokens):
        for s in range(top):
            e, w = int(ids[t, s]), weights[t, s]
            a = (w * x[t].float()).to(x.dtype).float() if weight_on_input else x[t].float()
            g = (gate_up[e, :ff].float() @ a).to(x.dtype).float()
            u = (gate_up[e, ff:].float() @ a).to(x.dtype).float()
            hidden = ((g * torch.sigmoid(g)).to(x.dtype).float() * u).to(x.dtype).float()
            if not weight_on_input:
                hidden = (w * hidden).to(x.dtype).float()
            out[t * top + s] = (down[e].float() @ hidden).to(x.dtype)
    return out


def moe_combine(expert_out, tokens, top, shared=None, gates=None):
    y = expert_out.float().view(tokens, top, -1).sum(1)
    if shared is not None:
        y = y + (shared.float() if gates is None else gates[:, :1] * shared.float())
    return y.to(expert_out.dtype)


def linear(x, weight, bias=None, *, out_dtype=None):
    y = x.float() @ weight.float().T
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def linear_silu_mul(x, weight, bias=None, *, group=0):
    return silu_mul(linear(x, weight, bias), group)


def norm_linear(h, residual, norm_weight, eps, weight, bias=None, *, silu_group=None, sumsq=None):
    if h is None:
        x = rmsnorm(residual, norm_weight, eps)
    elif residual is None:
        x, residual = rmsnorm(h, norm_weight, eps), h
    else:
        x = add_rmsnorm(h, residual, norm_weight, eps)
    out = linear(x, weight, bias) if silu_group is None else linear_silu_mul(x, weight, bias, group=silu_group)
    return out, residual


def linear_add_residual(x, weight, bias, residual):
    return linear(x, weight, bias), None


# ---- mixers with a matrix state, turned and normed attention inputs ------------------------------------
def embed_scaled(table, ids, scale):
    return table[ids.long()].float() * scale


def turn_norm_kv_write(rows, inv_freq, rot, ctx, table, cache, *, q_heads, k_heads, dim, value_width, norm=True,
                       eps=0.0, q_weight=None, k_weight=None, write=True, q_temp=None, mix_values=None,
                       mix_weight=None):
    tokens = rows.shape[0]
    page_size = cache.shape[2]
    qc, kc = q_heads * dim, k_heads * dim
    rot = rot if inv_freq is not None else 0

    def prepare(x, weight):                       # [T, heads, dim] float
        x = x.clone()
        if rot:
            angle = ctx.positions.float()[:, None, None] * inv_freq[: rot // 2].float()
            cos, sin = torch.cos(angle), torch.sin(angle)
            even, odd = x[..., 0:rot:2].clone(), x[..., 1:rot:2].clone()
            x[..., 0:rot:2] = even * cos - odd * sin
            x[..., 1:rot:2] = odd * cos + even * sin
        if norm:
            x = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        return x if weight is None else x * weight.float()

    q = prepare(rows[:, :qc].float().reshape(tokens, q_heads, dim), q_weight)
    if q_temp is not None:
        steps = torch.div(ctx.positions + 1, q_temp[1], rounding_mode="floor") + 1
        q = q * (1.0 + q_temp[0] * torch.log(steps.float()))[:, None, None]
    k = prepare(rows[:, qc:qc + kc].float().reshape(tokens, k_heads, dim), k_weight).to(rows.dtype)
    rows[:, :qc] = q.to(rows.dtype).reshape(tokens, qc)
    if not write:
        return
    values = rows[:, qc + kc:qc + kc + value_width]
    if mix_values is not None:
        lam = mix_weight.float()
        values = ((1.0 - lam) * values.float() + lam * mix_values.float()).to(rows.dtype)
    for t in range(tokens):
        pos = int(ctx.positions[t])
        page = int(table[int(ctx.req_index[t]), pos // page_size])
        assert page > 0
        cache[page, 0, pos % page_size, :kc] = k[t].reshape(kc)
        cache[page, 0, pos % page_size, kc:] = values[t]


def head_gate(o, gate, out, scale=1.0):
    tokens, heads, width = o.shape
    factor = scale if gate is None else torch.sigmoid(gate.float())[:, :, None] * scale
    out.copy_((o * factor).reshape(tokens, heads * width).to(out.dtype))
    return out


def _request_ranges(ctx):
    starts = [int(x) for x in ctx.query_start]
    return [(r, starts[r], starts[r + 1], int(ctx.state_slots[r])) for r in range(ctx.num_reqs)]


def gla_scan(q, k, v, z, state, ctx, *, heads, dim, value_dim, q_scale, tau, state_offset=0):
    tokens = q.shape[0]
    out = torch.empty((tokens, heads, value_dim), dtype=torch.float32, device=q.device)
    n = heads * dim * value_dim
    alpha = torch.exp(torch.nn.functional.logsigmoid(z.float()) / tau).reshape(tokens, heads, dim)
    qf = q.float().reshape(tokens, heads, dim) * q_scale
    kf, vf = k.float().reshape(tokens, heads, dim), v.float().reshape(tokens, heads, value_dim)
    for _, begin, end, slot in _request_ranges(ctx):
        S = state[slot, state_offset:state_offset + n].reshape(heads, value_dim, dim).transpose(1, 2).clone()   # kept column by column
        for t in range(begin, end):
            S = S * alpha[t][:, :, None] + kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, qf[t])
        state[slot, state_offset:state_offset + n] = S.transpose(1, 2).reshape(n)
    return out


def conv_prepare(rows, taps, state, ctx, a_log, dt_bias, *, heads, kv_heads, dim, value_dim, b_col, a_col, q_scale,
                 unit_eps, state_offset):
    tokens = rows.shape[0]
    channels, num_taps = taps.shape
    keep = num_taps - 1
    qk = kv_heads * dim
    out = torch.empty((tokens, channels + 2 * heads), dtype=torch.float32, device=rows.device)
    x = rows[:, :channels].float()
    for _, begin, end, slot in _request_ranges(ctx):
        held = state[slot, state_offset:state_offset + channels * keep].reshape(channels, keep)
        history = torch.cat([held.T.clone(), x[begin:end]])            # [keep + n, channels]
        acc = torch.zeros((end - begin, channels))
        for j in range(num_taps):
            acc = acc + history[j:j + end - begin] * taps[:, j].float()
        out[begin:end, :channels] = acc * torch.sigmoid(acc)
        if keep:
            state[slot, state_offset:state_offset + channels * keep] = history[-keep:].T.reshape(-1)
    for lo, scale in ((0, q_scale), (qk, 1.0)):
        vec = out[:, lo:lo + qk].reshape(tokens, kv_heads, dim)
        out[:, lo:lo + qk] = (vec / torch.sqrt(vec.pow(2).sum(-1, keepdim=True) + unit_eps) * scale).reshape(tokens, qk)
    out[:, channels:channels + heads] = torch.sigmoid(rows[:, b_col:b_col + heads].float())
    step = torch.nn.functional.softplus(rows[:, a_col:a_col + heads].float() + dt_bias.float())
    out[:, channels + heads:] = torch.exp(-torch.exp(a_log.float()) * step)
    return out


def delta_scan(prepared, state, ctx, *, heads, kv_heads, dim, value_dim, state_offset=0):
    tokens = prepared.shape[0]
    qk, n = kv_heads * dim, heads * dim * value_dim
    share = torch.arange(heads) // (heads // kv_heads)
    q = prepared[:, :qk].reshape(tokens, kv_heads, dim)[:, share]
    k = prepared[:, qk:2 * qk].reshape(tokens, kv_heads, dim)[:, share]
    v = prepared[:, 2 * qk:2 * qk + heads * value_dim].reshape(tokens, heads, value_dim)
    beta = prepared[:, 2 * qk + heads * value_dim:][:, :heads]
    gate = prepared[:, 2 * qk + heads * value_dim + heads:]
    out = torch.empty((tokens, heads, value_dim), dtype=torch.float32, device=prepared.device)
    for _, begin, end, slot in _request_ranges(ctx):
        S = state[slot, state_offset:state_offset + n].reshape(heads, value_dim, dim).transpose(1, 2).clone()   # kept column by column
        for t in range(begin, end):
            S = S * gate[t][:, None, None]
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S = S + k[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, q[t])
        state[slot, state_offset:state_offset + n] = S.transpose(1, 2).reshape(n)
    return out


def lightning_scan(q, k, v, decay, state, ctx, *, heads, dim, value_dim, q_scale=1.0, state_offset=0):
    tokens = q.shape[0]
    out = torch.empty((tokens, heads, value_dim), dtype=torch.float32, device=q.device)
    n = heads * dim * value_dim
    silu = torch.nn.functional.silu
    qf = silu(q.float()).reshape(tokens, heads, dim) * q_scale
    kf, vf = silu(k.float()).reshape(tokens, heads, dim), silu(v.float()).reshape(tokens, heads, value_dim)
    for _, begin, end, slot in _request_ranges(ctx):
        S = state[slot, state_offset:state_offset + n].reshape(heads, value_dim, dim).transpose(1, 2).clone()   # kept column by column
        for t in range(begin, end):
            S = S * decay.float()[:, None, None] + kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, qf[t])
        state[slot, state_offset:state_offset + n] = S.transpose(1, 2).reshape(n)
    return out


def gated_rms_norm(o, gate, weight, eps, out, scale=1.0, *, gate_act="silu"):
    tokens, heads, width = o.shape
    g = gate.float().reshape(tokens, heads, width)
    factor = g * torch.sigmoid(g) if gate_act == "silu" else torch.sigmoid(g)
    y = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * weight.float() * factor * scale
    out.copy_(y.reshape(tokens, heads * width).to(out.dtype))
    return out


# ---- sampling: the same counter-based noise as the CUDA kernel --------------------------------
def philox4x32_10(counter, key):
    c = [np.uint64(x) for x in counter]
    k = [np.uint64(x) for x in key]
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k[0]) & mask, lo1, (hi0 ^ c[3] ^ k[1]) & mask, lo0]
        k = [(k[0] + np.uint64(0x9E3779B9)) & mask, (k[1] + np.uint64(0xBB67AE85)) & mask]
    return [int(x) for x in c]


def exponential_noise(vocab: int, seed: int, token_index: int) -> np.ndarray:
    """q[i] ~ Exp(1) exactly as the kernel draws it (float32 arithmetic)."""
    q = np.empty(vocab, dtype=np.float32)
    lo, hi = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for group in range((vocab + 3) // 4):
        r = philox4x32_10((group, token_index, 0, 0), (lo, hi))
        for j in range(4):
            i = group * 4 + j
            if i < vocab:
                u = (np.float32(r[j]) + np.float32(0.5)) * np.float32(2.3283064365386963e-10)
                u = min(u, np.float32(0.99999994))
                q[i] = -np.log(u, dtype=np.float32)
    return q


def sample_row(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
               token_index: int, eps: float = 1e-5):
    """Returns (token, scores) where scores[i] = (x_i - max) - log(q_i) over kept entries."""
    from plain_llama import masked_logits

    if temperature < eps:
        return int(torch.argmax(logits)), None
    vocab = logits.numel()
    x = masked_logits(logits, temperature, top_k if top_k < vocab else None, top_p)
    q = torch.from_numpy(exponential_noise(vocab, seed, token_index))
    scores = (x - x.max()) - torch.log(q)
    return int(torch.argmax(scores)), scores


def sample(logits, packed_params, eps):
    out = torch.empty(logits.shape[0], dtype=torch.int32)
    for row in range(logits.shape[0]):
        temperature, top_k, top_p, lo, hi, index = packed_params[row].tolist()
        seed = int(lo) | (int(hi) << 32)
        out[row], _ = sample_row(logits[row].float().cpu(), temperature, int(top_k), top_p, seed, int(index), eps)
    return out.to(logits.device)


_NAMES = [
    "require_device", "ensure_built", "read_status", "peek_status", "raise_on_status", "check_attention_shape", "gather_rows", "feed_tokens", "rmsnorm",
    "add_rmsnorm", "silu_mul", "rope_inplace", "rope_table", "rope_kv_write", "paged_attention", "linear", "linear_silu_mul", "norm_linear", "linear_add_residual", "sample",
    "rms_norm_shift", "stream_add_norm", "attention_dims", "latent_prepare", "head_norm_kv_write", "maps_combine",
    "sigmoid_gate_mul", "heads_linear", "gather_cached_rows",
    "embed_scaled", "turn_norm_kv_write", "head_gate", "gla_scan", "conv_prepare", "delta_scan", "gated_rms_norm",
    "lightning_scan", "gelu_mul", "layer_norm", "stream_add", "qk_prepare", "glu_clamped", "moe_route", "moe_experts", "moe_combine", "moe_path",
]


def install(monkeypatch) -> None:
    """Replace the CUDA wrappers of ``kvcore_b200.kernels`` by the functions of this file."""
    import kvcore_b200.kernels as K

    module = globals()
    for name in _NAMES:
        monkeypatch.setattr(K, name, module[name])
