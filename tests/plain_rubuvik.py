"""The Rubuvik decoder stated plainly: whole sequences, no cache, no batching, one function per mechanism.

Written from the design's equations in this file's own notation; it shares no code with the product.
``forward(config, weights, tokens)`` returns the logits at every position (in the dtype of the weights:
tests use float64).  ``config`` is the dict a model folder's config.json holds.  Notation: T tokens, E stream
width, H heads, G key/value heads, D query/key size, V value size, W window, F inner width of a feed-forward,
X experts.

    x_0 = table[token] * embedding.scale
    per layer   x <- x + m * N_1b(mixer(N_1(x)))
                x <- x + m * N_2b(ff(N_2(x)))                       (layers with a feed-forward)
                x <- x + m * rms(y) * side.norm,  y = P (gelu(G x) * e_i(token))     (models with a token side)
    logits = table @ N_final(x)
    N(x) = x / sqrt(mean(x^2) + eps) * (1 + w),  m = residual_mult
"""
from __future__ import annotations

import math

import torch


# ---- configurations and weights of the tests --------------------------------------------------------
def lightning_layer(*, heads, dim, vdim, decay=None, mlp=None):
    if decay is None:
        decay = [math.exp(-1.0 / (1.5 + 4.0 * h)) for h in range(heads)]
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)), mlp=mlp)


def attention_layer(*, kind="attention", heads, kv_heads, dim, vdim, window=None, scale=None, q_temp=None, v_mix=False,
                    mlp=None):
    mixer = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if window is not None:
        mixer["mask"] = dict(size=window)
    if q_temp is not None:
        mixer["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    if v_mix:
        mixer["v_mix"] = True
    return dict(type=kind, mixer=mixer, mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(*, experts, top, ff, groups=None, scale=1.0, shared=None):
    router = dict(experts=experts, top=top, scale=scale)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    out = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        out["shared"] = dict(ff=shared)
    return out


def model_config(layers, *, vocab, width, eps=1e-5, embedding_scale=1.0, residual_mult=1.0, side=None):
    cfg = dict(architecture="Rubuvik", vocab=vocab, width=width, norm=dict(eps=eps),
               embedding=dict(scale=embedding_scale), residual_mult=residual_mult, layers=[dict(l) for l in layers])
    if side is not None:
        cfg["token_side"] = dict(dim=side)
    return cfg


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "final.norm": (E,)}
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        shapes["side.embed"] = (cfg["vocab"], side * len(cfg["layers"]))
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        shapes.update({p + "norm1": (E,), p + "norm1b": (E,)})
        H, D, V = m["heads"], m["dim"], m["vdim"]
        if kind == "lightning":
            shapes.update({p + "mix.q": (H * D, E), p + "mix.k": (H * D, E), p + "mix.v": (H * V, E),
                           p + "mix.g": (H * V, E), p + "mix.o": (E, H * V), p + "mix.norm": (H * V,)})
        else:
            G = m["kv_heads"]
            shapes.update({p + "mix.q": (H * D, E), p + "mix.k": (G * D, E), p + "mix.v": (G * V, E),
                           p + "mix.o": (E, H * V)})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
            if kind == "attention_2":
                shapes.update({p + "mix.q.b": (H * D,), p + "mix.k.b": (G * D,), p + "mix.v.b": (G * V,),
                               p + "mix.sink": (H,), p + "mix.g": (H, E)})
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes.update({p + "norm2": (E,), p + "norm2b": (E,)})
            if mlp["kind"] == "dense":
                F = mlp["ff"]
                shapes.update({p + "mlp.gate": (F, E), p + "mlp.up": (F, E), p + "mlp.down": (E, F)})
            else:
                F, X = mlp["expert"]["ff"], mlp["router"]["experts"]
                for e in range(X):
                    shapes.update({f"{p}mlp.e{e}.gate": (F, E), f"{p}mlp.e{e}.up": (F, E), f"{p}mlp.e{e}.down": (E, F)})
                shapes.update({p + "mlp.router": (X, E), p + "mlp.correction": (X,)})
                if mlp.get("shared"):
                    F = mlp["shared"]["ff"]
                    shapes.update({p + "mlp.shared.gate": (F, E), p + "mlp.shared.up": (F, E),
                                   p + "mlp.shared.down": (E, F)})
        if side:
            shapes.update({p + "side.gate": (side, E), p + "side.proj": (E, side), p + "side.norm": (E,)})
    return shapes


def random_weights(cfg, seed, dtype=torch.float32):
    """Weights that keep every mechanism alive: norm weights around zero (or around one where the weight is
    plain), projections at a scale that leaves the stream of order one, routers that spread their choices."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("mix.norm") or name.endswith("side.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "vmix":
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif leaf == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "router":      # decisive routers: most close calls are between experts that weigh little
            t = 4.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        # what a bfloat16 file would hold, so that a 64-bit evaluation and a loaded model see one model
        out[name] = t.to(torch.bfloat16).to(dtype)
    return out


# ---- mechanisms ---------------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_unit(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def lightning(h, m, w, p, eps):
    """Linear attention with one fixed decay a head: S_t = a S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = unit_rms(out.reshape(T, H * V), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def attention(h, m, w, p, eps, second, v_first):
    """Both attention mixers; ``second`` adds biases, unit q and k, the sink and the gate a head.  Returns the
    mixer's output and the values as cached (``v_first`` is None in the first layer that mixes values)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if second:
        q, k, v = q + w[p + "q.b"], k + w[p + "k.b"], v + w[p + "v.b"]
    if m.get("v_mix") and v_first is not None:          # entry by entry over all key/value heads together
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    cached = v
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, V)
    if second:
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    position = torch.arange(T)
    if m.get("q_temp"):
        steps = torch.floor((position + 1) / m["q_temp"]["every"]) + 1.0
        q = q * (1.0 + m["q_temp"]["coef"] * torch.log(steps)).to(h.dtype)[:, None, None]
    distance = position[:, None] - position[None, :]                    # i - j
    seen = distance >= 0
    if m.get("mask"):
        seen = seen & (distance < m["mask"]["size"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        score = (q[:, head] @ k[:, kv].T) * m["scale"] - slope * distance.to(h.dtype)
        score = score.masked_fill(~seen, -math.inf)
        if second:
            top = torch.maximum(score.max(-1, keepdim=True).values, w[p + "sink"][head])
            e = torch.exp(score - top)
            weights = e / (e.sum(-1, keepdim=True) + torch.exp(w[p + "sink"][head] - top))
        else:
            weights = torch.softmax(score, -1)
        out[:, head] = weights @ v[:, kv]
    if second:
        out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T, cached


STAKE_FLOOR = 0.05      # a close call between experts that both weigh less than this is no close call


def route(h, mlp, w, p):
    """Chosen experts [T, top] and their weights; also the margin of every token's choice: the gap between the
    last chosen and the first refused choice score, and between the last kept and the first refused group
    (infinite where the scores at stake are all below STAKE_FLOOR: either choice then gives nearly the same sum)."""
    r = mlp["router"]
    X, top = r["experts"], r["top"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"]
    margin = torch.full((h.shape[0],), math.inf, dtype=h.dtype)
    if r.get("groups"):
        count, keep = r["groups"]["count"], r["groups"]["keep"]
        best = choice.view(-1, count, X // count).max(-1).values
        order = torch.sort(best, -1, descending=True)
        if keep < count:
            weight = s.view(-1, count, X // count).max(-1).values
            stake = torch.maximum(weight.gather(1, order.indices[:, keep - 1:keep]),
                                  weight.gather(1, order.indices[:, keep:keep + 1]))[:, 0]
            gap = order.values[:, keep - 1] - order.values[:, keep]
            margin = torch.where(stake > STAKE_FLOOR, gap, margin)
        kept = torch.zeros_like(best, dtype=torch.bool).scatter(1, best.topk(keep, -1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(X // count, 1), -math.inf)
    order = torch.sort(choice, -1, descending=True)
    if top < X:
        stake = torch.maximum(s.gather(1, order.indices[:, top - 1:top]), s.gather(1, order.indices[:, top:top + 1]))[:, 0]
        gap = order.values[:, top - 1] - order.values[:, top]
        margin = torch.minimum(margin, torch.where(stake > STAKE_FLOOR, gap, torch.full_like(gap, math.inf)))
    ids = choice.topk(top, -1).indices
    return ids, s.gather(1, ids) * r["scale"], margin


def experts(h, mlp, w, p):
    ids, weights, margin = route(h, mlp, w, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), weights[t]):
            q = f"{p}e{e}."
            out[t] += a * gated_unit(h[t], w[q + "gate"], w[q + "up"], w[q + "down"])
    if mlp.get("shared"):
        out = out + gated_unit(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"])
    return out, margin


def token_side(x, tokens, index, cfg, w, p, eps):
    dim = cfg["token_side"]["dim"]
    e = w["side.embed"][tokens][:, index * dim:(index + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return unit_rms(y, eps) * w[p + "norm"]


def forward(cfg, w, tokens, *, streams=None, margins=None, leave_out=()):
    """Logits [T, vocab].  ``streams`` (a list) receives the stream after every layer; ``margins`` (a list) the
    routers' smallest margin at every position; ``leave_out`` names mechanisms to drop (tests use it to show
    that each one moves the logits)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    v_first = None
    worst = torch.full((len(tokens),), math.inf, dtype=x.dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = zero_centred_norm(x, w[p + "norm1"], eps)
        mixer = dict(layer["mixer"])
        for key in leave_out:
            mixer.pop(key, None)
        if layer["type"] == "lightning":
            a = lightning(h, mixer, w, p + "mix.", eps)
        else:
            a, v = attention(h, mixer, w, p + "mix.", eps, layer["type"] == "attention_2", v_first)
            if mixer.get("v_mix") and v_first is None:
                v_first = v
        x = x + m * zero_centred_norm(a, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = zero_centred_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                f = gated_unit(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
            else:
                f, margin = experts(h, mlp, w, p + "mlp.")
                worst = torch.minimum(worst, margin)
            x = x + m * zero_centred_norm(f, w[p + "norm2b"], eps)
        if cfg.get("token_side") and "token_side" not in leave_out:
            x = x + m * token_side(x, tokens, i, cfg, w, p + "side.", eps)
        if streams is not None:
            streams.append(x.clone())
    if margins is not None:
        margins.append(worst)
    return zero_centred_norm(x, w["final.norm"], eps) @ w["embed"].T
