"""The Dutivik decoder stated plainly: whole sequences, no cache, no batching, one function per mechanism.

Written from the design's equations in this file's own notation; it shares no code with the product.
``forward(config, weights, tokens)`` returns the logits at every position (in the dtype of the weights:
tests use float64).  Notation: T tokens, E stream width, H heads, G key/value heads, D query/key size,
V value size, R rotated entries, W window, C taps of the short convolution.
"""
from __future__ import annotations

import math

import torch


# ---- configurations and weights of the tests --------------------------------------------------------
def gla_layer(*, heads, dim, vdim, tau=4.0, rank=8, ff=48, weights_of=None):
    layer = dict(type="gla", mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau),
                 mlp=None if ff is None else dict(kind="dense", ff=ff))
    layer["_rank"] = rank          # the low-rank size of the decay projection is a tensor's shape, not a key
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def parallel_layer(*, heads, kv_heads, dim, vdim, window, rot_dims=None, base=10000.0, factor=None, scale=None,
                   r_heads, r_kv_heads, r_dim, r_vdim, conv=4, left_scale=1.0, right_scale=1.0, ff=48,
                   weights_of=None):
    rot = dict(base=base, dims=dim if rot_dims is None else rot_dims)
    if factor is not None:
        rot["scaling"] = dict(factor=factor)
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=window), rot=rot,
                scale=scale if scale is not None else dim ** -0.5)
    right = dict(heads=r_heads, kv_heads=r_kv_heads, dim=r_dim, vdim=r_vdim, conv=conv)
    layer = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale),
                 mlp=None if ff is None else dict(kind="dense", ff=ff))
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def model_config(layers, *, vocab, width, eps=1e-5, embedding_scale=None):
    layers = [dict(layer) for layer in layers]
    for layer in layers:
        if "weights_of" in layer:      # the entry of a layer that borrows its weights equals the owner's
            owner = layers[layer["weights_of"]]
            layer.update(type=owner["type"], mixer=owner["mixer"], mlp=owner["mlp"], _rank=owner.get("_rank"))
    return dict(architecture="Dutivik", vocab=vocab, width=width, norm=dict(eps=eps),
                embedding=dict(scale=math.sqrt(width) if embedding_scale is None else embedding_scale), layers=layers)


def public_config(cfg):
    """The configuration as a model folder stores it (without this file's private keys)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in layer.items() if not k.startswith("_")} for layer in cfg["layers"]]
    return out


def tensor_shapes(cfg):
    E = cfg["width"]
    shapes = {"embed": (cfg["vocab"], E), "final.norm": (E,), "final.norm.b": (E,)}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (E,), p + "norm1.b": (E,)})
        if layer["type"] == "gla":
            H, D, V, r = m["heads"], m["dim"], m["vdim"], layer["_rank"]
            shapes.update({p + "mix.q": (H * D, E), p + "mix.k": (H * D, E), p + "mix.v": (H * V, E),
                           p + "mix.g": (H * V, E), p + "mix.o": (E, H * V), p + "mix.norm": (V,),
                           p + "mix.a1": (r, E), p + "mix.a2": (H * D, r), p + "mix.a2.b": (H * D,)})
        else:
            a, b = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            shapes.update({p + "mix.left.q": (H * D, E), p + "mix.left.k": (G * D, E), p + "mix.left.v": (G * V, E),
                           p + "mix.left.g": (H, E), p + "mix.left.o": (E, H * V)})
            H, G, D, V, C = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
            q = p + "mix.right."
            shapes.update({q + "q": (G * D, E), q + "q.conv": (G * D, C), q + "k": (G * D, E), q + "k.conv": (G * D, C),
                           q + "v": (H * V, E), q + "v.conv": (H * V, C), q + "b": (H, E), q + "a": (H, E),
                           q + "A_log": (H,), q + "dt_bias": (H,), q + "norm": (V,), q + "g": (H * V, E),
                           q + "o": (E, H * V)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (F, E), p + "mlp.up": (F, E), p + "mlp.down": (E, F)})
    return shapes


def random_weights(cfg, seed, dtype=torch.float32):
    """Weights that keep every mechanism alive: norms near one, decays spread over (0, 1), projections at a
    scale that leaves the stream of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith("norm1") or name.endswith(".norm") and len(shape) == 1:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".b") and len(shape) == 1:
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.5 + 3.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) - 2.0
        elif leaf == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf == "a2":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        if name.endswith("mix.a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        # what a bfloat16 file would hold, so that a 64-bit evaluation and a loaded model see one model
        out[name] = t.to(torch.bfloat16).to(dtype)
    return out


# ---- mechanisms ---------------------------------------------------------------------------------------
def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def dense_feed_forward(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def turn_pairs(x, positions, base, dims, factor):
    """``x [T, heads, D]``: entries 2i and 2i+1 (i < dims/2) turn by ``position * base^(-2i/dims) / factor``."""
    out = x.clone()
    if dims == 0:
        return out
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims) / factor
    angle = positions.to(x.dtype)[:, None, None] * freq
    cos, sin = torch.cos(angle), torch.sin(angle)
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def windowed_attention(q, k, v, scale, window):
    """``q [T, H, D]``, ``k [T, G, D]``, ``v [T, G, V]``; position i sees j with ``0 <= i - j < window``."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def left_mixer(h, w, p, m, eps):
    """Sliding-window attention with turned, unit-rms q and k and a sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
    pos = torch.arange(T)
    q = turn_pairs((h @ w[p + "q"].T).view(T, H, D), pos, float(rot["base"]), rot["dims"], factor)
    k = turn_pairs((h @ w[p + "k"].T).view(T, G, D), pos, float(rot["base"]), rot["dims"], factor)
    v = (h @ w[p + "v"].T).view(T, G, V)
    o = windowed_attention(unit_rms(q, eps), unit_rms(k, eps), v, m["scale"], m["mask"]["size"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w[p + "o"].T


def short_convolution(x, taps):
    """``x [T, channels]``, ``taps [channels, C]``: the last column multiplies the current token, zeros before the start."""
    T, C = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(C - 1, x.shape[1], dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for j in range(C):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def unit_vector(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, decay):
    """``q, k [T, H, D]``, ``v [T, H, V]``, ``beta, decay [T, H]``: the state is decayed, corrected towards the
    value by the delta rule, and read after the write."""
    T, H, D = q.shape
    V = v.shape[2]
    S = torch.zeros(H, D, V, dtype=q.dtype)
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        S = S * decay[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def right_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    share = torch.arange(H) // (H // G)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = gated_delta_rule(q[:, share], k[:, share], v, beta, decay)
    o = unit_rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * left_mixer(h, w, p + "left.", m["left"], eps)
            + m["right_scale"] * right_mixer(h, w, p + "right.", m["right"], eps))


def gated_linear_attention(q, k, v, alpha):
    """``q, k, alpha [T, H, D]``, ``v [T, H, V]``: a decay per key channel, read after the write."""
    T, H, D = q.shape
    V = v.shape[2]
    S = torch.zeros(H, D, V, dtype=q.dtype)
    out = torch.zeros(T, H, V, dtype=q.dtype)
    for t in range(T):
        S = S * alpha[t][:, :, None] + torch.einsum("hd,hv->hdv", k[t], v[t])
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def gla_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).view(T, H, D) ** (1.0 / m["tau"])
    o = gated_linear_attention(q, k, v, alpha)
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * V) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- the model ------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, collect=None):
    """Logits ``[T, vocab]``; ``collect`` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    w = weights
    x = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "gla":
            y = gla_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
        if layer["mlp"] is not None:
            y = y + dense_feed_forward(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
        x = x + y
        if collect is not None:
            collect.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["embed"].T


__all__ = ["forward", "gla_layer", "model_config", "parallel_layer", "public_config", "random_weights", "tensor_shapes"]
