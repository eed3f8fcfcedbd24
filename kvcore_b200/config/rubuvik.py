"""Typed reader of a Rubuvik model folder's config.json, and its description as parts.

Rubuvik is a decoder on one 32-bit stream with a norm on both sides of each sub-layer and a factor ``m`` on
every addition: ``x <- x + m * norm1b(mixer(norm1(x)))``, then ``x <- x + m * norm2b(ff(norm2(x)))``; every
such norm is an RMS norm whose stored weight lies around zero (``x * rsqrt(mean(x^2) + eps) * (1 + w)``).
Behind the feed-forward a layer may add a *token side input*: a second embedding table holds ``dim`` entries
per token and layer, ``e``; ``y = P (gelu_tanh(G x) * e)`` reads the stream itself, and
``x <- x + m * y * rsqrt(mean(y^2) + eps) * w_side`` (a plain weight).  The embedded tokens are multiplied by
a constant; the head is the embedding table without it, behind a final norm.  Its keys:

    architecture     "Rubuvik"
    vocab, width     vocabulary and stream width
    norm.eps         eps of every norm of the model
    embedding.scale  factor on the embedded tokens
    residual_mult    the factor m
    token_side.dim   entries per token and layer of the side table (key absent: no side input)
    layers[i]        type ("lightning" | "attention" | "attention_2"), mixer {...},
                     mlp (null | {kind "dense", ff} | {kind "moe", expert {ff}, router {experts, top, scale,
                     groups {count, keep}}, shared {ff}})

``lightning``: linear attention with one fixed decay a head, mixer {heads, dim, vdim, decay [heads]}; q, k and v
pass SiLU, the heads' read-outs are RMS-normed together and gated by ``sigmoid(W_g h)``.
``attention`` / ``attention_2``: grouped-query attention without rotation, mixer {heads, kv_heads, dim, vdim,
scale, mask {size}, q_temp {coef, every}, v_mix}: a bias ``slope_h * (i - j)`` is taken off the scores
(``slope_h = 2^(-8 (h + 1) / heads)``), a sliding window of ``mask.size`` positions, q times
``1 + coef * ln(floor((p + 1) / every) + 1)``; layers with ``v_mix`` behind the first such layer cache
``(1 - lambda) v + lambda v_first``.  ``attention_2`` adds biases on q, k and v, a weightless RMS norm per
head on q and k, a sink per head in the softmax's denominator and a sigmoid gate per head on the output.
The mixture of experts takes a softmax over all experts, chooses by ``score + correction`` among the
``groups.keep`` best of ``groups.count`` groups of neighbouring experts, and weights the chosen experts'
outputs by ``score * router.scale``; a shared expert is added.

Tensors: ``embed``, ``side.embed``, ``final.norm``, ``l<i>.norm{1,1b,2,2b}``, ``l<i>.mix.{q,k,v,g,o,norm}``
(lightning), ``l<i>.mix.{q,k,v,o,vmix}`` (+ ``q.b, k.b, v.b, sink, g``: attention_2),
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router, correction, e<j>.{gate,up,down}, shared.{gate,up,down}}``,
``l<i>.side.{gate,proj,norm}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .config_json import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, default_schedule
from .toposun import DEFAULT_MAX_POSITIONS, _need, _number, _positive_int

ARCHITECTURE = "Rubuvik"
# constants the design fixes
NORM_WEIGHT_OFFSET = 1.0        # norms multiply by (1 + w)
SLOPE_EXPONENT = 8.0            # slope of head h: 2^(-8 (h + 1) / heads)
PLAIN_NAMES = {"gate": "gate", "up": "up", "down": "down"}


@dataclass(frozen=True)
class RubuvikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    side_dim: int
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int
    stored_dtype: str | None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RubuvikConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        for index, layer in enumerate(layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{index}] is not an object")
        side = raw.get("token_side")
        return cls(
            vocab=_positive_int(raw, "vocab", "the model"),
            width=_positive_int(raw, "width", "the model"),
            eps=_number(_need(raw, "norm", "the model"), "eps", "norm"),
            embedding_scale=_number(_need(raw, "embedding", "the model"), "scale", "embedding"),
            residual_mult=_number(raw, "residual_mult", "the model"),
            side_dim=_positive_int(side, "dim", "token_side") if side is not None else 0,
            layers=tuple(layers),
            max_positions=int(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
            stored_dtype=raw.get("dtype") or raw.get("torch_dtype"),
        )

    # ---- parts ---------------------------------------------------------------------------------
    def _norm(self, tensor: str, multiplier: float = 1.0) -> PartSpec:
        return PartSpec("rmsnorm_stream", dict(size=self.width, eps=self.eps, name=tensor, tensor=tensor,
                                               offset=NORM_WEIGHT_OFFSET, multiplier=multiplier))

    def _lightning(self, index: int, m: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer"
        heads = _positive_int(m, "heads", where)
        decay = _need(m, "decay", where)
        if (not isinstance(decay, (list, tuple)) or len(decay) != heads
                or any(isinstance(a, bool) or not isinstance(a, (int, float)) or not 0.0 <= a < float("inf") for a in decay)):
            raise ConfigError(f"config.json: {where}.decay must be {heads} numbers that are not negative, one a head")
        return PartSpec("lightning_attention", dict(
            hidden_size=self.width, num_heads=heads, head_dim=_positive_int(m, "dim", where),
            value_dim=_positive_int(m, "vdim", where), decay=tuple(float(a) for a in decay), eps=self.eps,
            name=f"l{index}.mix"))

    def _attention(self, index: int, m: Mapping[str, Any], second: bool, mixes: str | None) -> PartSpec:
        where = f"layers[{index}].mixer"
        heads, kv_heads = _positive_int(m, "heads", where), _positive_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv_heads}")
        mask, temp = m.get("mask"), m.get("q_temp")
        q_temp = None
        if temp:
            q_temp = (_number(temp, "coef", where + ".q_temp"), _positive_int(temp, "every", where + ".q_temp"))
        return PartSpec("gated_window_attention", dict(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=_positive_int(m, "dim", where),
            value_dim=_positive_int(m, "vdim", where), scale=_number(m, "scale", where),
            window=_positive_int(mask, "size", where + ".mask") if mask else None,
            rot_dims=0, rot_base=1.0, qk_norm=second, eps=self.eps, head_gate=second, bias=second, sink=second,
            slope_exponent=SLOPE_EXPONENT, q_temp=q_temp, value_mix=mixes, name=f"l{index}.mix"))

    def _gated_unit(self, name: str, ff: int) -> PartSpec:
        return PartSpec("swiglu", dict(hidden_size=self.width, intermediate_size=ff, tensor_names=PLAIN_NAMES, name=name))

    def _feed_forward(self, index: int, layer: Mapping[str, Any]) -> PartSpec | None:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where, name = f"layers[{index}].mlp", f"l{index}.mlp"
        kind = _need(mlp, "kind", where)
        if kind == "dense":
            return self._gated_unit(name, _positive_int(mlp, "ff", where))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design")
        router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
        experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top {top} exceeds experts {experts}")
        groups = router.get("groups")
        count = keep = 1
        if groups:
            count = _positive_int(groups, "count", where + ".router.groups")
            keep = _positive_int(groups, "keep", where + ".router.groups")
            if experts % count or keep > count or keep * (experts // count) < top:
                raise ConfigError(f"config.json: {where}.router.groups: {count} equal groups of {experts} experts, "
                                  f"of which {keep} must hold {top} experts")
        shared = mlp.get("shared")
        return PartSpec("routed_experts", dict(
            hidden_size=self.width, num_experts=experts, top_k=top,
            expert_size=_positive_int(expert, "ff", where + ".expert"), score="softmax", renormalize=False,
            weight_on="output", weight_scale=_number(router, "scale", where + ".router") if "scale" in router else 1.0,
            choice_correction=True, group_count=count, group_keep=keep,
            shared=self._gated_unit(f"{name}.shared", _positive_int(shared, "ff", where + ".shared")) if shared else None,
            tensor_names={"router": "router", "correction": "correction", "gate": "e{index}.gate", "up": "e{index}.up",
                          "down": "e{index}.down"},
            name=name))

    def to_model_spec(self) -> ModelSpec:
        layers = []
        count = len(self.layers)
        first_mix: int | None = None      # width of a token's values in the first layer that mixes values
        for index, layer in enumerate(self.layers):
            kind = _need(layer, "type", f"layers[{index}]")
            m = _need(layer, "mixer", f"layers[{index}]")
            if kind == "lightning":
                mixer = self._lightning(index, m)
            elif kind in ("attention", "attention_2"):
                mixes = None
                if m.get("v_mix"):
                    # the values are mixed entry by entry: what must agree is the width of a token's values
                    sizes = _positive_int(m, "kv_heads", f"layers[{index}].mixer") * _positive_int(m, "vdim", f"layers[{index}].mixer")
                    if first_mix is None:
                        first_mix, mixes = sizes, "first"
                    elif sizes != first_mix:
                        raise ConfigError(f"config.json: layers[{index}].mixer mixes in values of other sizes than its own")
                    else:
                        mixes = "later"
                mixer = self._attention(index, m, kind == "attention_2", mixes)
            else:
                raise ConfigError(f"config.json: layers[{index}].type {kind!r} is not a mixer of this design")
            feed_forward = self._feed_forward(index, layer)
            prefix = f"l{index}"
            norms = {"mixer_norm": self._norm(f"{prefix}.norm1"),
                     "mixer_out_norm": self._norm(f"{prefix}.norm1b", self.residual_mult)}
            if feed_forward is not None:
                norms["feed_forward_norm"] = self._norm(f"{prefix}.norm2")
                norms["feed_forward_out_norm"] = self._norm(f"{prefix}.norm2b", self.residual_mult)
            block = dict(hidden_size=self.width)
            if feed_forward is None:     # a layer without a feed-forward may still carry the norms around one
                block["unused_tensors"] = (f"{prefix}.norm2", f"{prefix}.norm2b")
            if self.side_dim:
                block["token_side"] = dict(dim=self.side_dim, index=index, eps=self.eps, scale=self.residual_mult,
                                           name=f"{prefix}.side")
            layers.append(LayerSpec(prefix=prefix, block=PartSpec("sandwich_residual", block), mixer=mixer,
                                    feed_forward=feed_forward, norms=norms))
        embedding = dict(vocab_size=self.vocab, hidden_size=self.width, name="embed", tensor="embed",
                         scale=self.embedding_scale)
        if self.side_dim:
            embedding.update(side_tensor="side.embed", side_width=self.side_dim * count)
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=default_schedule(count),
            embedding=PartSpec("token_embedding", embedding),
            final_norm=self._norm("final.norm"),
            lm_head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=self.width, name="lm_head",
                                             tied_to="embed")),
            max_position_embeddings=self.max_positions,
            stored_dtype=self.stored_dtype,
        )


__all__ = ["ARCHITECTURE", "RubuvikConfig"]
