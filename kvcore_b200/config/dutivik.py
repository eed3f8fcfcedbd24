"""Typed reader of a Dutivik model folder's config.json, and its description as parts.

Dutivik is a decoder whose layers read ONE layer norm (weight and bias) with both sub-layers and add their
sum to a 32-bit stream: ``h = norm1(x)``, ``x <- x + (mixer(h) + ff(h))``.  The embedded tokens are scaled;
the output head is the embedding table without that scale, behind a final layer norm.  Its keys:

    architecture     "Dutivik"
    vocab, width     vocabulary and stream width
    norm.eps         eps of every norm of the model
    embedding.scale  factor on the embedded tokens
    layers[i]        type ("gla" | "parallel"), mixer {...}, mlp (null | {kind "dense", ff}),
                     weights_of (optional): the layer runs layer j's tensors with a cache and state of its own

``gla``: gated linear attention, mixer {heads, dim, vdim, tau}; the inner size of the decay's projection is
the shape of tensor ``l<i>.mix.a1`` (or the key ``decay_rank`` where there are no tensors to ask).
``parallel``: two mixers side by side, mixer {left {...}, right {...}, left_scale, right_scale}.  ``left`` is
sliding-window attention {heads, kv_heads, dim, vdim, scale, mask {size}, rot {base, dims, scaling {factor}}}
with q and k turned in neighbouring pairs, then divided by their root mean square, and a sigmoid gate per
head; ``right`` is the gated delta rule {heads, kv_heads, dim, vdim, conv} behind a short convolution.
The feed-forward is ``down(silu(gate h) * up h)``.

Tensors: ``embed``, ``final.norm[.b]``, ``l<i>.norm1[.b]``, ``l<i>.mlp.{gate,up,down}``,
``l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}`` (gla), ``l<i>.mix.left.{q,k,v,g,o}`` and
``l<i>.mix.right.{q,k,v,g,o,b,a,A_log,dt_bias,norm,q.conv,k.conv,v.conv}`` (parallel).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .config_json import ConfigError
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .toposun import DEFAULT_MAX_POSITIONS, _need, _number, _positive_int

ARCHITECTURE = "Dutivik"


@dataclass(frozen=True)
class DutivikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple[Mapping[str, Any], ...]
    max_positions: int
    stored_dtype: str | None
    tensor_shapes: Mapping[str, tuple[int, ...]] | None = None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], tensor_shapes: Mapping[str, tuple[int, ...]] | None = None) -> "DutivikConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        return cls(
            vocab=_positive_int(raw, "vocab", "the model"),
            width=_positive_int(raw, "width", "the model"),
            eps=_number(_need(raw, "norm", "the model"), "eps", "norm"),
            embedding_scale=_number(_need(raw, "embedding", "the model"), "scale", "embedding"),
            layers=tuple(layers),
            max_positions=int(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
            stored_dtype=raw.get("dtype") or raw.get("torch_dtype"),
            tensor_shapes=tensor_shapes,
        )

    # ---- parts ---------------------------------------------------------------------------------
    def _norm(self, tensor: str) -> PartSpec:
        return PartSpec("layernorm", dict(size=self.width, eps=self.eps, name=tensor, tensor=tensor, bias=True,
                                          bias_tensor=tensor + ".b"))

    def _gla(self, index: int, m: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer"
        name = f"l{index}.mix"
        shape = (self.tensor_shapes or {}).get(f"{name}.a1")
        if shape is not None and len(shape) == 2:
            rank = int(shape[0])
        elif isinstance(m, Mapping) and "decay_rank" in m:
            rank = _positive_int(m, "decay_rank", where)
        else:
            raise ConfigError(f"config.json: the inner size of {where}'s decay projection is the shape of tensor "
                              f"{name}.a1; without tensors, give {where}.decay_rank")
        tau = _number(m, "tau", where)
        if not tau > 0:
            raise ConfigError(f"config.json: {where}.tau must be positive, got {tau}")
        return PartSpec("gated_linear_attention", dict(
            hidden_size=self.width, num_heads=_positive_int(m, "heads", where), head_dim=_positive_int(m, "dim", where),
            value_dim=_positive_int(m, "vdim", where), tau=tau, decay_rank=rank, eps=self.eps, name=name))

    def _left(self, index: int, m: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer.left"
        heads, kv_heads = _positive_int(m, "heads", where), _positive_int(m, "kv_heads", where)
        dim = _positive_int(m, "dim", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv_heads}")
        rot = m.get("rot") or {}
        rot_dims = _positive_int(rot, "dims", where + ".rot", minimum=0) if rot else 0
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim {dim}, got {rot_dims}")
        scaling = rot.get("scaling") if rot else None
        factor = _number(scaling, "factor", where + ".rot.scaling") if scaling else 1.0
        if not factor > 0:
            raise ConfigError(f"config.json: {where}.rot.scaling.factor must be positive, got {factor}")
        mask = m.get("mask")
        return PartSpec("gated_window_attention", dict(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
            value_dim=_positive_int(m, "vdim", where), scale=_number(m, "scale", where),
            window=_positive_int(mask, "size", where + ".mask") if mask else None,
            rot_dims=rot_dims, rot_base=_number(rot, "base", where + ".rot") if rot_dims else 1.0, rot_factor=factor,
            qk_norm=True, eps=self.eps, head_gate=True, name=f"l{index}.mix.left"))

    def _right(self, index: int, m: Mapping[str, Any]) -> PartSpec:
        where = f"layers[{index}].mixer.right"
        heads, kv_heads = _positive_int(m, "heads", where), _positive_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv_heads}")
        taps = _positive_int(m, "conv", where)
        if taps > 9:
            raise ConfigError(f"config.json: {where}.conv {taps} exceeds the 9 taps the convolution kernel takes")
        return PartSpec("gated_delta_rule", dict(
            hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=_positive_int(m, "dim", where),
            value_dim=_positive_int(m, "vdim", where), conv_taps=taps, eps=self.eps, name=f"l{index}.mix.right"))

    def _mixer(self, index: int, layer: Mapping[str, Any]) -> PartSpec:
        kind = _need(layer, "type", f"layers[{index}]")
        m = _need(layer, "mixer", f"layers[{index}]")
        where = f"layers[{index}].mixer"
        if kind == "gla":
            return self._gla(index, m)
        if kind == "parallel":
            return PartSpec("side_by_side", dict(
                hidden_size=self.width,
                members=(self._left(index, _need(m, "left", where)), self._right(index, _need(m, "right", where))),
                scales=(_number(m, "left_scale", where), _number(m, "right_scale", where)), name=f"l{index}.mix"))
        raise ConfigError(f"config.json: layers[{index}].type {kind!r} is not a mixer of this design")

    def _feed_forward(self, index: int, layer: Mapping[str, Any]) -> PartSpec | None:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        where = f"layers[{index}].mlp"
        kind = _need(mlp, "kind", where)
        if kind != "dense":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design")
        return PartSpec("swiglu", dict(hidden_size=self.width, intermediate_size=_positive_int(mlp, "ff", where),
                                       tensor_names={"gate": "gate", "up": "up", "down": "down"}, name=f"l{index}.mlp"))

    def _owner(self, index: int) -> int:
        """The layer whose tensors layer ``index`` runs."""
        seen = {index}
        while isinstance(self.layers[index], Mapping) and self.layers[index].get("weights_of") is not None:
            owner = self.layers[index]["weights_of"]
            if not isinstance(owner, int) or isinstance(owner, bool) or not 0 <= owner < len(self.layers):
                raise ConfigError(f"config.json: layers[{index}].weights_of {owner!r} names no layer")
            if owner in seen:
                raise ConfigError(f"config.json: layers[{index}].weights_of runs in a circle")
            seen.add(owner)
            index = owner
        return index

    def to_model_spec(self) -> ModelSpec:
        layers: list[LayerSpec] = []
        place: dict[int, int] = {}          # layer of config.json -> its place among the layers that hold tensors
        schedule = []
        for index, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{index}] is not an object")
            owner = self._owner(index)
            if owner != index:
                mine, theirs = dict(layer), dict(self.layers[owner])
                for entry in (mine, theirs):
                    entry.pop("weights_of", None)
                if mine != theirs:
                    raise ConfigError(f"config.json: layers[{index}] runs layer {owner}'s tensors but describes "
                                      "another layer")
            if owner not in place:
                source = self.layers[owner]
                place[owner] = len(layers)
                layers.append(LayerSpec(
                    prefix=f"l{owner}", block=PartSpec("parallel_residual"), mixer=self._mixer(owner, source),
                    feed_forward=self._feed_forward(owner, source), norms={"mixer_norm": self._norm(f"l{owner}.norm1")}))
            schedule.append(ScheduleEntry(layer=place[owner]))
        return ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=self.width, name="embed",
                                                       tensor="embed", scale=self.embedding_scale)),
            final_norm=self._norm("final.norm"),
            lm_head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=self.width, name="lm_head",
                                             tied_to="embed")),
            max_position_embeddings=self.max_positions,
            stored_dtype=self.stored_dtype,
        )


__all__ = ["ARCHITECTURE", "DutivikConfig"]
