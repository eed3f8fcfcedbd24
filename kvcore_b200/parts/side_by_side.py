"""Sliding-window attention with turned and normed q and k and a gate per head, and the mixer that runs several
mixers side by side on one input.

``GatedWindowAttention``: grouped-query attention whose key width and value width may differ.  The first
``rot_dims`` entries of every q and k head turn by the token's position in neighbouring pairs (entry 2i with
entry 2i+1, frequency ``rot_base^(-2i/rot_dims) / rot_factor``); after the turn every head is divided by its
root mean square (no weight); scores are ``q . k * scale`` over the last ``window`` positions (the token's own
included), ordinary softmax; head ``h``'s output is multiplied by ``sigmoid(W_g x)_h``.  Further mechanisms, each
a parameter: biases on q, k and v (``bias``); a sink per head that joins the softmax's denominator (``sink``); a
bias ``slope_h * (i - j)`` taken off the score of query ``i`` and key ``j`` with
``slope_h = 2^(-slope_exponent (h + 1) / heads)`` (``slope_exponent``); a query temperature, q times
``1 + coef * ln(floor((position + 1) / every) + 1)`` (``q_temp = (coef, every)``); value mixing
(``value_mix``): the ``"first"`` such layer of a model leaves its values of the step's tokens for the
``"later"`` ones, which cache ``(1 - lambda) v + lambda v_first`` with their own number ``lambda``.  A token's keys and
values are one cached row ``[k of all kv heads | v of all kv heads]``, so layers of any sizes share the page
pool's machinery, and pages wholly behind the window are handed back while the request lives.

``SideBySideMixers``: ``sum_i scale_i * mixer_i(x)`` for mixers of the ``ProjectedMixer`` form.  Their input
projections are rows of one matrix and their output projections columns of one matrix, so the step runs one
product in front of all of them and one behind, and the weighted sum is formed in that product's 32-bit
accumulators.  At most one member may keep pages; the members' per-request states lie one after the other in
one state row.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import PartSpec
from .base import MIXERS, CacheSpec, Mixer, StateSpec, WeightSlot
from .recurrent import ProjectedMixer, _round8
from .rope import rope_inverse_frequencies


class GatedWindowAttention(ProjectedMixer):
    graph_safe = True

    DEFAULT_TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "q_bias": "q.b", "k_bias": "k.b",
                            "v_bias": "v.b", "sink": "sink", "value_mix": "vmix"}

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, window: int | None, rot_dims: int, rot_base: float, rot_factor: float = 1.0,
                 qk_norm: bool = True, eps: float, head_gate: bool = True, name: str, bias: bool = False,
                 sink: bool = False, slope_exponent: float | None = None, q_temp: tuple | None = None,
                 value_mix: str | None = None, value_mix_key: str = "values_of_first_mixing_layer",
                 tensor_names: dict | None = None, dtype: torch.dtype, device: torch.device) -> None:
        if min(num_heads, num_kv_heads, head_dim, value_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} must be a positive multiple of num_kv_heads {num_kv_heads}")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
            raise ValueError(f"the turned entries must be an even number within head_dim {head_dim}, got {rot_dims}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive when set, got {window}")
        if value_dim > 512:
            raise ValueError(f"value_dim {value_dim} exceeds the attention kernels' value width of 512")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.window, self.eps = float(scale), None if window is None else int(window), float(eps)
        self.rot_dims, self.qk_norm, self.has_gate, self.name = int(rot_dims), bool(qk_norm), bool(head_gate), name
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.q_cols = self.num_heads * self.head_dim
        self.k_cols = self.num_kv_heads * self.head_dim
        self.v_cols = self.num_kv_heads * self.value_dim
        # one packed projection: q, k, v, then a column a head for the gate
        self.g_col = self.q_cols + self.k_cols + self.v_cols
        self.in_rows = _round8(self.g_col + (self.num_heads if self.has_gate else 0))
        self.out_cols = self.num_heads * self.value_dim
        self._allocate(dtype, device)
        self.inv_freq = None
        if self.rot_dims:
            table = rope_inverse_frequencies(self.rot_dims, rot_base, "linear", rot_factor)
            self.inv_freq = table if torch.device(device).type == "meta" else table.to(device)
        if value_mix not in (None, "first", "later"):
            raise ValueError(f"value_mix is None, 'first' or 'later', got {value_mix!r}")
        if q_temp is not None and (len(q_temp) != 2 or int(q_temp[1]) <= 0):
            raise ValueError(f"q_temp is (coef, every) with every > 0, got {q_temp!r}")
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        on_device = (lambda t: t) if torch.device(device).type == "meta" else (lambda t: t.to(device))
        self.in_bias = torch.zeros(self.in_rows, dtype=dtype, device=device) if bias else None
        self.sink = torch.empty(self.num_heads, dtype=torch.float32, device=device) if sink else None
        self.lam = torch.empty((), dtype=torch.float32, device=device) if value_mix else None
        self.slopes = None
        if slope_exponent is not None:
            heads = torch.arange(1, self.num_heads + 1, dtype=torch.float64)
            self.slopes = on_device(torch.exp2(-float(slope_exponent) * heads / self.num_heads).to(torch.float32))

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, 1, self.k_cols + self.v_cols, self.window)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        q, k, w = self.q_cols, self.k_cols, self.in_weight
        slots = [WeightSlot(self._tensor("q"), w[:q]), WeightSlot(self._tensor("k"), w[q:q + k]),
                 WeightSlot(self._tensor("v"), w[q + k:self.g_col]), WeightSlot(self._tensor("o"), self.o_weight)]
        if self.has_gate:
            slots.append(WeightSlot(self._tensor("g"), w[self.g_col:self.g_col + self.num_heads]))
        if self.in_bias is not None:
            b = self.in_bias
            slots += [WeightSlot(self._tensor("q_bias"), b[:q]), WeightSlot(self._tensor("k_bias"), b[q:q + k]),
                      WeightSlot(self._tensor("v_bias"), b[q + k:self.g_col])]
        if self.sink is not None:
            slots.append(WeightSlot(self._tensor("sink"), self.sink, init="zeros"))
        if self.lam is not None:      # the first mixing layer's number is a tensor of the model too, and unused
            slots.append(WeightSlot(self._tensor("value_mix"), self.lam, init="zeros"))
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        # a layer that mixes no values in may still carry the number it would mix them with
        return [self._tensor("value_mix")] if self.lam is None else []

    def mix_rows(self, rows, ctx, cache, out, scale: float = 1.0) -> None:
        tokens = rows.shape[0]
        table = ctx.block_table(cache.group)
        plane = cache.planes[0]                                # [pages, 1, page, k_cols + v_cols]
        num_pages, _, page, width = plane.shape
        values = rows[:, self.q_cols + self.k_cols:self.g_col]
        first = None
        if self.value_mix == "later":
            first = ctx.shared(self.value_mix_key, lambda: None)
            if first is None or first.shape != values.shape:
                raise RuntimeError(f"{self.name}: no layer in front has left values of this layer's sizes to mix in")
        K.turn_norm_kv_write(rows, self.inv_freq, self.rot_dims, ctx, table, plane, q_heads=self.num_heads,
                             k_heads=self.num_kv_heads, dim=self.head_dim, value_width=self.v_cols,
                             norm=self.qk_norm, eps=self.eps, write=cache.owner, q_temp=self.q_temp,
                             mix_values=first, mix_weight=self.lam if first is not None else None)
        if self.value_mix == "first":
            ctx.shared(self.value_mix_key, lambda: values)
        q = rows[:, : self.q_cols].unflatten(1, (self.num_heads, self.head_dim))
        # without a gate and without a scale the attention writes the rows of the output product itself
        direct = not self.has_gate and scale == 1.0
        o = K.attention_dims(
            q, plane, plane.view(-1)[self.k_cols:], table, ctx, value_heads=self.num_kv_heads,
            group=self.num_heads // self.num_kv_heads, maps=1, key_width=self.head_dim, value_width=self.value_dim,
            page_size=page, num_pages=num_pages, key_strides=(page * width, self.head_dim, width),
            value_strides=(page * width, self.value_dim, width), scale=self.scale, window=self.window,
            sink=self.sink, slopes=self.slopes, out_dtype=torch.float32,
            out=out.unflatten(1, (self.num_heads, self.value_dim)) if direct else None)
        if direct:
            return
        gate = rows[:, self.g_col:self.g_col + self.num_heads] if self.has_gate else None
        K.head_gate(o.view(tokens, self.num_heads, self.value_dim), gate, out, scale)


class SideBySideMixers(Mixer):
    def __init__(self, *, hidden_size: int, members: tuple, scales: tuple, name: str,
                 dtype: torch.dtype, device: torch.device) -> None:
        if not members or len(members) != len(scales):
            raise ValueError("side-by-side mixers need one scale per member")
        self.hidden_size, self.name = int(hidden_size), name
        self.scales = tuple(float(s) for s in scales)
        self.members: list[ProjectedMixer] = []
        for spec in members:
            if not isinstance(spec, PartSpec):
                raise ValueError("the members of side-by-side mixers are part specs")
            member = MIXERS.build(spec, dtype=dtype, device=device)
            if not isinstance(member, ProjectedMixer) or member.in_bias is not None:
                raise ValueError(f"mixer kind {spec.kind!r} cannot share its projections with others")
            self.members.append(member)
        if sum(1 for m in self.members if m.cache_spec() is not None) > 1:
            raise ValueError("at most one of the mixers side by side may keep pages")
        self.in_weight = torch.zeros(sum(m.in_rows for m in self.members), self.hidden_size, dtype=dtype, device=device)
        self.o_weight = torch.empty(self.hidden_size, sum(m.out_cols for m in self.members), dtype=dtype, device=device)
        row = col = state = 0
        self.sections = []
        for member in self.members:
            member.adopt(self.in_weight[row:row + member.in_rows], self.o_weight[:, col:col + member.out_cols], state)
            self.sections.append((row, col))
            row, col = row + member.in_rows, col + member.out_cols
            spec = member.state_spec()
            if spec is not None:
                if spec.dtype != torch.float32 or len(spec.shape) != 1:
                    raise ValueError("mixers side by side keep their states as 32-bit rows")
                state += spec.shape[0]
        self.state_floats = state

    @property
    def graph_safe(self) -> bool:
        return all(member.graph_safe for member in self.members)

    def cache_spec(self) -> CacheSpec | None:
        return next((m.cache_spec() for m in self.members if m.cache_spec() is not None), None)

    def state_spec(self) -> StateSpec | None:
        return StateSpec((self.state_floats,), torch.float32) if self.state_floats else None

    def weight_slots(self) -> list[WeightSlot]:
        return [slot for member in self.members for slot in member.weight_slots()]

    def ignorable_tensor_names(self) -> list[str]:
        return [name for member in self.members for name in member.ignorable_tensor_names()]

    def finalize_weights(self) -> None:
        for member in self.members:
            member.finalize_weights()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        rows = K.linear(x, self.in_weight)
        out = torch.empty((x.shape[0], self.o_weight.shape[1]), dtype=rows.dtype, device=rows.device)
        for member, scale, (row, col) in zip(self.members, self.scales, self.sections):
            member.mix_rows(rows[:, row:row + member.in_rows], ctx, cache, out[:, col:col + member.out_cols], scale)
        return K.linear(out, self.o_weight)


MIXERS.register("gated_window_attention", GatedWindowAttention)
MIXERS.register("side_by_side", SideBySideMixers)

__all__ = ["GatedWindowAttention", "SideBySideMixers"]
