"""Mixers that keep a matrix-valued state per request and head instead of cached keys and values, and the
interface that lets several mixers stand side by side on one input.

``ProjectedMixer``: a mixer of the form ``W_o · f(W_in x)`` that can run on rows somebody else has projected
and write its result in front of the output projection into columns somebody else owns.  A mixer that holds
several of them (``side_by_side``) then needs one input product and one output product for all, and their sum
is formed in the output product's 32-bit accumulators.

``GatedLinearAttention``: per head ``S_t = diag(a_t) S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` with a decay
per key channel ``a_t = sigmoid(W_a2 (W_a1 x) + b)^(1/tau)`` and ``q`` scaled by ``dim^(-1/2)``; each head's
``o`` gets an RMS norm with one weight for all heads and is multiplied by ``silu(W_g x)``.

``GatedDeltaRule``: q and k (``num_kv_heads`` heads shared by groups of value heads) and v pass a short causal
convolution over time and SiLU; q and k become unit vectors (q times ``dim^(-1/2)``); per head
``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q`` with ``beta = sigmoid(W_b x)`` and
``g = exp(-exp(A_log) softplus(W_a x + dt_bias))``; ``o`` gets an RMS norm with one weight for all heads and is
multiplied by ``silu(W_g x)``.  The state of a request is ``S`` and the last ``taps - 1`` inputs of the
convolution.  Both mixers keep ``S`` column by column (``[heads, value_dim, head_dim]``).

``LightningAttention``: per head ``S_t = a S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` with one fixed decay
``a`` a head (a constant of the model) and ``q``, ``k``, ``v`` passed through SiLU; the heads' read-outs are
RMS-normed together (one weight over all heads' values) and multiplied by ``sigmoid(W_g x)``.

Decays, step sizes, unit norms, the state, the read-out and the norm behind it are 32-bit whatever the
activation type.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import MIXERS, Mixer, StateSpec, WeightSlot


def _round8(n: int) -> int:
    return (n + 7) & ~7


def _round4(n: int) -> int:
    """State rows are whole 16-byte pieces, so that every request's (and every member's) state starts on a
    16-byte boundary and the state kernels move it in such pieces."""
    return (n + 3) & ~3


class ProjectedMixer(Mixer):
    """``forward(x) = W_o · mix_rows(W_in x)``.  Subclasses set ``in_rows`` (rows of ``W_in``, a multiple of 8 so
    that the rows of several mixers can share one matrix with every section on a 16-byte boundary) and
    ``out_cols`` (columns of ``W_o``) before calling ``_allocate``; ``state_offset`` is where this mixer's
    state begins in its request's state row (a mixer that holds several gives each its place)."""

    hidden_size: int
    in_rows: int
    out_cols: int
    state_offset = 0
    in_bias = None            # a bias on the input projection (a mixer with one does not share its matrices)

    def _allocate(self, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype = dtype
        self.in_weight = torch.zeros(self.in_rows, self.hidden_size, dtype=dtype, device=device)
        self.o_weight = torch.empty(self.hidden_size, self.out_cols, dtype=dtype, device=device)

    def adopt(self, in_weight: torch.Tensor, o_weight: torch.Tensor, state_offset: int) -> None:
        """Take rows of a shared input matrix and columns of a shared output matrix (before weights are
        loaded) in place of the mixer's own."""
        if tuple(in_weight.shape) != (self.in_rows, self.hidden_size) or tuple(o_weight.shape) != (self.hidden_size, self.out_cols):
            raise ValueError("the shared matrices do not have this mixer's sizes")
        self.in_weight, self.o_weight, self.state_offset = in_weight, o_weight, int(state_offset)

    def mix_rows(self, rows: torch.Tensor, ctx, cache, out: torch.Tensor, scale: float = 1.0) -> None:
        """``rows [T, in_rows]`` (a view of projected rows) -> ``out [T, out_cols]`` (a view), times ``scale``."""
        raise NotImplementedError

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        rows = K.linear(x, self.in_weight, self.in_bias)
        out = torch.empty((x.shape[0], self.out_cols), dtype=rows.dtype, device=rows.device)
        self.mix_rows(rows, ctx, cache, out)
        return K.linear(out, self.o_weight)


class GatedLinearAttention(ProjectedMixer):
    graph_safe = True

    DEFAULT_TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2",
                            "a2_bias": "a2.b"}

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, tau: float,
                 decay_rank: int, eps: float, name: str, tensor_names: dict | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        if min(num_heads, head_dim, value_dim, decay_rank) <= 0 or not tau > 0:
            raise ValueError("gated linear attention needs positive heads, sizes, decay rank and tau")
        if head_dim > 512:
            raise ValueError(f"head_dim {head_dim} exceeds the state kernel's 512 key channels")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.value_dim, self.decay_rank = int(head_dim), int(value_dim), int(decay_rank)
        self.tau, self.eps, self.name = float(tau), float(eps), name
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.qk_cols, self.v_cols = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        # one packed projection: q, k, v, the gate, the decay's inner projection
        self.a1_col = 2 * self.qk_cols + 2 * self.v_cols
        self.in_rows = _round8(self.a1_col + self.decay_rank)
        self.out_cols = self.v_cols
        self._allocate(dtype, device)
        self.a2_weight = torch.empty(self.qk_cols, self.decay_rank, dtype=dtype, device=device)
        self.a2_bias = torch.empty(self.qk_cols, dtype=dtype, device=device)
        self.norm_weight = torch.empty(self.value_dim, dtype=dtype, device=device)

    def state_spec(self) -> StateSpec:
        return StateSpec((_round4(self.num_heads * self.head_dim * self.value_dim),), torch.float32)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        qk, v, a1 = self.qk_cols, self.v_cols, self.a1_col
        w = self.in_weight
        return [
            WeightSlot(self._tensor("q"), w[:qk]), WeightSlot(self._tensor("k"), w[qk:2 * qk]),
            WeightSlot(self._tensor("v"), w[2 * qk:2 * qk + v]), WeightSlot(self._tensor("g"), w[2 * qk + v:a1]),
            WeightSlot(self._tensor("a1"), w[a1:a1 + self.decay_rank]),
            WeightSlot(self._tensor("a2"), self.a2_weight), WeightSlot(self._tensor("a2_bias"), self.a2_bias),
            WeightSlot(self._tensor("norm"), self.norm_weight, init="ones"),
            WeightSlot(self._tensor("o"), self.o_weight),
        ]

    def mix_rows(self, rows, ctx, cache, out, scale: float = 1.0) -> None:
        qk, v, a1 = self.qk_cols, self.v_cols, self.a1_col
        z = K.linear(rows[:, a1:a1 + self.decay_rank], self.a2_weight, self.a2_bias)
        o = K.gla_scan(rows[:, :qk], rows[:, qk:2 * qk], rows[:, 2 * qk:2 * qk + v], z, cache.state, ctx,
                       heads=self.num_heads, dim=self.head_dim, value_dim=self.value_dim,
                       q_scale=self.head_dim ** -0.5, tau=self.tau, state_offset=self.state_offset)
        K.gated_rms_norm(o, rows[:, 2 * qk + v:a1], self.norm_weight, self.eps, out, scale)


class GatedDeltaRule(ProjectedMixer):
    graph_safe = True
    UNIT_EPS = 1e-6       # q and k become x / sqrt(sum(x^2) + UNIT_EPS)

    DEFAULT_TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "b": "b", "a": "a",
                            "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "A_log": "A_log",
                            "dt_bias": "dt_bias"}

    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 conv_taps: int, eps: float, name: str, tensor_names: dict | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        if min(num_heads, num_kv_heads, head_dim, value_dim) <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} must be a positive multiple of num_kv_heads {num_kv_heads}")
        if not 1 <= conv_taps <= 9:
            raise ValueError(f"the short convolution has 1 to 9 taps, got {conv_taps}")
        if head_dim > 512:
            raise ValueError(f"head_dim {head_dim} exceeds the state kernel's 512 key channels")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim, self.conv_taps = int(head_dim), int(value_dim), int(conv_taps)
        self.eps, self.name = float(eps), name
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.qk_cols, self.v_cols = self.num_kv_heads * self.head_dim, self.num_heads * self.value_dim
        self.channels = 2 * self.qk_cols + self.v_cols            # what passes the convolution: q, k, v
        # one packed projection: q, k, v, the gate, then a column a head for beta and for the step size
        self.b_col = self.channels + self.v_cols
        self.a_col = self.b_col + self.num_heads
        self.in_rows = _round8(self.a_col + self.num_heads)
        self.out_cols = self.v_cols
        self._allocate(dtype, device)
        self.taps = torch.empty(self.channels, self.conv_taps, dtype=dtype, device=device)
        self.a_log = torch.empty(self.num_heads, dtype=dtype, device=device)
        self.dt_bias = torch.empty(self.num_heads, dtype=dtype, device=device)
        self.norm_weight = torch.empty(self.value_dim, dtype=dtype, device=device)
        self.matrix_floats = self.num_heads * self.head_dim * self.value_dim

    def state_spec(self) -> StateSpec:
        return StateSpec((_round4(self.matrix_floats + self.channels * (self.conv_taps - 1)),), torch.float32)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        qk, ch, w, heads = self.qk_cols, self.channels, self.in_weight, self.num_heads
        return [
            WeightSlot(self._tensor("q"), w[:qk]), WeightSlot(self._tensor("k"), w[qk:2 * qk]),
            WeightSlot(self._tensor("v"), w[2 * qk:ch]), WeightSlot(self._tensor("g"), w[ch:self.b_col]),
            WeightSlot(self._tensor("b"), w[self.b_col:self.a_col]),
            WeightSlot(self._tensor("a"), w[self.a_col:self.a_col + heads]),
            WeightSlot(self._tensor("q_conv"), self.taps[:qk]), WeightSlot(self._tensor("k_conv"), self.taps[qk:2 * qk]),
            WeightSlot(self._tensor("v_conv"), self.taps[2 * qk:]),
            WeightSlot(self._tensor("A_log"), self.a_log, init="zeros"),
            WeightSlot(self._tensor("dt_bias"), self.dt_bias, init="zeros"),
            WeightSlot(self._tensor("norm"), self.norm_weight, init="ones"),
            WeightSlot(self._tensor("o"), self.o_weight),
        ]

    def mix_rows(self, rows, ctx, cache, out, scale: float = 1.0) -> None:
        sizes = dict(heads=self.num_heads, kv_heads=self.num_kv_heads, dim=self.head_dim, value_dim=self.value_dim)
        prepared = K.conv_prepare(rows, self.taps, cache.state, ctx, self.a_log, self.dt_bias, b_col=self.b_col,
                                  a_col=self.a_col, q_scale=self.head_dim ** -0.5, unit_eps=self.UNIT_EPS,
                                  state_offset=self.state_offset + self.matrix_floats, **sizes)
        o = K.delta_scan(prepared, cache.state, ctx, state_offset=self.state_offset, **sizes)
        K.gated_rms_norm(o, rows[:, self.channels:self.b_col], self.norm_weight, self.eps, out, scale)


class LightningAttention(ProjectedMixer):
    graph_safe = True

    DEFAULT_TENSOR_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, *, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: tuple,
                 eps: float, name: str, q_scale: float = 1.0, tensor_names: dict | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        if min(num_heads, head_dim, value_dim) <= 0 or len(decay) != num_heads:
            raise ValueError("lightning attention needs positive heads and sizes and one decay a head")
        if head_dim > 512:
            raise ValueError(f"head_dim {head_dim} exceeds the state kernel's 512 key channels")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.eps, self.name, self.q_scale = float(eps), name, float(q_scale)
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        self.qk_cols, self.v_cols = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        # one packed projection: q, k, v, the gate
        self.in_rows = _round8(2 * self.qk_cols + 2 * self.v_cols)
        self.out_cols = self.v_cols
        self._allocate(dtype, device)
        self.norm_weight = torch.empty(self.v_cols, dtype=dtype, device=device)
        table = torch.tensor([float(a) for a in decay], dtype=torch.float32)
        self.decay = table if torch.device(device).type == "meta" else table.to(device)

    def state_spec(self) -> StateSpec:
        return StateSpec((_round4(self.num_heads * self.head_dim * self.value_dim),), torch.float32)

    def _tensor(self, key: str) -> str:
        return f"{self.name}.{self.tensor_names[key]}"

    def weight_slots(self) -> list[WeightSlot]:
        qk, v, w = self.qk_cols, self.v_cols, self.in_weight
        return [
            WeightSlot(self._tensor("q"), w[:qk]), WeightSlot(self._tensor("k"), w[qk:2 * qk]),
            WeightSlot(self._tensor("v"), w[2 * qk:2 * qk + v]), WeightSlot(self._tensor("g"), w[2 * qk + v:2 * qk + 2 * v]),
            WeightSlot(self._tensor("norm"), self.norm_weight, init="ones"),
            WeightSlot(self._tensor("o"), self.o_weight),
        ]

    def mix_rows(self, rows, ctx, cache, out, scale: float = 1.0) -> None:
        qk, v = self.qk_cols, self.v_cols
        o = K.lightning_scan(rows[:, :qk], rows[:, qk:2 * qk], rows[:, 2 * qk:2 * qk + v], self.decay, cache.state, ctx,
                             heads=self.num_heads, dim=self.head_dim, value_dim=self.value_dim, q_scale=self.q_scale,
                             state_offset=self.state_offset)
        # one norm over all heads' values: a single "head" as wide as the read-out
        K.gated_rms_norm(o.view(o.shape[0], 1, v), rows[:, 2 * qk + v:2 * qk + 2 * v], self.norm_weight, self.eps,
                         out, scale, gate_act="sigmoid")


MIXERS.register("gated_linear_attention", GatedLinearAttention)
MIXERS.register("lightning_attention", LightningAttention)
MIXERS.register("gated_delta_rule", GatedDeltaRule)

__all__ = ["GatedDeltaRule", "GatedLinearAttention", "LightningAttention", "ProjectedMixer"]
