"""Mixture of experts as a feed-forward part: a router picks ``top_k`` of ``num_experts`` small gated
feed-forwards per token; an optional shared expert runs for every token.

    z = router x                      (32-bit logits; the router matrix is kept in 32-bit)
    s = sigmoid(z)  or  softmax(z)    (``score``)
    chosen = the top_k largest s; weights = their s, divided by their sum if ``renormalize``
             ``choice_correction``: the choice goes by ``s + c`` with a tensor ``c [experts]``, the weights stay
             the chosen experts' ``s``; ``group_count`` / ``group_keep``: the experts form ``group_count`` equal
             groups of neighbours, a group's score is its largest choice score, and only experts of the
             ``group_keep`` best groups can be chosen; ``weight_scale`` multiplies the weights
    y = sum over chosen e of  expert_e(w_e * x)        (``weight_on="input"``)
                         or   w_e * expert_e(x)        (``weight_on="output"``)
    y += sigmoid(g . x) * shared(x)   (``shared`` given; ``shared_gate`` False: plain sum)

    expert(a) = down(silu(gate a) * (up a)), no biases.

The experts' matrices are stacked ``[E, 2F, K]`` (gate rows, then up rows) and ``[E, K, F]``; the
(token, expert) pairs are grouped by expert on the device and the two products run as grouped
products over that order, so the launches depend on the batch's shape only.  The shared expert is any
registered feed-forward part.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, FeedForward, WeightSlot


class RoutedExperts(FeedForward):
    DEFAULT_TENSOR_NAMES = {
        "router": "router", "shared_gate": "shared_gate", "correction": "correction",
        # expert tensors: formatted with the expert's index
        "gate": "experts.{index}.gate_proj.weight", "up": "experts.{index}.up_proj.weight",
        "down": "experts.{index}.down_proj.weight",
    }

    def __init__(self, *, hidden_size: int, num_experts: int, top_k: int, expert_size: int, name: str,
                 score: str = "sigmoid", renormalize: bool = False, weight_on: str = "input",
                 shared: PartSpec | None = None, shared_gate: bool = False, weight_scale: float = 1.0,
                 choice_correction: bool = False, group_count: int = 1, group_keep: int = 1,
                 tensor_names: dict | None = None, dtype: torch.dtype, device: torch.device) -> None:
        self.hidden_size, self.num_experts = int(hidden_size), int(num_experts)
        self.top_k, self.expert_size = int(top_k), int(expert_size)
        if not 0 < self.top_k <= self.num_experts:
            raise ValueError(f"top_k {top_k} must lie in [1, num_experts {num_experts}]")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {score!r}")
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got {weight_on!r}")
        self.score, self.renormalize, self.weight_on = score, bool(renormalize), weight_on
        self.weight_scale, self.group_count, self.group_keep = float(weight_scale), int(group_count), int(group_keep)
        if (self.group_count <= 0 or self.num_experts % self.group_count or not 0 < self.group_keep <= self.group_count
                or self.group_keep * (self.num_experts // self.group_count) < self.top_k):
            raise ValueError(f"{group_keep} of {group_count} equal groups of {num_experts} experts must hold top_k {top_k}")
        self.name = name
        self.tensor_names = dict(self.DEFAULT_TENSOR_NAMES)
        self.tensor_names.update(tensor_names or {})
        experts, ff, hidden = self.num_experts, self.expert_size, self.hidden_size
        self.router_weight = torch.empty(experts, hidden, dtype=torch.float32, device=device)
        self.correction = torch.empty(experts, dtype=torch.float32, device=device) if choice_correction else None
        self.gate_up_weight = torch.empty(experts, 2 * ff, hidden, dtype=dtype, device=device)
        self.down_weight = torch.empty(experts, hidden, ff, dtype=dtype, device=device)
        self.shared = None if shared is None else FEED_FORWARDS.build(shared, dtype=dtype, device=device)
        if shared_gate and self.shared is None:
            raise ValueError("a shared gate needs a shared expert")
        self.shared_gate_weight = (torch.empty(1, hidden, dtype=torch.float32, device=device)
                                   if shared_gate else None)

    @property
    def graph_safe(self) -> bool:
        return self.shared is None or self.shared.graph_safe

    def _tensor(self, key: str, index: int | None = None) -> str:
        return f"{self.name}.{self.tensor_names[key].format(index=index)}"

    def weight_slots(self) -> list[WeightSlot]:
        ff = self.expert_size
        slots = [WeightSlot(self._tensor("router"), self.router_weight)]
        if self.correction is not None:
            slots.append(WeightSlot(self._tensor("correction"), self.correction, init="zeros"))
        for e in range(self.num_experts):
            slots += [
                WeightSlot(self._tensor("gate", e), self.gate_up_weight[e, :ff]),
                WeightSlot(self._tensor("up", e), self.gate_up_weight[e, ff:]),
                WeightSlot(self._tensor("down", e), self.down_weight[e]),
            ]
        if self.shared is not None:
            slots += self.shared.weight_slots()
        if self.shared_gate_weight is not None:
            slots.append(WeightSlot(self._tensor("shared_gate"), self.shared_gate_weight))
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        return [] if self.shared is None else self.shared.ignorable_tensor_names()

    def finalize_weights(self) -> None:
        if self.shared is not None:
            self.shared.finalize_weights()

    def prepare(self, x: torch.Tensor, ctx):
        """The router and the grouping of the pairs by expert, ahead of ``forward``: a block that has other
        work to launch in between (its mixer) calls this first, so that what the host must know of the
        grouping has arrived by the time ``forward`` asks for it."""
        routed = K.moe_route(x, self.router_weight, self.top_k, score=self.score,
                             renormalize=self.renormalize, gate_rows=self.shared_gate_weight,
                             correction=self.correction, group_count=self.group_count, group_keep=self.group_keep,
                             weight_scale=self.weight_scale)
        grouping = None
        if K.moe_path(x, x.shape[0] * self.top_k, self.expert_size) == "library":
            grouping = K.moe_group(routed[0], self.num_experts, for_library=True)
        return routed, grouping

    def forward(self, x: torch.Tensor, ctx, prepared=None) -> torch.Tensor:
        (ids, weights, gates), grouping = prepared if prepared is not None else self.prepare(x, ctx)
        pairs = K.moe_experts(x, ids, weights, self.gate_up_weight, self.down_weight,
                              weight_on_input=self.weight_on == "input", grouping=grouping)
        shared = None if self.shared is None else self.shared.forward(x, ctx)
        return K.moe_combine(pairs, x.shape[0], self.top_k, shared, gates)


FEED_FORWARDS.register("routed_experts", RoutedExperts)

__all__ = ["RoutedExperts"]
