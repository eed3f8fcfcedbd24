"""RMS normalisation with the residual sum folded in, and layer normalisation over a 32-bit stream.

Formula as the reference computes it (kvcore/model/layer/rmsnorm.py:19-26): the optional
residual is added first and becomes the new residual; then in 32-bit
``y = x * rsqrt(mean(x^2) + eps)`` and ``out = (weight * y)`` cast to the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import NORMS, Norm, WeightSlot


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, *, size: int, eps: float, name: str, dtype: torch.dtype, device: torch.device):
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.weight = torch.empty(self.size, dtype=dtype, device=device)

    def _rebind(self, tensor: torch.Tensor) -> None:
        self.weight = tensor

    def weight_slots(self) -> list[WeightSlot]:
        return [
            WeightSlot(f"{self.name}.weight", self.weight, init="ones", keep_f32=True, rebind=self._rebind)
        ]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rmsnorm(x, self.weight, self.eps)

    def forward_residual(self, h: torch.Tensor, residual: torch.Tensor):
        return K.add_rmsnorm(h, residual, self.weight, self.eps), residual

    def as_rms_scale(self):
        return self.weight, self.eps


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` with the biased variance, statistics in 32-bit.

    It reads rows of the activation type or of a 32-bit residual stream and writes the activation type, so a
    block that keeps its stream in 32-bit normalises it without a copy.  ``tensor`` is the weight's full
    checkpoint name (default ``<name>.weight``); ``bias`` adds ``<name>.bias`` (or ``bias_tensor``)."""

    graph_safe = True

    def __init__(self, *, size: int, eps: float, name: str, tensor: str | None = None, bias: bool = False,
                 bias_tensor: str | None = None, dtype: torch.dtype, device: torch.device):
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.dtype = dtype
        self.tensor = tensor or f"{name}.weight"
        self.bias_tensor = bias_tensor or f"{name}.bias"
        self.weight = torch.empty(self.size, dtype=dtype, device=device)
        self.bias = torch.empty(self.size, dtype=dtype, device=device) if bias else None

    def weight_slots(self) -> list[WeightSlot]:
        slots = [WeightSlot(self.tensor, self.weight, init="ones")]
        if self.bias is not None:
            slots.append(WeightSlot(self.bias_tensor, self.bias, init="zeros"))
        return slots

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.layer_norm(x, self.weight, self.bias, self.eps, out_dtype=self.dtype)

    def forward_residual(self, h: torch.Tensor, residual: torch.Tensor):
        residual = K.stream_add(residual, h) if residual.dtype == torch.float32 else residual.add_(h)
        return self.forward(residual), residual


class RMSNormStream(Norm):
    """``x * rsqrt(mean(x^2) + eps) * weight`` over rows of a 32-bit residual stream (or of the activation
    type), written in the activation type; statistics and scaling in 32-bit.  ``tensor`` is the weight's full
    checkpoint name (default ``<name>.weight``).

    ``offset`` and ``multiplier``: the factor is ``(stored + offset) * multiplier`` for the tensor ``stored`` of
    the checkpoint (a weight stored around zero has ``offset`` 1; a norm whose result enters a sum with a
    constant factor carries it as ``multiplier``).  The factor is then formed once, in 32-bit, and stays 32-bit
    whatever the activation type: ``1 + w`` has more digits than the stored ``w``."""

    graph_safe = True

    def __init__(self, *, size: int, eps: float, name: str, tensor: str | None = None, offset: float = 0.0,
                 multiplier: float = 1.0, dtype: torch.dtype, device: torch.device):
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.dtype = dtype
        self.tensor = tensor or f"{name}.weight"
        self.offset, self.multiplier = float(offset), float(multiplier)
        self.derived = self.offset != 0.0 or self.multiplier != 1.0
        self.stored = torch.empty(self.size, dtype=dtype, device=device)
        self.weight = torch.empty(self.size, dtype=torch.float32, device=device) if self.derived else self.stored

    def weight_slots(self) -> list[WeightSlot]:
        return [WeightSlot(self.tensor, self.stored, init="zeros" if self.offset == 1.0 else "ones")]

    def finalize_weights(self) -> None:
        if self.derived:
            self.weight.copy_((self.stored.to(torch.float32) + self.offset) * self.multiplier)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rms_norm_shift(x, self.weight, self.eps, self.dtype)

    def forward_residual(self, h: torch.Tensor, residual: torch.Tensor):
        residual = K.stream_add(residual, h) if residual.dtype == torch.float32 else residual.add_(h)
        return self.forward(residual), residual

    def as_rms_scale(self):
        return self.weight, self.eps


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("rmsnorm_stream", RMSNormStream)
NORMS.register("layernorm", LayerNorm)

__all__ = ["LayerNorm", "RMSNorm", "RMSNormStream"]
