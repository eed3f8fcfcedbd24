"""Arrangements of one layer: pre-norm mixer and feed-forward in sequence on a deferred residual, side
by side on a 32-bit stream, or in sequence on a 32-bit stream with a norm on both sides of each.

As the reference's decoder layer (kvcore/model/models/llama3.py:124-142): the running
``residual`` and the last sub-layer output ``h`` stay separate and are summed inside the
next norm; the first block starts with ``residual = h``.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import LayerSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, StateSpec, Summed, WeightSlot


class PreNormResidualBlock(Block):
    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.mixer_norm = NORMS.build(layer.norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward_norm = NORMS.build(layer.norms["feed_forward_norm"], dtype=dtype, device=device)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def weight_slots(self) -> list[WeightSlot]:
        slots: list[WeightSlot] = []
        for part in self.parts():
            slots += part.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        names: list[str] = []
        for part in self.parts():
            names += part.ignorable_tensor_names()
        return names

    def finalize_weights(self) -> None:
        for part in self.parts():
            part.finalize_weights()

    def forward(self, h, residual, ctx, cache):
        # A part that can take its input before the norm (and fold the norm into its first matrix
        # product, the residual sum into its last) gets it that way; otherwise the norm runs as a
        # step of its own.  ``h`` may be ``Summed``: the part in front added its output already.
        scale, prenorm = self.mixer_norm.as_rms_scale(), getattr(self.mixer, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            a, residual = prenorm(h, residual, scale, ctx, cache)
        else:
            if isinstance(h, Summed):
                x = self.mixer_norm.forward(residual)
            elif residual is None:
                residual = h
                x = self.mixer_norm.forward(h)
            else:
                x, residual = self.mixer_norm.forward_residual(h, residual)
            a = self.mixer.forward(x, ctx, cache)
        scale, prenorm = self.feed_forward_norm.as_rms_scale(), getattr(self.feed_forward, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            h, residual = prenorm(a, residual, scale, ctx)
        else:
            if isinstance(a, Summed):
                x = self.feed_forward_norm.forward(residual)
            else:
                x, residual = self.feed_forward_norm.forward_residual(a, residual)
            h = self.feed_forward.forward(x, ctx)
        return h, residual


class ParallelResidualBlock(Block):
    """Mixer and feed-forward side by side on one stream: ``x <- x + (mixer(norm_a(x)) + ff(norm_b(x)))``,
    both norms reading the same ``x``.  The stream ``x`` is kept in 32-bit whatever the activation type:
    the two sub-layer outputs are added to each other and then to the stream in 32-bit by one kernel.
    A layer without a feed-forward (``layer.feed_forward is None``) adds the mixer alone.  A layer whose
    norms name no ``feed_forward_norm`` has one norm, and both sub-layers read its output:
    ``h = norm(x)``, ``x <- x + (mixer(h) + ff(h))``.

    In the ``(h, residual)`` pair that runs through the blocks this block returns ``(Summed, stream)``."""

    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.mixer_norm = NORMS.build(layer.norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            if "feed_forward_norm" in layer.norms:
                self.feed_forward_norm = NORMS.build(layer.norms["feed_forward_norm"], dtype=dtype, device=device)
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
                     if p is not None)

    graph_safe = PreNormResidualBlock.graph_safe
    weight_slots = PreNormResidualBlock.weight_slots
    ignorable_tensor_names = PreNormResidualBlock.ignorable_tensor_names
    finalize_weights = PreNormResidualBlock.finalize_weights

    def forward(self, h, residual, ctx, cache):
        if residual is None:                       # the embedded tokens start the stream
            stream = K.stream_add(h)
        else:
            stream = residual if residual.dtype == torch.float32 else K.stream_add(residual)
            if not isinstance(h, Summed):          # a block in front left its last output unsummed
                stream = K.stream_add(stream, h)
        # Both sub-layers read the same stream, so a feed-forward that has something to get ready (a
        # ``prepare(x, ctx)`` whose result ``forward`` takes: a router whose grouping the host must see)
        # does that ahead of the mixer's launches, and nothing waits for it later.
        fx = prepared = mx = None
        if self.feed_forward is not None:
            fx = mx = (self.feed_forward_norm or self.mixer_norm).forward(stream)
            prepare = getattr(self.feed_forward, "prepare", None)
            prepared = None if prepare is None else prepare(fx, ctx)
        if mx is None or self.feed_forward_norm is not None:
            mx = self.mixer_norm.forward(stream)
        a = self.mixer.forward(mx, ctx, cache)
        f = None
        if self.feed_forward is not None:
            f = (self.feed_forward.forward(fx, ctx) if prepared is None
                 else self.feed_forward.forward(fx, ctx, prepared))
        return Summed(None), K.stream_add(stream, a, f)


class SandwichResidualBlock(Block):
    """A norm before and after each sub-layer on one 32-bit stream:
    ``x <- x + norm_b(mixer(norm_a(x)))`` and then ``x <- x + norm_d(ff(norm_c(x)))`` (a layer may have no
    feed-forward).  The four norms are RMS scales (``as_rms_scale``), so each pair of steps around a sub-layer
    is one kernel: norm (+ token shift) in front, norm + sum (+ depth average) behind.

    Two optional mechanisms, each with its constants as parameters:

    * ``token_shift`` (the name of a ``[width]`` tensor): what the mixer reads, ``y = norm_a(x)``, becomes
      ``y_t + (y_{t-1} - y_t) * shift`` with ``y_{t-1}`` the unshifted normed row of the token in front (zeros
      for a request's first token).  The last normed row of a request is per-request state of the block
      (``state_spec``), kept in 32-bit.
    * ``depth_average`` (the name of a ``[depth + 1]`` tensor) with ``depth`` results in front of this layer
      (the embedded tokens and the results of the layers before it) out of ``depth_slots`` in the model: the
      layer's result ``X`` joins them, and what goes on to the next layer is
      ``sum_j c[j] * X_j + c[depth] * X``.  The results of a step live in one ``[depth_slots, T, width]``
      32-bit tensor shared through the step's context.

    * ``token_side`` (``dict(dim, index, eps, scale, name)``): behind the last sub-layer the layer adds an input
      of the token itself.  The model's embedding holds a side table with ``dim`` entries per token and layer;
      with ``e`` this layer's entries (columns ``[index * dim, (index + 1) * dim)`` of the token's row),
      ``y = P (gelu_tanh(G x) * e)`` reads the stream ``x`` itself, and
      ``x <- x + scale * y * rsqrt(mean(y^2) + eps) * w``.  Tensors ``<name>.gate`` (``G [dim, width]``),
      ``<name>.proj`` (``P [width, dim]``) and ``<name>.norm`` (``w [width]``).

    In the ``(h, residual)`` pair that runs through the blocks this block returns ``(Summed, stream)``."""

    def __init__(self, *, layer: LayerSpec, hidden_size: int, token_shift: str | None = None,
                 depth_average: str | None = None, depth: int = 0, depth_slots: int = 0,
                 token_side: dict | None = None, unused_tensors: tuple = (), dtype: torch.dtype,
                 device: torch.device) -> None:
        self.hidden_size = int(hidden_size)
        # names a checkpoint may carry for this layer although the layer has no use for them
        self.unused_tensors = tuple(unused_tensors)
        self.dtype = dtype
        norms = layer.norms
        self.mixer_norm = NORMS.build(norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer_out_norm = NORMS.build(norms["mixer_out_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_out_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = NORMS.build(norms["feed_forward_norm"], dtype=dtype, device=device)
            self.feed_forward_out_norm = NORMS.build(norms["feed_forward_out_norm"], dtype=dtype, device=device)
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)
        for norm in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward_out_norm):
            if norm is not None and norm.as_rms_scale() is None:
                raise ValueError("a sandwich block fuses its norms with the sums around them: they must be RMS scales")
        self.shift_tensor, self.average_tensor = token_shift, depth_average
        self.shift = torch.empty(self.hidden_size, dtype=dtype, device=device) if token_shift else None
        self.depth, self.depth_slots = int(depth), int(depth_slots)
        self.average = None
        if depth_average:
            if not 0 < self.depth < self.depth_slots:
                raise ValueError(f"a depth average over {self.depth} results in front needs 0 < depth < depth_slots "
                                 f"({self.depth_slots})")
            self.average = torch.empty(self.depth + 1, dtype=dtype, device=device)
        self.side = None
        if token_side:
            side = dict(token_side)
            dim = int(side["dim"])
            if dim <= 0 or int(side["index"]) < 0:
                raise ValueError(f"a token side input needs a positive size and a place in the table, got {side}")
            self.side = dict(dim=dim, column=int(side["index"]) * dim, eps=float(side["eps"]),
                             scale=float(side.get("scale", 1.0)), name=side["name"])
            self.side_gate = torch.empty(dim, self.hidden_size, dtype=dtype, device=device)
            self.side_proj = torch.empty(self.hidden_size, dim, dtype=dtype, device=device)
            self.side_norm = torch.empty(self.hidden_size, dtype=dtype, device=device)
            # the norm's weight times the factor of the sum, formed once in 32-bit
            self.side_factor = torch.empty(self.hidden_size, dtype=torch.float32, device=device)

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.feed_forward_norm,
                                 self.feed_forward, self.feed_forward_out_norm) if p is not None)

    graph_safe = PreNormResidualBlock.graph_safe

    def ignorable_tensor_names(self) -> list[str]:
        return PreNormResidualBlock.ignorable_tensor_names(self) + list(self.unused_tensors)

    def finalize_weights(self) -> None:
        PreNormResidualBlock.finalize_weights(self)
        if self.side is not None:
            self.side_factor.copy_(self.side_norm.to(torch.float32) * self.side["scale"])

    def weight_slots(self) -> list[WeightSlot]:
        slots = PreNormResidualBlock.weight_slots(self)
        if self.shift is not None:
            slots.append(WeightSlot(self.shift_tensor, self.shift, init="normal"))
        if self.average is not None:
            slots.append(WeightSlot(self.average_tensor, self.average, init="normal"))
        if self.side is not None:
            name = self.side["name"]
            slots += [WeightSlot(f"{name}.gate", self.side_gate), WeightSlot(f"{name}.proj", self.side_proj),
                      WeightSlot(f"{name}.norm", self.side_norm, init="ones")]
        return slots

    def state_spec(self) -> StateSpec | None:
        """The block's own per-request state: the last normed row the mixer's shift has seen."""
        return StateSpec((self.hidden_size,), torch.float32) if self.shift is not None else None

    def forward(self, h, residual, ctx, cache):
        stack = None
        if self.average is not None:
            stack = ctx.shared(("depth_results", self.depth_slots, self.hidden_size), lambda: torch.empty(
                (self.depth_slots, ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=h.device))
        if residual is None:                      # the embedded tokens start the stream (and are result 0)
            x = K.stream_add(h, out=None if stack is None else stack[0])
        else:
            x = residual if residual.dtype == torch.float32 else K.stream_add(residual)
            if not isinstance(h, Summed):
                x = K.stream_add(x, h)
            if stack is not None and self.depth == 1:
                stack[0].copy_(x)                  # a block of another kind stood in front: its result is result 0
        weight, eps = self.mixer_norm.as_rms_scale()
        y = K.rms_norm_shift(x, weight, eps, self.dtype, shift=self.shift,
                             state=None if self.shift is None else cache.block_state, ctx=ctx)
        a = self.mixer.forward(y, ctx, cache)
        # The sums behind the sub-layers (and behind the token side input), in order: the last one is the layer's
        # result.  It goes to its place among the results when they are averaged; the stream handed in is then
        # left as it was (it may be a result itself).  The sum in front of a token side input also leaves the
        # new stream in the activation type, for the side input's first product.
        place = None if stack is None else stack[self.depth]
        average = dict(stack=stack, depth=self.depth, coeffs=self.average) if stack is not None else {}
        narrow = self.dtype if self.side is not None and self.dtype != torch.float32 else None

        def add(x, a, scale, last_sub_layer: bool):
            weight, eps = scale
            if last_sub_layer and self.side is None:
                result, mean = K.stream_add_norm(x, a, weight, eps, out=place, **average)
                return (result if mean is None else mean), None
            if last_sub_layer and narrow is not None:
                result, _, rounded = K.stream_add_norm(x, a, weight, eps, out=place, rounded=narrow)
                return result, rounded
            result, _ = K.stream_add_norm(x, a, weight, eps, out=place)
            return result, None

        x, rounded = add(x, a, self.mixer_out_norm.as_rms_scale(), self.feed_forward is None)
        if self.feed_forward is not None:
            weight, eps = self.feed_forward_norm.as_rms_scale()
            f = self.feed_forward.forward(K.rms_norm_shift(x, weight, eps, self.dtype), ctx)
            x, rounded = add(x, f, self.feed_forward_out_norm.as_rms_scale(), True)
        if self.side is not None:
            rows = ctx.shared("token_side_rows", lambda: None)
            if rows is None:
                raise RuntimeError(f"{self.side['name']}: the model's embedding has no side table")
            z = K.linear(x if rounded is None else rounded, self.side_gate)
            g = K.gelu_mul(z, rows, self.side["column"])
            y = K.linear(g, self.side_proj)
            result, mean = K.stream_add_norm(x, y, self.side_factor, self.side["eps"], **average)
            x = result if mean is None else mean
        return Summed(None), x


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
BLOCKS.register("sandwich_residual", SandwichResidualBlock)
BLOCKS.register("parallel_residual", ParallelResidualBlock)

__all__ = ["ParallelResidualBlock", "PreNormResidualBlock", "SandwichResidualBlock"]
