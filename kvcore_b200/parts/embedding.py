"""Token embedding and output head.

Embedding is a row gather (kvcore/model/models/llama3.py:161-165, 178-180).  The head
multiplies the selected hidden rows with the ``[V, E]`` matrix, shares the embedding matrix
when tied, and applies ``logit_scale`` when it is not 1 (llama3.py:219-225, 245-247;
kvcore/sample/logits_processor.py:46-54).  Logits leave the head in 32-bit.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import EMBEDDINGS, LM_HEADS, Part, WeightSlot


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, name: str, tensor: str | None = None,
                 scale: float | None = None, side_tensor: str | None = None, side_width: int = 0,
                 dtype, device) -> None:
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        # ``scale``: the embedded tokens are ``table[id] * scale``, formed in 32-bit; the result is then the
        # first value of a 32-bit residual stream rather than rows of the activation type
        self.scale = None if scale is None else float(scale)
        self.tensor = tensor or f"{name}.weight"     # the table's full checkpoint name
        self.weight = torch.empty(self.vocab_size, self.hidden_size, dtype=dtype, device=device)
        # ``side_tensor``: a second table ``[vocab, side_width]`` whose row of a token is an input of the
        # layers themselves (each block reads its own columns); gathered once a step by ``side_rows``
        self.side_tensor, self.side_width = side_tensor, int(side_width)
        if (side_tensor is None) != (self.side_width == 0):
            raise ValueError("a side table needs both its tensor's name and its width")
        self.side_weight = (torch.empty(self.vocab_size, self.side_width, dtype=dtype, device=device)
                            if side_tensor is not None else None)

    def weight_slots(self) -> list[WeightSlot]:
        slots = [WeightSlot(self.tensor, self.weight)]
        if self.side_weight is not None:
            slots.append(WeightSlot(self.side_tensor, self.side_weight))
        return slots

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        if self.scale is not None:
            return K.embed_scaled(self.weight, token_ids, self.scale)
        return K.gather_rows(self.weight, token_ids)

    def side_rows(self, token_ids: torch.Tensor) -> torch.Tensor | None:
        """The step's rows ``[T, side_width]`` of the side table (None without one)."""
        return None if self.side_weight is None else K.gather_rows(self.side_weight, token_ids)


class LMHead(Part):
    graph_safe = True

    def __init__(
        self,
        *,
        vocab_size: int,
        hidden_size: int,
        name: str,
        tied_to: str | None = None,
        logit_scale: float = 1.0,
        tied_weight: torch.Tensor | None = None,
        tensor: str | None = None,
        dtype,
        device,
    ) -> None:
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        self.tied_to = tied_to
        self.logit_scale = float(logit_scale)
        self.tensor = tensor or f"{name}.weight"     # the matrix's full checkpoint name
        if tied_to is not None:
            if tied_weight is None:
                raise ValueError(f"lm head is tied to {tied_to!r} but no such matrix was given")
            self.weight = tied_weight
        else:
            self.weight = torch.empty(self.vocab_size, self.hidden_size, dtype=dtype, device=device)

    def weight_slots(self) -> list[WeightSlot]:
        if self.tied_to is not None:
            return []
        return [WeightSlot(self.tensor, self.weight)]

    def ignorable_tensor_names(self) -> list[str]:
        # a checkpoint may still carry the tied matrix under the head's own name
        return [self.tensor] if self.tied_to is not None else []

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        logits = K.linear(hidden, self.weight, None, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            logits = logits * self.logit_scale
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
LM_HEADS.register("lm_head", LMHead)

__all__ = ["LMHead", "TokenEmbedding"]
