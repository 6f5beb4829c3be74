"""What a model says about the tensors it needs, and where tensors come from."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Protocol

import torch

# kinds decide the random initialisation and the dtype a tensor is kept in
MATRIX = "matrix"        # [out, in] projection or embedding table: compute dtype
NORM = "norm"            # scale vector of a norm: always float32 on the device
NORM_ZERO = "norm_zero"  # scale vector of a norm that is stored around zero (the norm multiplies by 1 + w): float32
VECTOR = "vector"        # a bias: float32 on the device


@dataclass(frozen=True)
class WeightSpec:
    """One tensor of a checkpoint: its name there, its shape, and its kind.

    ``optional`` tensors may be absent (and are ignored when present), e.g.
    ``lm_head.weight`` of a model whose output head is tied to the embedding.
    A dimension that is None is whatever the checkpoint stores (a size that no
    configuration key names, such as the rank of a low-rank pair); ``fill`` is
    then the shape a source of random weights draws.
    """

    name: str
    shape: tuple
    kind: str = MATRIX
    optional: bool = False
    fill: Optional[tuple] = None

    def fits(self, stored: tuple) -> bool:
        return len(stored) == len(self.shape) and all(w is None or int(g) == int(w) for g, w in zip(stored, self.shape))

    @property
    def drawn_shape(self) -> tuple:
        shape = self.fill if self.fill is not None else self.shape
        if any(d is None for d in shape):
            raise ValueError(f"{self.name}: a free dimension needs a size to draw random weights")
        return tuple(shape)


class TensorSource(Protocol):
    """Tensors by checkpoint name, on the CPU, in the dtype they are stored in."""

    def names(self) -> Iterable[str]: ...

    def shape(self, name: str) -> tuple[int, ...]: ...

    def get(self, name: str) -> torch.Tensor: ...


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every fault."""
