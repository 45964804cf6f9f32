"""What a model adds to the residual stream between layers, outside any layer.

``pass_entry``: where a group of layers that runs several times is entered, the stream gets,
before the pass's first layer, (a) from the second pass on the embedding's output again (the
stream as it was before the first layer) and (b) a learned vector of the pass, row t of a
[passes, d] table.  All in 32-bit.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..config.spec import ParamSource, ParamSpec
from .base import Part, Runtime
from .registry import register


@register("inject", "pass_entry")
class PassEntry(Part):
    needs_embedding_output = True

    def __init__(self, runtime: Runtime, hidden_size: int, passes: int, name: Optional[str]):
        self.runtime = runtime
        self.d, self.passes, self.name = hidden_size, passes, name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        if self.name is None:
            return {}
        return {"table": ParamSpec((ParamSource(self.name, (self.passes, self.d)),), role="vector", init="normal")}

    def forward(self, x: torch.Tensor, embedded: Optional[torch.Tensor], step, row: int, again: bool) -> None:
        """x += (embedded if again) + table[row], in place."""
        if not (0 <= row < self.passes):
            raise ValueError(f"pass {row} of {self.passes}")
        K.residual_inject(x, embedded if again else None, self.table[row] if self.table is not None else None)
