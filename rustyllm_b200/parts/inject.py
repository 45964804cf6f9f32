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


@register("inject", "token_side_input")
class TokenSideInput(Part):
    """A per-token, per-layer learned vector gating a narrow projection of the stream:

        e = table[token, offset : offset + n];  g = gelu_tanh(W_gate x) * e;  y = W_proj g;  x += rms_norm(y) * w

    ``table`` ([vocab, columns]) is shared by all layers that use it; each reads its own ``n`` columns.  The
    projections run in the compute dtype, the norm and the addition in 32-bit."""

    def __init__(self, runtime: Runtime, hidden_size: int, vocab_size: int, columns: int, offset: int, size: int,
                 eps: float, names: Dict[str, str], table_owner: Optional[str] = None):
        """``names``: "table", "gate", "proj", "norm", "suffix".  ``table_owner``: the parameter path of the part
        that holds the shared table (all others alias it); ``None``: this part owns it."""
        if not (0 <= offset and offset + size <= columns):
            raise ValueError(f"columns [{offset}, {offset + size}) lie outside the table's {columns}")
        self.runtime = runtime
        self.d, self.V, self.columns, self.offset, self.n = hidden_size, vocab_size, columns, offset, size
        self.eps = float(eps)
        self.names, self.table_owner = names, table_owner
        self.table = self.w_gate = self.w_proj = self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        sfx = n.get("suffix", ".weight")
        return {
            "table": ParamSpec((ParamSource(n["table"], (self.V, self.columns)),), role="table", alias_of=self.table_owner),
            "w_gate": ParamSpec((ParamSource(n["gate"] + sfx, (self.n, self.d)),)),
            "w_proj": ParamSpec((ParamSource(n["proj"] + sfx, (self.d, self.n)),)),
            "weight": ParamSpec((ParamSource(n["norm"], (self.d,)),), role="vector", init="ones"),
        }

    def forward(self, x: torch.Tensor, embedded: Optional[torch.Tensor], step, rounded: Optional[torch.Tensor] = None):
        """Changes x in place; ``rounded``: x in the compute dtype if the caller has it.  Returns the new x in
        bfloat16 in a bfloat16 run (for the next reader), else ``None``."""
        from .linear import OUT_F32, OUT_SAME, linear
        dt = self.runtime.compute_dtype
        h = rounded
        if h is None:
            h = x
            if dt != torch.float32:
                h = torch.empty(x.shape, dtype=dt, device=x.device)
                K.convert(x, h)
        M = x.shape[0]
        t = torch.empty((M, self.n), dtype=dt, device=x.device)
        linear(h, self.w_gate, t, OUT_SAME)
        g = torch.empty((M, self.n), dtype=dt, device=x.device)
        K.gelu_gate(t, step.tokens, self.table, self.offset, g)
        y = torch.empty((M, self.d), dtype=torch.float32, device=x.device)
        linear(g, self.w_proj, y, OUT_F32)
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if dt == torch.bfloat16 else None
        K.norm_add(x, y, 1.0, None, 0.0, self.weight, self.eps, out)
        return out
