"""What a schedule entry may add to the residual stream before its layer runs.

``pass_input``: a span of layers that runs several times in a row adds, at the start of pass ``row``, that row
of a learned table ``[rows, hidden]`` to every token, and (``add_embedding``) the embedding's output as it was
before the first layer.  The sum is 32-bit.  Parameters: ``hidden_size``, ``rows``, ``row``, ``table`` (a tensor
name, taken as it stands), ``add_embedding``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..weights.loader import TensorSpec
from .base import StreamInput, register_part


class PassInput(StreamInput):
    graph_safe = True

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden_size"])
        self.rows = int(params["rows"])
        self.row = int(params["row"])
        if not (0 <= self.row < self.rows):
            raise ValueError(f"pass_input: row {self.row} lies outside a table of {self.rows} rows")
        self.needs_embedding = bool(params.get("add_embedding"))
        self.vector: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.params["table"]: TensorSpec((self.rows, self.hidden), "norm")}

    def bind(self, tensors) -> None:
        self.vector = tensors[self.params["table"]][self.row].float().contiguous()

    def kernel_files(self):
        return ("layernorm",)

    def forward(self, stream, embedded, ctx) -> None:
        if self.needs_embedding and embedded is None:
            raise RuntimeError("pass_input: the model did not keep the embedding's output")
        stream.add_rows(embedded if self.needs_embedding else None, self.vector)


register_part("stream_input", "pass_input", PassInput)
