"""Parts that feed the stream from something other than the layer before: an input from the token itself at the end
of a layer ("token_input" family) and what a run of the schedule starts with ("run_input" family).

A tensor name that begins with "/" is a tensor of the whole model, not of the part's layer: the layers' token inputs
share one table, of which each reads its own columns.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec, register_part
from .stream import settle


@register_part("token_input", "gated_token_rows")
class GatedTokenRows(Part):
    """`W_proj (gelu_tanh(W_gate x) * e)`, with e the columns [first_column, first_column + dim) of the token's row
    of a table [vocab, columns].  params: hidden_size, dim, vocab_size, table_columns, first_column, table_name
    (begin it with "/" for a table of the whole model), gate_name, proj_name.  Returns float32 rows; the norm that
    they pass before they are added is the arrangement's."""

    graph_safe = True
    graph_safe_prompts = True

    def weight_specs(self):
        p = self.params
        return {p["table_name"]: WeightSpec((p["vocab_size"], p["table_columns"])),
                p["gate_name"]: WeightSpec((p["dim"], p["hidden_size"])),
                p["proj_name"]: WeightSpec((p["hidden_size"], p["dim"]))}

    def load(self, tensors):
        p = self.params
        self.table, self.w_gate, self.w_proj = tensors[p["table_name"]], tensors[p["gate_name"]], tensors[p["proj_name"]]
        if not (self.table.dtype == self.w_gate.dtype == self.w_proj.dtype):
            self.table = self.table.to(self.w_gate.dtype)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate, self.w_proj))

    def forward(self, x, step, rows=None):
        gate = ops.linear(x, self.w_gate, self.runtime.dtype)
        g = ops.token_gate(gate, self.table, int(self.params["first_column"]), step.tok_ids, rows)
        return ops.linear(g, self.w_proj, torch.float32)


@register_part("run_input", "step_vector")
class StepVector(Part):
    """What a run of the schedule adds to the stream before its layer: row `index` of a table [entries, hidden] and,
    where asked, the stream as the embedding left it.  params: hidden_size, entries, name."""

    graph_safe = True
    graph_safe_prompts = True

    def weight_specs(self):
        return {self.params["name"]: WeightSpec((self.params["entries"], self.params["hidden_size"]), init="normal")}

    def load(self, tensors):
        self.table = tensors[self.params["name"]].to(torch.float32).contiguous()

    def weight_bytes(self):
        return 0

    def forward(self, stream, index: int, first=None):
        settle(stream, None, vec=self.table[index], extra=first)
