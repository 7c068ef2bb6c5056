"""Steps on the residual stream that are not sublayers of a block (category ``stream``).

A stream part offers ``forward(hs, ctx) -> None``: it changes the float32 stream ``hs`` of the
step's rows in place.  The step function runs a schedule entry's ``before`` part right ahead of
the entry's layer; a block runs its layer's ``stream_after`` part after its sublayers.

``pass_start``: the start of a pass over a stretch of layers that runs several times with the same
weights.  ``hs += embedding_output`` when ``add_embedding`` (the embedding's rows of the step, which
the step function keeps in ``ctx.embedding_output`` for a plan that asks for it), then
``hs += table[row]``, a learned vector per pass.  Parameters: ``table_name`` (a tensor
``[rows, hidden]`` named from the model's root), ``rows``, ``row``, ``hidden_size``, ``add_embedding``.

``token_side``: a per-layer input chosen by the token.  With ``e`` the columns
``[offset, offset + dim)`` of row ``token`` of a table shared by the layers:
``g = gelu_tanh(W_gate hs) * e``; ``y = W_proj g``; ``hs += y / sqrt(mean(y^2) + eps) * w``.  The
norm's statistics and the add are float32; the two products read the stream and ``g`` in the
activation dtype.  Parameters: ``hidden_size``, ``dim``, ``offset``, ``table_name`` (from the
model's root) and ``table_shape``, ``eps``, ``names`` (``gate``, ``proj``, ``norm`` under the part's
prefix).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import kernels as K
from .base import Part, register_part
from .linear import project
from .plan import ParamSpec


@register_part("stream", "pass_start")
class PassStart(Part):
    needs_embedding_output = True

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.rows = int(spec["rows"])
        self.row = int(spec["row"])
        self.table_name = spec.get("table_name") or None
        self.add_embedding = bool(spec.get("add_embedding", False))
        self.needs_embedding_output = self.add_embedding
        if self.table_name and not 0 <= self.row < self.rows:
            raise ValueError(f"pass_start: row {self.row} is outside the table's {self.rows} rows")
        self.vector = None

    def params(self) -> Dict[str, ParamSpec]:
        return {self.table_name: ParamSpec((self.rows, self.hidden), role="vector")} if self.table_name else {}

    def libraries(self) -> set:
        return {"stream_ops"}

    def load(self, source) -> None:
        if self.table_name:
            self.vector = self.fetch_shared(source, self.table_name)[self.row].contiguous()

    def forward(self, hs: torch.Tensor, ctx) -> None:
        K.tag = "pass start"
        K.add_rows(hs, ctx.embedding_output if self.add_embedding else None, self.vector)
        K.tag = None


@register_part("stream", "token_side")
class TokenSide(Part):
    needs_embedding_output = False

    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.hidden = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.offset = int(spec["offset"])
        self.eps = float(spec["eps"])
        self.table_name = str(spec["table_name"])
        self.table_shape = tuple(int(n) for n in spec["table_shape"])
        if self.offset < 0 or self.offset + self.dim > self.table_shape[1]:
            raise ValueError(f"token_side: columns [{self.offset}, {self.offset + self.dim}) are outside the table's {self.table_shape[1]}")
        names = dict(spec.get("names") or {})
        self.n_gate = self.name(names.get("gate", "gate"))
        self.n_proj = self.name(names.get("proj", "proj"))
        self.n_norm = self.name(names.get("norm", "norm"))
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def params(self) -> Dict[str, ParamSpec]:
        return {self.table_name: ParamSpec(self.table_shape),
                self.n_gate: ParamSpec((self.dim, self.hidden)),
                self.n_proj: ParamSpec((self.hidden, self.dim)),
                self.n_norm: ParamSpec((self.hidden,), role="vector", init="ones")}

    def libraries(self) -> set:
        libs = {"stream_ops", "gemm_simt"}
        if self.runtime.fast_kernels and self.hidden >= 128:
            libs.add("gemm_tc")
        return libs

    def load(self, source) -> None:
        self.table = self.fetch_shared(source, self.table_name)
        self.w_gate = self.fetch(source, self.n_gate)
        self.w_proj = self.fetch(source, self.n_proj)
        self.norm_w = self.fetch(source, self.n_norm)

    def forward(self, hs: torch.Tensor, ctx) -> None:
        rt = self.runtime
        T = hs.shape[0]
        x = hs
        if rt.act_dtype != torch.float32:
            x = torch.empty(hs.shape, dtype=rt.act_dtype, device=hs.device)
            K.tag = "cast"
            K.stream_cast(hs, x)
        a = torch.empty((T, self.dim), dtype=torch.float32, device=hs.device)
        K.tag = "side gate"
        project(rt, x, self.w_gate, a)
        g = torch.empty((T, self.dim), dtype=rt.act_dtype, device=hs.device)
        K.tag = "side gelu * table"
        K.gelu_gate(a, self.table, self.offset, ctx.token_ids, g)
        y = torch.empty((T, self.hidden), dtype=torch.float32, device=hs.device)
        K.tag = "side proj"
        project(rt, g, self.w_proj, y)
        K.tag = "side norm + add"
        K.stream_norm_add(hs, y, self.norm_w, self.eps)
        K.tag = None
