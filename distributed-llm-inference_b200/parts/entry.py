"""Parts that act on the residual stream between layers."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.gemm import project
from ..weights.loader import TensorDecl
from .base import Part, ResidualStream, build_part, register_part, tensor_name


@register_part("stream_entry", "reinject")
class Reinject(Part):
    """What a looped span of layers adds to the stream before one of its passes: the embedding of the step's
    tokens once more (if ``table`` names the embedding tensor) and row ``row`` of a learned table of vectors
    [rows, size] (if ``vector`` names it).  One kernel: h += table[token_ids] + vector[row].
    params: size, vocab_size, table, vector, row, rows."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.size, self.vocab = int(p["size"]), int(p["vocab_size"])
        self.table_name, self.vector_name = p.get("table"), p.get("vector")
        self.row, self.rows = int(p.get("row", 0)), int(p.get("rows", 1))
        self.table: torch.Tensor | None = None
        self.vector: torch.Tensor | None = None

    def declare(self):
        out = {}
        if self.table_name:
            out[self.table_name] = TensorDecl((self.vocab, self.size))
        if self.vector_name:
            out[self.vector_name] = TensorDecl((self.rows, self.size), "vector32")
        return out

    def load(self, tensors):
        if self.table_name:
            self.table = tensors[self.table_name]
        if self.vector_name:
            self.vector = tensors[self.vector_name][self.row].contiguous()

    def apply(self, stream: ResidualStream, batch) -> None:
        h = stream.settle()
        if self.table is not None or self.vector is not None:
            ops.stream_reinject(h, self.table, batch.token_ids if self.table is not None else None, self.vector)


@register_part("stream_entry", "token_gated_input")
class TokenGatedInput(Part):
    """A per-layer input from the token itself, added to the stream: with e = ``dim`` columns (from ``col0``) of the token's row
    of a table that all layers share,

        g = gelu_tanh(W_gate x) * e;    y = W_proj g;    x <- x + norm(y)

    where ``norm`` (a PartSpec of a norm with ``add_scaled_into``) carries the factor of the addition.
    params: hidden_size, vocab_size, dim, col0, table_cols, norm, tensors (names of table, gate, proj)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.vocab, self.dim = int(p["hidden_size"]), int(p["vocab_size"]), int(p["dim"])
        self.col0, self.table_cols = int(p["col0"]), int(p["table_cols"])
        self.names = {role: tensor_name(spec, role, default) for role, default in (("table", "table"), ("gate", "gate.weight"), ("proj", "proj.weight"))}
        self.norm = build_part("norm", p["norm"], env)
        self.table = self.w_gate = self.w_proj = None

    def children(self):
        return [self.norm]

    def declare(self):
        nm = self.names
        return {nm["table"]: TensorDecl((self.vocab, self.table_cols)), nm["gate"]: TensorDecl((self.dim, self.hidden)),
                nm["proj"]: TensorDecl((self.hidden, self.dim))}

    def load(self, tensors):
        nm = self.names
        self.table, self.w_gate, self.w_proj = tensors[nm["table"]], tensors[nm["gate"]], tensors[nm["proj"]]

    def apply(self, stream: ResidualStream, batch, want_cast: bool = False) -> None:
        h = stream.settle()
        g = project(stream.activation(self.env.dtype), self.w_gate)
        ops.gelu_mul_rows(g, self.table, self.col0, batch.token_ids)
        stream.cast = self.norm.add_scaled_into(h, project(g, self.w_proj), want_cast)


@register_part("stream_entry", "depth_average")
class DepthAverage(Part):
    """What goes on behind layer ``index`` is a learned mixture of the embedding output X_0 and of every layer's result so far:
    x <- sum over j <= index + 1 of weight[j] * X_j, X_(i+1) being what layer i left (before this mixing).  The results of a
    step live in one buffer [layers, n, size] (in the step's scratch); a layer works in place in its slot, and this part
    writes the mixture into the next slot, where the next layer works.  ``begin`` (called before the layer runs) sets X_0
    aside and moves the stream into the first slot.  params: size, index, layers, tensor (the weights' name)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.size, self.index, self.layers = int(p["size"]), int(p["index"]), int(p["layers"])
        self.name = tensor_name(spec, "weight", "weight")
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.name: TensorDecl((self.index + 2,), "vector32")}

    def load(self, tensors):
        self.weight = tensors[self.name]

    def begin(self, stream: ResidualStream, batch) -> None:
        if "depth_average" in batch.scratch:
            return
        if self.index != 0:
            raise RuntimeError("depth_average: the first layer of the model starts the history of a step")
        h = stream.settle()
        hist = torch.empty((self.layers + 1, *h.shape), dtype=torch.float32, device=h.device)
        hist[0].copy_(h)
        batch.scratch["depth_average"] = (h, hist)  # X_0 stays where the embedding wrote it
        stream.h = hist[0]

    def apply(self, stream: ResidualStream, batch, want_cast: bool = False) -> None:
        x0, hist = batch.scratch["depth_average"]
        if stream.settle().data_ptr() != hist[self.index].data_ptr():
            raise RuntimeError("depth_average: the layer did not work in its slot of the step's history")
        out = hist[self.index + 1]
        y = torch.empty(out.shape, dtype=self.env.dtype, device=out.device) if want_cast and self.env.dtype != torch.float32 else None
        ops.depth_average(out, x0, hist, self.weight, self.index + 2, y)
        stream.h, stream.cast = out, y


@register_part("stream_entry", "concat_project")
class ConcatProject(Part):
    """What a looped span of layers does to the stream before one of its passes: x <- W [x; x0], a product that reads the
    stream and the embedding output x0 side by side (W [size, 2 size], the stream's columns first).  x0 is gathered again
    from the embedding table by the step's token ids, so no copy of it is kept across the layers; one kernel lays
    [x; x0] out in the activation dtype, and the product's float32 sums become the new stream.
    params: size, vocab_size, table (the embedding tensor's name), tensor (W's name)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.size, self.vocab = int(p["size"]), int(p["vocab_size"])
        self.table_name, self.name = p["table"], tensor_name(spec, "weight", "weight")
        self.table = self.weight = None

    def declare(self):
        return {self.table_name: TensorDecl((self.vocab, self.size)), self.name: TensorDecl((self.size, 2 * self.size))}

    def load(self, tensors):
        self.table, self.weight = tensors[self.table_name], tensors[self.name]

    def apply(self, stream: ResidualStream, batch) -> None:
        h = stream.settle()
        both = torch.empty((h.shape[0], 2 * self.size), dtype=self.env.dtype, device=h.device)
        ops.concat_stream_rows(both, h, self.table, batch.token_ids)
        stream.h = project(both, self.weight, out_dtype=torch.float32)
        stream.cast = None
