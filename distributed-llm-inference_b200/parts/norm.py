"""RMS normalisation, fused with the residual addition that precedes it."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, PendingScaled, PendingSum, register_part, tensor_name


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = (h + delta) * rsqrt(mean((h + delta)^2) + eps) * weight, all in float32 and rounded
    once (src/dli/model/llama.py:41-44 rounds before the weight product; one rounding is closer
    to the float32 result).  params: size, eps, tensor (the weight's name; default prefix + "weight"),
    offset (added to the stored weight at load: 1.0 for checkpoints that store the deviation from one).

    ``delta`` may be a ``PendingSum`` of two sublayer outputs (layers whose branches run side by side): both are
    added in the same kernel.  It may be a ``PendingScaled`` (one or two outputs with constant factors and a learned
    scale per feature): multiplied and added in the same kernel too.  ``add_norm_pair`` also norms the same sum with a second norm's weight — two readers
    of one stream share the sum of squares."""

    graph_capturable = True
    takes_pending_sum = True
    takes_pending_scaled = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.name = tensor_name(spec, "weight", "weight")
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.name: TensorDecl((self.size,), "vector32")}

    def load(self, tensors):
        self.weight = tensors[self.name] + self.offset if self.offset else tensors[self.name]

    def _out(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        return torch.empty((n, self.size), dtype=self.env.dtype, device=h.device)

    def add_norm(self, h: torch.Tensor, delta, rows: torch.Tensor | None = None) -> torch.Tensor:
        y = self._out(h, rows)
        if isinstance(delta, PendingSum):
            ops.add_rmsnorm_pair(y, None, h, delta.a, delta.b, self.weight, None, self.eps, rows)
        elif isinstance(delta, PendingScaled):
            ops.add_rmsnorm_scaled(y, h, delta.a, delta.fa, delta.b, delta.fb, delta.scale, self.weight, self.eps, rows)
        else:
            ops.add_rmsnorm(y, h, delta, self.weight, self.eps, rows)
        return y

    def add_norm_pair(self, h: torch.Tensor, delta, other: "RMSNorm") -> tuple[torch.Tensor, torch.Tensor] | None:
        """(self(h + delta), other(h + delta)) from one kernel, the sum written back to h; None if ``other`` does not
        divide by the same root mean square."""
        if not isinstance(other, RMSNorm) or other.eps != self.eps or other.size != self.size:
            return None
        y1, y2 = self._out(h, None), self._out(h, None)
        a, b = (delta.a, delta.b) if isinstance(delta, PendingSum) else (delta, None)
        ops.add_rmsnorm_pair(y1, y2, h, a, b, self.weight, other.weight, self.eps, None)
        return y1, y2

    def add_product_norm(self, h: torch.Tensor, product) -> ops.ScaledRows | None:
        """h += product (computed here, float32 sums added to float32 h) and the norm's first half
        in the product's epilogue; the factor rsqrt(mean(h^2) + eps) of each row travels with the
        result and is applied by the product that reads it, to its float32 sums."""
        if not ops.skinny_gemm_supported(h.shape[0], self.size) or h.shape[0] > 64:
            return None  # the product that reads the result could not take rows of this size
        return ops.skinny_gemm_residual(product.x, product.weight, h, self.weight, self.eps)


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """y = (v - mean(v)) / sqrt(var(v) + eps) * weight, var the mean of the squared deviations, no bias; float32
    arithmetic, one rounding.  params: size, eps, tensor (the weight's name; default prefix + "weight").

    Besides ``add_norm`` (v = h + delta) it norms on both sides of the residual addition in one kernel:
    ``post_add_norm(h, a, post)`` is h += post(a), y = self(h), for layers whose sublayer outputs are normed
    before they are added; ``add_into(h, a)`` is the first half alone."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = tensor_name(spec, "weight", "weight")
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.name: TensorDecl((self.size,), "vector32")}

    def load(self, tensors):
        self.weight = tensors[self.name]

    def _out(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        n = h.shape[0] if rows is None else rows.numel()
        return torch.empty((n, self.size), dtype=self.env.dtype, device=h.device)

    def add_norm(self, h: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor:
        if delta is not None:
            if rows is not None:
                raise ValueError("layernorm: a plain delta is added to the whole stream (rows=None)")
            h += delta.float()
        y = self._out(h, rows)
        ops.post_add_layernorm(y, h, None, None, self.weight, 0.0, self.eps, rows)
        return y

    def post_add_norm(self, h: torch.Tensor, a: torch.Tensor, post: "LayerNorm", rows: torch.Tensor | None = None) -> torch.Tensor:
        y = self._out(h, rows)
        ops.post_add_layernorm(y, h, a, post.weight, self.weight, post.eps, self.eps, rows)
        return y

    def add_into(self, h: torch.Tensor, a: torch.Tensor) -> None:
        ops.post_add_layernorm(None, h, a, self.weight, None, self.eps, 0.0)


@register_part("norm", "group_rmsnorm")
class GroupRMSNorm(Part):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive parts, each is divided by its own
    sqrt(mean(part^2) + eps), and the whole is multiplied by a weight; float32 arithmetic, one rounding.  groups = 1 is the
    plain RMS norm.  Two uses: ``add_norm`` norms rows of the stream (a model's last norm), and ``add_scaled_into(h, a)`` is
    h += mult * norm(a) * weight, for layers that norm a sublayer's OUTPUT before the residual addition.
    params: size, eps, groups (default 1), mult (default 1), tensor (the weight's name; default prefix + "weight")."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.groups = int(spec.params.get("groups", 1))
        self.mult = float(spec.params.get("mult", 1.0))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: size={self.size} is not a multiple of groups={self.groups}")
        self.name = tensor_name(spec, "weight", "weight")
        self.weight: torch.Tensor | None = None

    def declare(self):
        return {self.name: TensorDecl((self.size,), "vector32")}

    def load(self, tensors):
        self.weight = tensors[self.name]

    def add_norm(self, h: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor:
        if delta is not None:
            if rows is not None:
                raise ValueError("group_rmsnorm: a plain delta is added to the whole stream (rows=None)")
            h += delta.float()
        n = h.shape[0] if rows is None else rows.numel()
        y = torch.empty((n, self.size), dtype=self.env.dtype, device=h.device)
        ops.group_norm_rows(y, h, self.weight, self.groups, self.eps, rows)
        return y

    def add_scaled_into(self, h: torch.Tensor, a: torch.Tensor, want_cast: bool = False) -> torch.Tensor | None:
        """h += mult * norm(a) * weight.  With ``want_cast`` (and a in a 16-bit dtype) the new h is also returned in a's dtype,
        written by the same kernel: what the next sublayer's product reads."""
        y = torch.empty_like(a) if want_cast and a.dtype != torch.float32 else None
        ops.group_norm_add(h, a, self.weight, self.groups, self.eps, self.mult, y)
        return y
