"""Feed-forwards: gated (SwiGLU and its kin) and plain."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.gemm import dense_product, fused_epilogue, last_product, project
from ..weights.loader import TensorDecl
from .base import Part, register_part, tensor_name


@register_part("feed_forward", "glu")
@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(act(gate(x)) * up(x)), act = SiLU (src/dli/model/llama.py:189-191) or another activation of
    ``ops.GLU_ACTIVATIONS``.  gate and up are read by their own names and laid together at load, so one
    product yields both: side by side, or — when the intermediate size is a multiple of 64 — interleaved in
    blocks of 64 rows, the layout in which the decode product applies act(gate) * up in its own epilogue.
    With ``limit`` > 0 the gate is bounded from above by it and up to [-limit, limit] before the activation, and ``up_shift`` is
    added to up: act(min(gate, limit)) * (clamp(up) + up_shift).
    params: hidden_size, intermediate_size, activation (default ``silu``), limit, up_shift, tensors (names of gate, up, down)."""

    graph_capturable = True
    takes_scaled_rows = True  # the input only goes to the gate | up product
    defer_output = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation", "silu")
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not supported (known: {sorted(ops.GLU_ACTIVATIONS)})")
        self.limit = float(spec.params.get("limit") or 0.0)
        self.up_shift = float(spec.params.get("up_shift") or 0.0)
        self.names = {role: tensor_name(spec, role, role + "_proj.weight") for role in ("gate", "up", "down")}
        self.w_gate_up: torch.Tensor | None = None
        self.tiled = False
        self.w_down: torch.Tensor | None = None

    def declare(self):
        nm = self.names
        return {
            nm["gate"]: TensorDecl((self.inter, self.hidden)),
            nm["up"]: TensorDecl((self.inter, self.hidden)),
            nm["down"]: TensorDecl((self.hidden, self.inter)),
        }

    def load(self, tensors):
        gate, up = tensors[self.names["gate"]], tensors[self.names["up"]]
        self.tiled = self.inter % 64 == 0 and self.env.dtype == torch.bfloat16
        if self.tiled:
            blocks = self.inter // 64
            self.w_gate_up = torch.stack([gate.view(blocks, 64, self.hidden), up.view(blocks, 64, self.hidden)], 1).reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], 0).contiguous()
        self.w_down = tensors[self.names["down"]]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tiled and fused_epilogue(x):
            act = ops.skinny_gemm_swiglu(x, self.w_gate_up, self.activation, self.limit, self.up_shift)
        elif self.tiled and dense_product(x, 2 * self.inter, "swiglu"):
            act = ops.dense_gemm_swiglu(x, self.w_gate_up, self.activation, self.limit, self.up_shift)
        else:
            gate_up = project(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            ops.silu_mul(act, gate_up, self.tiled, self.activation, self.limit, self.up_shift)
        return last_product(act, self.w_down, self.defer_output)


@register_part("feed_forward", "dense_act")
class DenseActMLP(Part):
    """down(act(up(x))): a plain feed-forward without a gate.  params: hidden_size, intermediate_size, activation
    (``relu2``: the square of relu; ``gelu_tanh``; ``silu``), tensors (names of up, down)."""

    graph_capturable = True
    takes_scaled_rows = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = spec.params.get("activation", "relu2")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not supported (known: {sorted(ops.ACTIVATIONS)})")
        self.names = {"up": tensor_name(spec, "up", "up_proj.weight"), "down": tensor_name(spec, "down", "down_proj.weight")}
        self.w_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def declare(self):
        return {self.names["up"]: TensorDecl((self.inter, self.hidden)), self.names["down"]: TensorDecl((self.hidden, self.inter))}

    def load(self, tensors):
        self.w_up, self.w_down = tensors[self.names["up"]], tensors[self.names["down"]]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if fused_epilogue(x):  # a decode step's few tokens: the activation rides in the up product's epilogue
            return project(ops.skinny_gemm_act(x, self.w_up, self.activation), self.w_down)
        if dense_product(x, self.inter, "act"):  # a long portion: the same in the epilogue of the product for many tokens
            return project(ops.dense_gemm_act(x, self.w_up, self.activation), self.w_down)
        return project(ops.activation(project(x, self.w_up), self.activation), self.w_down)


@register_part("feed_forward", "routed_glu")
class RoutedGLU(Part):
    """A mixture of ``num_experts`` small gated feed-forwards down_e(act(gate_e(x)) * up_e(x)), of which each token uses ``top``.

    The router's logits z = W_r x and everything that follows them are float32.  Scores are sigmoid(z) (``score``:
    ``"sigmoid"``).  The experts are CHOSEN by score + correction (a learned number per expert that steers the choice and
    nothing else); they are WEIGHTED by their scores without it, divided by their sum (+ 1e-20) and multiplied by ``route_scale``.
    With ``group_count`` > 1 the experts form that many equal groups of neighbours; a group's mark is the sum of its two
    largest choice scores, and only experts of the ``group_keep`` best groups can be chosen.  The output is the weighted
    sum of the chosen experts' outputs, added up in float32 in the order of the choice.

    One kernel routes; the tokens of every expert are then gathered by a counting sort on the device (no shape depends on
    the data, so a step with this part can be recorded in a CUDA graph), and two grouped products run over the sorted rows.
    params: hidden_size, intermediate_size, num_experts, top, route_scale, group_count, group_keep, activation, score, tensors
    (names of router, correction and, with ``{}`` for the expert's number, gate, up, down)."""

    graph_capturable = True
    takes_scaled_rows = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["intermediate_size"])
        self.experts, self.top = int(p["num_experts"]), int(p["top"])
        self.route_scale = float(p.get("route_scale", 1.0))
        self.group_count, self.group_keep = int(p.get("group_count") or 1), int(p.get("group_keep") or 1)
        self.activation = p.get("activation", "silu")
        if p.get("score", "sigmoid") != "sigmoid":
            raise ValueError(f"routed_glu: score={p['score']!r} (known: sigmoid)")
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not supported (known: {sorted(ops.GLU_ACTIVATIONS)})")
        per = self.experts // self.group_count
        if self.experts % self.group_count or self.group_keep > self.group_count or self.top > self.group_keep * per or self.top > ops.MOE_MAX_TOP:
            raise ValueError("routed_glu: experts must divide into the groups, and the kept groups must hold at least ``top`` experts")
        defaults = {"router": "router.weight", "correction": "router.correction", "gate": "experts.{}.gate_proj.weight",
                    "up": "experts.{}.up_proj.weight", "down": "experts.{}.down_proj.weight"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    def declare(self):
        nm = self.names
        out = {nm["router"]: TensorDecl((self.experts, self.hidden), "vector32"), nm["correction"]: TensorDecl((self.experts,), "vector32")}
        for e in range(self.experts):
            out[nm["gate"].format(e)] = TensorDecl((self.inter, self.hidden))
            out[nm["up"].format(e)] = TensorDecl((self.inter, self.hidden))
            out[nm["down"].format(e)] = TensorDecl((self.hidden, self.inter))
        return out

    def load(self, tensors):
        nm = self.names
        self.w_router, self.correction = tensors[nm["router"]], tensors[nm["correction"]]
        # [experts, 2 ff, H]: an expert's gate rows, then its up rows; [experts, H, ff]
        self.w_gate_up = torch.stack([torch.cat([tensors[nm["gate"].format(e)], tensors[nm["up"].format(e)]], 0) for e in range(self.experts)], 0).contiguous()
        self.w_down = torch.stack([tensors[nm["down"].format(e)] for e in range(self.experts)], 0).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n = x.shape[0]
        ids = torch.empty((n, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((n, self.top), dtype=torch.float32, device=x.device)
        ops.moe_route(ids, weights, x, self.w_router, self.correction, self.group_count, self.group_keep, self.route_scale)
        out = torch.empty((n, self.hidden), dtype=x.dtype, device=x.device)
        ops.moe_experts(out, x, ids, weights, self.w_gate_up, self.w_down, self.activation)
        return out
