"""Recurrent mixers (state-space, delta rule): per-request state of fixed size instead of keys and values in pages."""

from __future__ import annotations

import torch

from ..cache.needs import StateNeed
from ..kernels import ops
from ..kernels.gemm import project
from ..weights.loader import TensorDecl
from .base import Part, register_part, tensor_name


@register_part("mixer", "mamba2")
class Mamba2Mixer(Part):
    """Mamba-2 (state-space duality) on any mix of prompt portions and decoded tokens.

    The input projection yields z | x | B | C | dt (inner = num_heads * head_dim columns each for z and x,
    groups * state_size each for B and C, one dt per head).  x | B | C pass a causal convolution per channel
    (``conv_taps`` taps, bias) and SiLU.  Per head, with dt = softplus(dt + dt_bias) and its group's B and C:

        S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T        (S: state_size x head_dim, float32; kept transposed)
        y_t = S_t^T C_t + D x_t

    y * silu(z) is divided by its RMS in ``norm_groups`` equal parts of the row, multiplied by a weight, and goes
    through the output projection.  A request keeps S and the convolution's last taps - 1 inputs in its state
    slot; both start at zero.  The step sizes, decays, the state and every sum of the recurrence are float32.

    params: hidden_size, num_heads, head_dim, state_size, groups, conv_taps, norm_groups, eps, tensors (names of
    in, conv, conv_bias, dt_bias, A_log, D, norm, o)."""

    graph_capturable = True  # padding rows of a replayed graph name a state slot that no request owns

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.P, self.N = int(p["num_heads"]), int(p["head_dim"]), int(p["state_size"])
        self.groups, self.taps, self.parts = int(p["groups"]), int(p["conv_taps"]), int(p["norm_groups"])
        self.eps = float(p["eps"])
        if self.heads % self.groups or (self.heads * self.P) % self.parts or self.taps < 1:
            raise ValueError("mamba2: heads must be a multiple of groups, heads * head_dim of norm_groups, and conv_taps >= 1")
        if self.N > ops.SSM_SCAN_MAX_STATE:
            raise ValueError(f"mamba2: state_size={self.N} is above the scan kernel's {ops.SSM_SCAN_MAX_STATE}")
        self.inner = self.heads * self.P
        self.channels = self.inner + 2 * self.groups * self.N
        self.names = {role: tensor_name(spec, role, default) for role, default in (
            ("in", "in_proj.weight"), ("conv", "conv1d.weight"), ("conv_bias", "conv1d.bias"), ("dt_bias", "dt_bias"),
            ("A_log", "A_log"), ("D", "D"), ("norm", "norm.weight"), ("o", "out_proj.weight"))}
        self.w: dict[str, torch.Tensor] = {}

    def declare(self):
        nm = self.names
        return {
            nm["in"]: TensorDecl((self.inner + self.channels + self.heads, self.hidden)),
            nm["conv"]: TensorDecl((self.channels, self.taps), "vector32"),
            nm["conv_bias"]: TensorDecl((self.channels,), "vector32"),
            nm["dt_bias"]: TensorDecl((self.heads,), "vector32"),
            nm["A_log"]: TensorDecl((self.heads,), "vector32"),
            nm["D"]: TensorDecl((self.heads,), "vector32"),
            nm["norm"]: TensorDecl((self.inner,), "vector32"),
            nm["o"]: TensorDecl((self.hidden, self.inner)),
        }

    def load(self, tensors):
        self.w = {role: tensors[name] for role, name in self.names.items()}
        self.w["conv"] = self.w["conv"].t().contiguous()  # [taps, channels]: the kernel reads a tap's weights side by side

    def cache_need(self):
        """The recurrent state (float32) and the convolution's carried inputs (activation dtype), per request."""
        return (StateNeed((self.heads, self.P, self.N), torch.float32), StateNeed((self.taps - 1, self.channels), self.env.dtype))

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        w = self.w
        n = x.shape[0]
        ssm_state, conv_state = cache.states
        u = project(x, w["in"])  # z | x | B | C | dt
        xbc = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv_silu(xbc, u, self.inner, w["conv"], w["conv_bias"], conv_state, batch.seq_of_token, batch.q_start, batch.state_slot)
        if self.taps > 1:
            ops.conv_state_update(conv_state, u, self.inner, batch.q_start, batch.state_slot)
        y = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        ops.ssm_scan(y, xbc, u, self.inner + self.channels, w["dt_bias"], w["A_log"], w["D"], ssm_state, batch.q_start, batch.state_slot,
                     self.groups, max_len=batch.max_q_len)
        gated = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(gated, y, u, 0, w["norm"], self.parts, self.eps)
        return project(gated, w["o"])


@register_part("mixer", "gated_delta")
class GatedDeltaRule(Part):
    """The gated delta rule on any mix of prompt portions and decoded tokens: a linear recurrence whose state is a
    matrix S (head_dim x value_dim) per head.

    One product yields q | k | v | g | b | a (q and k: ``num_kv_heads`` heads of ``head_dim``; v and g: ``num_heads``
    heads of ``value_dim``; b and a: one number per head).  q | k | v pass a causal convolution per channel
    (``conv_taps`` taps, no bias) and SiLU; q and k are then made unit vectors per head (float32; ``unit_eps`` inside
    the root) and q is multiplied by head_dim^-1/2.  Head h reads q/k head h // (num_heads / num_kv_heads).  Per head
    and token, with beta = sigmoid(b) and the decay gamma = exp(-exp(A_log) softplus(a + dt_bias)):

        S <- gamma S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q

    (the read-out sees the token's own write).  Each head's o is divided by its root mean square (``eps``), multiplied
    by a weight of ``value_dim`` numbers that the heads share and by silu(g), and goes through the output projection.
    A request keeps S (float32) and the convolution's last taps - 1 inputs in its state slot; both start at zero.

    params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, conv_taps, eps, unit_eps, tensors (names of q,
    k, v, b, a, g, o, A_log, dt_bias, norm, q_conv, k_conv, v_conv)."""

    graph_capturable = True  # padding rows of a replayed graph name a state slot that no request owns

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.d, self.dv, self.taps = int(p["head_dim"]), int(p["value_dim"]), int(p["conv_taps"])
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps", 1e-6))
        if self.heads % self.kv_heads or self.taps < 1:
            raise ValueError("gated_delta: num_heads must be a multiple of num_kv_heads, and conv_taps >= 1")
        if self.d > ops.DELTA_MAX_HEAD_DIM:
            raise ValueError(f"gated_delta: head_dim={self.d} is above the scan kernel's {ops.DELTA_MAX_HEAD_DIM}")
        self.qk, self.inner = self.kv_heads * self.d, self.heads * self.dv
        self.channels = 2 * self.qk + self.inner  # what passes the convolution: q | k | v
        self.g_col = self.channels
        self.b_col = self.g_col + self.inner
        self.a_col = self.b_col + self.heads
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "b": "b_proj.weight", "a": "a_proj.weight",
                    "g": "g_proj.weight", "o": "o_proj.weight", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm.weight",
                    "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.w: dict[str, torch.Tensor] = {}

    def declare(self):
        nm, H = self.names, self.hidden
        return {
            nm["q"]: TensorDecl((self.qk, H)), nm["k"]: TensorDecl((self.qk, H)), nm["v"]: TensorDecl((self.inner, H)),
            nm["g"]: TensorDecl((self.inner, H)), nm["b"]: TensorDecl((self.heads, H)), nm["a"]: TensorDecl((self.heads, H)),
            nm["o"]: TensorDecl((H, self.inner)),
            nm["q_conv"]: TensorDecl((self.qk, self.taps), "vector32"), nm["k_conv"]: TensorDecl((self.qk, self.taps), "vector32"),
            nm["v_conv"]: TensorDecl((self.inner, self.taps), "vector32"),
            nm["A_log"]: TensorDecl((self.heads,), "vector32"), nm["dt_bias"]: TensorDecl((self.heads,), "vector32"),
            nm["norm"]: TensorDecl((self.dv,), "vector32"),
        }

    def load(self, tensors):
        t = {role: tensors[name] for role, name in self.names.items()}
        self.w = {
            "in": torch.cat([t["q"], t["k"], t["v"], t["g"], t["b"], t["a"]], 0).contiguous(),
            # [taps, channels]: the kernel reads a tap's weights side by side
            "conv": torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], 0).t().contiguous(),
            "A_log": t["A_log"], "dt_bias": t["dt_bias"], "o": t["o"],
            "norm": t["norm"].repeat(self.heads).contiguous(),  # the heads share the weight; the kernel reads one per column
        }

    def cache_need(self):
        """The recurrent state (float32; kept transposed, a value column's head_dim numbers together) and the
        convolution's carried inputs (activation dtype), per request."""
        return (StateNeed((self.heads, self.dv, self.d), torch.float32), StateNeed((self.taps - 1, self.channels), self.env.dtype))

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        w = self.w
        n = x.shape[0]
        state, conv_state = cache.states
        u = project(x, w["in"])  # q | k | v | g | b | a
        qkv = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv_silu(qkv, u, 0, w["conv"], None, conv_state, batch.seq_of_token, batch.q_start, batch.state_slot)
        if self.taps > 1:
            ops.conv_state_update(conv_state, u, 0, batch.q_start, batch.state_slot)
        o = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        ops.delta_rule_scan(o, qkv, u, self.b_col, self.a_col, w["dt_bias"], w["A_log"], state, batch.seq_of_token, batch.q_start, batch.state_slot,
                            self.kv_heads, self.d, self.unit_eps, max_len=batch.max_q_len)
        gated = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(gated, o, u, self.g_col, w["norm"], self.heads, self.eps, gate_after=True)
        return project(gated, w["o"])


@register_part("mixer", "mingru")
class MinGRU(Part):
    """minGRU on any mix of prompt portions and decoded tokens: a gated recurrence whose gates read only the current token.

    One product yields z | x | g (``width`` columns each).  With z = sigmoid(z + b_z), u = x + b_x and the candidate
    c = u + 1/2 where u >= 0, sigmoid(u) elsewhere, element by element

        S_t = (1 - z_t) S_(t-1) + z_t c_t,        out_t = W_o (S_t * silu(g_t)).

    A request keeps S (float32, ``width`` numbers) in its state slot; it starts at zero.  Gates, candidate and state are float32.
    params: hidden_size, width, tensors (names of z, z_bias, x, x_bias, g, o)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        defaults = {"z": "z_proj.weight", "z_bias": "z_proj.bias", "x": "x_proj.weight", "x_bias": "x_proj.bias", "g": "g_proj.weight",
                    "o": "o_proj.weight"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.w_in = self.wo = self.bz = self.bx = None

    def declare(self):
        nm, H, W = self.names, self.hidden, self.width
        return {nm["z"]: TensorDecl((W, H)), nm["x"]: TensorDecl((W, H)), nm["g"]: TensorDecl((W, H)), nm["o"]: TensorDecl((H, W)),
                nm["z_bias"]: TensorDecl((W,), "vector32"), nm["x_bias"]: TensorDecl((W,), "vector32")}

    def load(self, tensors):
        nm = self.names
        self.w_in = torch.cat([tensors[nm["z"]], tensors[nm["x"]], tensors[nm["g"]]], 0).contiguous()
        self.wo, self.bz, self.bx = tensors[nm["o"]], tensors[nm["z_bias"]], tensors[nm["x_bias"]]

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        p = project(x, self.w_in)  # z | x | g
        gated = torch.empty((x.shape[0], self.width), dtype=x.dtype, device=x.device)
        ops.mingru_scan(gated, p, self.bz, self.bx, cache.state, batch.q_start, batch.state_slot, max_len=batch.max_q_len)
        return project(gated, self.wo)


def _recurrence_row(kq_heads: int, heads: int, d: int, dv: int) -> int:
    """Floats of a token's row as ``ops.decay_recurrence`` reads it: read vectors | keys | decays | values | betas."""
    return ops.decay_recurrence_row(kq_heads, heads, d, dv)


@register_part("mixer", "shift_decay_recurrence")
class ShiftDecayRecurrence(Part):
    """A linear recurrence with token shift and a learned decay per head and key channel (RWKV-6 style time mixing), on any mix
    of prompt portions and decoded tokens.

    With x' the previous token's input (zeros before a sequence's first token), each of r, k, v, g, w reads its own blend
    x + (x' - x) * mu_s.  r, k, v are products of their blends (``num_heads`` heads of ``head_dim``), the gate is silu(W_g blend_g),
    the decay w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0)).  Per head, with the bonus u for the current token only:

        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;        S_t = diag(w_t) S_(t-1) + k_t v_t^T

    Each head's o is divided by its root mean square (``eps``), multiplied by a weight and the gate, and goes through the
    output projection.  A request keeps S (float32) and its last input row in its state slot; both start at zero.  Decays,
    the state and every sum of the recurrence are float32.

    params: hidden_size, num_heads, head_dim, eps, decay_rank (inner size of the decay's two products; absent: the checkpoint's),
    tensors (names of r, k, v, g, w1, w2, w0, u, norm, o, mu_r, mu_k, mu_v, mu_g, mu_w)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.heads, self.d = int(p["hidden_size"]), int(p["num_heads"]), int(p["head_dim"])
        self.eps = float(p["eps"])
        if self.d > ops.RECURRENCE_MAX_HEAD_DIM:
            raise ValueError(f"shift_decay_recurrence: head_dim={self.d} is above the scan kernel's {ops.RECURRENCE_MAX_HEAD_DIM}")
        self.inner = self.heads * self.d
        defaults = {"r": "r_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "w1": "w1.weight", "w2": "w2.weight",
                    "w0": "w0", "u": "bonus", "norm": "norm.weight", "o": "o_proj.weight"}
        defaults.update({"mu_" + s: "mu_" + s for s in "rkvgw"})
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.w: dict[str, torch.Tensor] = {}

    def declare(self):
        nm, H, I = self.names, self.hidden, self.inner
        out = {nm[r]: TensorDecl((I, H)) for r in ("r", "k", "v", "g")}
        out.update({nm["mu_" + s]: TensorDecl((H,), "vector32") for s in "rkvgw"})
        low = self.spec.params.get("decay_rank")  # None: whatever the checkpoint holds
        out.update({nm["w1"]: TensorDecl((low, H)), nm["w2"]: TensorDecl((I, low)),
                    nm["w0"]: TensorDecl((I,), "vector32"), nm["u"]: TensorDecl((self.heads, self.d), "vector32"),
                    nm["norm"]: TensorDecl((I,), "vector32"), nm["o"]: TensorDecl((H, I))})
        return out

    def load(self, tensors):
        t = {role: tensors[name] for role, name in self.names.items()}
        self.w = {
            "mu": torch.stack([t["mu_" + s] for s in "rkvgw"], 0).contiguous(),  # [5, H]
            "rkvg": torch.stack([t[r].t() for r in ("r", "k", "v", "g")], 0).contiguous(),  # [4, H, I]: the four products are one batched product
            "w1": t["w1"], "w2": t["w2"], "w0": t["w0"], "u": t["u"].contiguous(), "norm": t["norm"], "o": t["o"],
        }

    def cache_need(self):
        """The recurrent state (float32; kept transposed, a value column's head_dim numbers together) and the previous
        token's input row (activation dtype), per request."""
        return (StateNeed((self.heads, self.d, self.d), torch.float32), StateNeed((1, self.hidden), self.env.dtype))

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        from ..kernels.gemm import batched_project

        w = self.w
        n = x.shape[0]
        state, shift = cache.states
        blends = torch.empty((5, n, self.hidden), dtype=x.dtype, device=x.device)
        ops.token_shift_blend(blends, x, w["mu"], shift, batch.seq_of_token, batch.q_start, batch.state_slot)
        ops.conv_state_update(shift, x, 0, batch.q_start, batch.state_slot)
        rkvg = batched_project(blends[:4], w["rkvg"])  # [4, n, I]
        low = ops.activation(project(blends[4], w["w1"]), "tanh")
        wz = project(low, w["w2"])
        rows = torch.empty((n, _recurrence_row(self.heads, self.heads, self.d, self.d)), dtype=torch.float32, device=x.device)
        ops.shift_decay_prep(rows, rkvg, wz, w["w0"], self.heads, self.d)
        o = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        ops.decay_recurrence(o, rows, state, batch.q_start, batch.state_slot, self.heads, "bonus", w["u"], max_len=batch.max_q_len)
        gated = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(gated, o, rkvg[3], 0, w["norm"], self.heads, self.eps, gate_after=True)
        return project(gated, w["o"])


@register_part("mixer", "channel_delta")
class ChannelDeltaRule(Part):
    """The delta rule with one decay per head and KEY CHANNEL, on any mix of prompt portions and decoded tokens; the state
    is a matrix S (head_dim x value_dim) per head.

    One product yields q | k | v | a1 | g1 | b (q and k: ``num_kv_heads`` heads of ``head_dim``; v: ``num_heads`` heads of
    ``value_dim``; b: one number per head; a1 and g1: the inner halves of two low-rank products).  q | k | v pass a causal
    convolution per channel (``conv_taps`` taps, no bias) and SiLU; q and k are then made unit vectors per head (float32;
    ``unit_eps`` inside the root) and q is multiplied by head_dim^-1/2.  Head h reads q/k head h // (num_heads / num_kv_heads).
    Per head and token, with beta = sigmoid(b) and g = exp(-exp(A_log_h) softplus(W_a2 a1 + dt_bias)) [head_dim]:

        S <- diag(g) S;    w = beta (v - S^T k);    S <- S + k w^T;    o = S^T q

    Each head's o is divided by its root mean square (``eps``), multiplied by a weight of ``value_dim`` numbers that the
    heads share and by sigmoid(W_g2 g1), and goes through the output projection.  A request keeps S (float32) and the
    convolution's last taps - 1 inputs in its state slot; both start at zero.

    params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, conv_taps, eps, unit_eps, decay_rank and gate_rank (inner sizes
    of the two low-rank products; absent: the checkpoint's), tensors (names of q, k, v, b, a1, a2, g1, g2, o, A_log, dt_bias, norm, q_conv,
    k_conv, v_conv)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.d, self.dv, self.taps = int(p["head_dim"]), int(p["value_dim"]), int(p["conv_taps"])
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps", 1e-6))
        if self.heads % self.kv_heads or self.taps < 1:
            raise ValueError("channel_delta: num_heads must be a multiple of num_kv_heads, and conv_taps >= 1")
        if self.d > ops.RECURRENCE_MAX_HEAD_DIM:
            raise ValueError(f"channel_delta: head_dim={self.d} is above the scan kernel's {ops.RECURRENCE_MAX_HEAD_DIM}")
        self.qk, self.inner = self.kv_heads * self.d, self.heads * self.dv
        self.channels = 2 * self.qk + self.inner  # what passes the convolution: q | k | v
        self.b_col = self.channels  # set at load, behind the low-rank products' inner halves
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "b": "b_proj.weight", "a1": "a1.weight", "a2": "a2.weight",
                    "g1": "g1.weight", "g2": "g2.weight", "o": "o_proj.weight", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm.weight",
                    "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.ranks = (p.get("decay_rank"), p.get("gate_rank"))  # None: whatever the checkpoint holds
        self.w: dict[str, torch.Tensor] = {}
        self.a_cols = self.g_cols = (0, 0)

    def declare(self):
        nm, H = self.names, self.hidden
        return {
            nm["q"]: TensorDecl((self.qk, H)), nm["k"]: TensorDecl((self.qk, H)), nm["v"]: TensorDecl((self.inner, H)),
            nm["b"]: TensorDecl((self.heads, H)), nm["o"]: TensorDecl((H, self.inner)),
            nm["a1"]: TensorDecl((self.ranks[0], H)), nm["a2"]: TensorDecl((self.heads * self.d, self.ranks[0])),
            nm["g1"]: TensorDecl((self.ranks[1], H)), nm["g2"]: TensorDecl((self.inner, self.ranks[1])),
            nm["q_conv"]: TensorDecl((self.qk, self.taps), "vector32"), nm["k_conv"]: TensorDecl((self.qk, self.taps), "vector32"),
            nm["v_conv"]: TensorDecl((self.inner, self.taps), "vector32"),
            nm["A_log"]: TensorDecl((self.heads,), "vector32"), nm["dt_bias"]: TensorDecl((self.heads * self.d,), "vector32"),
            nm["norm"]: TensorDecl((self.dv,), "vector32"),
        }

    def load(self, tensors):
        t = {role: tensors[name] for role, name in self.names.items()}
        self.a_cols = (self.channels, self.channels + t["a1"].shape[0])
        self.g_cols = (self.a_cols[1], self.a_cols[1] + t["g1"].shape[0])
        self.b_col = self.g_cols[1]  # the betas' columns come last: the low-rank products' inner halves start on even columns
        self.w = {
            "in": torch.cat([t["q"], t["k"], t["v"], t["a1"], t["g1"], t["b"]], 0).contiguous(),
            "conv": torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], 0).t().contiguous(),  # [taps, channels]
            "a2": t["a2"], "g2": t["g2"], "A_log": t["A_log"], "dt_bias": t["dt_bias"], "o": t["o"],
            "norm": t["norm"].repeat(self.heads).contiguous(),  # the heads share the weight; the kernel reads one per column
        }

    def cache_need(self):
        return (StateNeed((self.heads, self.dv, self.d), torch.float32), StateNeed((self.taps - 1, self.channels), self.env.dtype))

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        w = self.w
        n = x.shape[0]
        state, conv_state = cache.states
        u = project(x, w["in"])  # q | k | v | a1 | g1 | b
        qkv = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv_silu(qkv, u, 0, w["conv"], None, conv_state, batch.seq_of_token, batch.q_start, batch.state_slot)
        if self.taps > 1:
            ops.conv_state_update(conv_state, u, 0, batch.q_start, batch.state_slot)
        a = project(u[:, self.a_cols[0] : self.a_cols[1]], w["a2"])  # [n, heads * head_dim]; the library reads the column slice in place
        g = project(u[:, self.g_cols[0] : self.g_cols[1]], w["g2"])  # [n, heads * value_dim]
        rows = torch.empty((n, _recurrence_row(self.kv_heads, self.heads, self.d, self.dv)), dtype=torch.float32, device=x.device)
        ops.channel_delta_prep(rows, qkv, u, self.b_col, a, w["dt_bias"], w["A_log"], self.heads, self.kv_heads, self.d, self.dv, self.unit_eps)
        o = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        ops.decay_recurrence(o, rows, state, batch.q_start, batch.state_slot, self.kv_heads, "delta", None, max_len=batch.max_q_len)
        gated = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        ops.gated_group_rmsnorm(gated, o, g, 0, w["norm"], self.heads, self.eps, gate_after=True, gate="sigmoid")
        return project(gated, w["o"])
