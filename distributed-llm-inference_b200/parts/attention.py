"""Attention over the paged cache: grouped-query, with a sink, and over a cached latent."""

from __future__ import annotations

import math

import torch

from ..cache.needs import PagedKVNeed
from ..kernels import attention as attn_kernels
from ..kernels import ops
from ..cache.needs import StateNeed
from ..kernels.gemm import heads_product, last_product, project, project_bias
from ..weights.loader import TensorDecl
from .base import Part, build_part, register_part, tensor_name


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q, k, v projections, position encoding, causal attention of each token over the keys of
    its own sequence at positions <= its own (optionally only the last ``window``), output
    projection (src/dli/model/llama.py:72-76,94-95,147-177).  Query head h reads kv head
    h // (num_heads / num_kv_heads).  The three projection matrices are read by their own
    names and laid side by side at load, so one product yields q | k | v.

    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window, position (PartSpec).
    """

    graph_capturable = True
    takes_scaled_rows = True  # the input only goes to the q | k | v product
    defer_output = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        if self.nh % self.nkv:
            raise ValueError(f"num_heads={self.nh} is not a multiple of num_kv_heads={self.nkv}")
        self.position = build_part("position", p["position"], env)
        self.wqkv: torch.Tensor | None = None
        self.wo: torch.Tensor | None = None

    def children(self):
        return [self.position]

    def declare(self):
        px, H, d = self.spec.prefix, self.hidden, self.d
        return {
            px + "q_proj.weight": TensorDecl((self.nh * d, H)),
            px + "k_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "v_proj.weight": TensorDecl((self.nkv * d, H)),
            px + "o_proj.weight": TensorDecl((H, self.nh * d)),
        }

    def load(self, tensors):
        px = self.spec.prefix
        self.wqkv = torch.cat([tensors[px + "q_proj.weight"], tensors[px + "k_proj.weight"], tensors[px + "v_proj.weight"]], 0).contiguous()
        self.wo = tensors[px + "o_proj.weight"]

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        """Into how many runs the decode kernel cuts each sequence's keys (1: not at all)."""
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.d, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        encode = getattr(self.position, "project_and_encode", None)
        if encode is not None:  # the position part may fuse the projection with its encoding
            q = encode(x, self.wqkv, batch, cache, self.nh, self.nkv, cache.writes)
        else:
            q = self.position.rotate_and_store(project(x, self.wqkv), batch, cache, self.nh, self.nkv, cache.writes)
        out = torch.empty((x.shape[0], self.nh * self.d), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)))
        return last_product(out, self.wo, self.defer_output)


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    """Causal grouped-query attention whose softmax has a sink, with options other designs can switch:

    * ``sink`` (a score, or None): exp(sink) is added to every softmax denominator and carries no value,
      p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)), so a token may attend to nothing;
    * ``qk_norm_eps`` (or None): q and k are each divided by the RMS of their whole projection (all heads
      together, before they are cut into heads) and multiplied by a weight of that size, before the position
      encoding;
    * ``values``: ``"keys"`` — the values are the keys as projected (before norm and rotation; no value matrix)
      — or ``"projected"`` (a value matrix of its own);
    * ``gate``: the concatenated heads are multiplied by sigmoid(Wg x) before the output projection.

    One product yields q | k (| v) (| g); one kernel norms, rotates and writes the cache (the position part's
    ``norm_rotate_and_store``); the framework's attention kernels run with their sink argument.
    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window, position (PartSpec), sink,
    qk_norm_eps, values, gate, tensors (names of q, k, v, g, o, q_norm, k_norm)."""

    graph_capturable = True
    takes_scaled_rows = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.sink = None if p.get("sink") is None else float(p["sink"])
        self.qk_norm_eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.values_from_keys = p.get("values", "projected") == "keys"
        self.gated = bool(p.get("gate", False))
        if p.get("values", "projected") not in ("keys", "projected"):
            raise ValueError(f"values={p['values']!r} (keys, projected)")
        if self.nh % self.nkv:
            raise ValueError(f"num_heads={self.nh} is not a multiple of num_kv_heads={self.nkv}")
        self.position = build_part("position", p["position"], env)
        if not hasattr(self.position, "norm_rotate_and_store"):
            raise ValueError(f"position part {p['position'].kind!r} cannot follow a norm over the whole projection")
        self.names = {role: tensor_name(spec, role, default) for role, default in (
            ("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("g", "g_proj.weight"), ("o", "o_proj.weight"),
            ("q_norm", "q_norm.weight"), ("k_norm", "k_norm.weight"))}
        self.w_in: torch.Tensor | None = None
        self.wo: torch.Tensor | None = None
        self.wq_norm = self.wk_norm = None
        self.gate_col = (self.nh + (1 if self.values_from_keys else 2) * self.nkv) * self.d

    def children(self):
        return [self.position]

    def declare(self):
        H, d, nm = self.hidden, self.d, self.names
        out = {nm["q"]: TensorDecl((self.nh * d, H)), nm["k"]: TensorDecl((self.nkv * d, H)), nm["o"]: TensorDecl((H, self.nh * d))}
        if not self.values_from_keys:
            out[nm["v"]] = TensorDecl((self.nkv * d, H))
        if self.gated:
            out[nm["g"]] = TensorDecl((self.nh * d, H))
        if self.qk_norm_eps is not None:
            out[nm["q_norm"]] = TensorDecl((self.nh * d,), "vector32")
            out[nm["k_norm"]] = TensorDecl((self.nkv * d,), "vector32")
        return out

    def load(self, tensors):
        nm = self.names
        rows = [tensors[nm["q"]], tensors[nm["k"]]]
        if not self.values_from_keys:
            rows.append(tensors[nm["v"]])
        if self.gated:
            rows.append(tensors[nm["g"]])
        self.w_in = torch.cat(rows, 0).contiguous()
        self.wo = tensors[nm["o"]]
        if self.qk_norm_eps is not None:
            self.wq_norm, self.wk_norm = tensors[nm["q_norm"]], tensors[nm["k_norm"]]

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.d, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        proj = project(x, self.w_in)
        q = self.position.norm_rotate_and_store(proj, self.wq_norm, self.wk_norm, self.qk_norm_eps or 0.0, batch, cache, self.nh, self.nkv,
                                                cache.writes, self.values_from_keys)
        out = torch.empty((x.shape[0], self.nh * self.d), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)),
                                     sink=self.sink)
        if self.gated:
            ops.sigmoid_gate(out, proj[:, self.gate_col : self.gate_col + self.nh * self.d])
        return project(out, self.wo)


@register_part("mixer", "conv_attention")
class ConvAttention(Part):
    """Causal grouped-query softmax attention whose q, k and v pass a short causal convolution over time right after their
    projections, with options other designs can switch:

    * ``bias``: q, k, v and the output projection have biases (added in the projection, before the convolution);
    * ``conv_taps``: taps of the per-channel convolution without bias or activation (1: a scale per channel); a request
      keeps the last taps - 1 projected rows in its state slot;
    * ``rotary_dim`` / ``theta``: rotate-half rotation of the first rotary_dim dimensions of every q and k head;
    * ``qk_unit_eps`` (or None): AFTER the rotation every q and k head is divided by its root mean square (no weight);
    * ``value_dim``: the values' size may differ from the keys'.  Pages hold rows of max(head_dim, value_dim) numbers, the
      shorter of keys and values padded with zeros, so every attention kernel of the engine serves; the output
      projection's matrix is padded with zero columns to match, once, at load.

    One product yields q | k | v; one kernel convolves; one kernel rotates, norms and writes the pages.
    params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, conv_taps, scale, window, bias, qk_unit_eps, rotary_dim,
    theta, tensors (names of q, k, v, o, q_bias, k_bias, v_bias, o_bias, q_conv, k_conv, v_conv)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.dv = int(p.get("value_dim") or self.d)
        self.row = max(self.d, self.dv)  # what a page keeps per token and KV head, for keys and for values
        self.taps = int(p.get("conv_taps") or 1)
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.bias = bool(p.get("bias", False))
        self.unit_eps = None if p.get("qk_unit_eps") is None else float(p["qk_unit_eps"])
        self.rotary_dim = int(p.get("rotary_dim") or 0)
        if self.nh % self.nkv or self.rotary_dim % 2 or self.rotary_dim > self.d or self.taps < 1:
            raise ValueError("conv_attention: num_heads must be a multiple of num_kv_heads, rotary_dim even and at most head_dim, conv_taps >= 1")
        self.inv_freq = None
        if self.rotary_dim:
            from .rotary import inverse_frequencies

            self.inv_freq = inverse_frequencies({"rotary_dim": self.rotary_dim, "theta": float(p["theta"])}).to(env.device)
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_bias": "q_proj.bias",
                    "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight",
                    "v_conv": "v_conv.weight"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.sizes = {"q": self.nh * self.d, "k": self.nkv * self.d, "v": self.nkv * self.dv}
        self.channels = sum(self.sizes.values())
        self.w_in = self.b_in = self.w_conv = self.wo = self.bo = None

    def declare(self):
        nm, H = self.names, self.hidden
        out = {nm["o"]: TensorDecl((H, self.nh * self.dv))}
        for role, size in self.sizes.items():
            out[nm[role]] = TensorDecl((size, H))
            out[nm[role + "_conv"]] = TensorDecl((size, self.taps), "vector32")
            if self.bias:
                out[nm[role + "_bias"]] = TensorDecl((size,))
        if self.bias:
            out[nm["o_bias"]] = TensorDecl((H,))
        return out

    def load(self, tensors):
        nm = self.names
        self.w_in = torch.cat([tensors[nm[r]] for r in ("q", "k", "v")], 0).contiguous()
        self.w_conv = torch.cat([tensors[nm[r + "_conv"]] for r in ("q", "k", "v")], 0).t().contiguous()  # [taps, channels]
        wo = tensors[nm["o"]]
        if self.row != self.dv:  # the attention kernels leave rows of ``row`` numbers per head: zero columns where the padding lies
            padded = torch.zeros((self.hidden, self.nh, self.row), dtype=wo.dtype, device=wo.device)
            padded[:, :, : self.dv] = wo.view(self.hidden, self.nh, self.dv)
            wo = padded.view(self.hidden, self.nh * self.row)
        self.wo = wo.contiguous()
        if self.bias:
            self.b_in = torch.cat([tensors[nm[r + "_bias"]] for r in ("q", "k", "v")], 0).contiguous()
            self.bo = tensors[nm["o_bias"]]

    def cache_need(self):
        return (PagedKVNeed(self.nkv, self.row, self.window), StateNeed((self.taps - 1, self.channels), self.env.dtype))

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        return attn_kernels.decode_splits(num_seqs, self.nh, self.nkv, self.row, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        n = x.shape[0]
        conv_state = cache.states[0]
        proj = project_bias(x, self.w_in, self.b_in)
        mixed = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv_silu(mixed, proj, 0, self.w_conv, None, conv_state, batch.seq_of_token, batch.q_start, batch.state_slot, activation=False)
        if self.taps > 1:
            ops.conv_state_update(conv_state, proj, 0, batch.q_start, batch.state_slot)
        group = batch.group(cache.group)
        q = torch.empty((n, self.nh * self.row), dtype=x.dtype, device=x.device)
        ops.rotary_unit_store(q, mixed, batch.positions, self.inv_freq, group.slots if cache.writes else None, cache.k if cache.writes else None,
                              cache.v if cache.writes else None, self.nh, self.nkv, self.d, self.dv, self.rotary_dim, self.unit_eps, cache.page_size)
        out = torch.empty((n, self.nh * self.row), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(out, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)))
        return project_bias(out, self.wo, self.bo)


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """Attention whose keys and values are both made from one small cached vector per token (a latent).

    The down projection yields ``kv_rank`` numbers, RMS-normed with a plain weight: the latent c, and — when
    ``rot_dim`` > 0 — ``rot_dim`` more, one key part that is rotated by the token's position and shared by all heads.
    Head a's keys are W_uk[a] c (``head_dim`` numbers) followed by the rotated part, its values W_uv[a] c
    (``value_dim`` numbers); its queries are laid out the same way, [head_dim plain | rot_dim rotated].  Only c and the
    rotated key part are cached: one row of kv_rank + rot_dim numbers per token, one "KV head".

    The up projections are never applied to the cache.  Since q . (W_uk c) = (W_uk^T q) . c, each head's plain query
    is carried into the latent space (a product of head_dim x kv_rank per head) and the framework's paged attention
    kernels run as multi-query attention over the cached rows, the values being the rows' first kv_rank numbers; the
    weighted sum of latents then goes through W_uv head by head.  Causal, with an optional sliding ``window``; with
    ``gate`` the concatenated heads are multiplied by sigmoid(W_g x) before the output projection.

    One product yields q | down | g; one kernel norms the latent, rotates, writes the cache row and places the rotated
    query parts behind the latent-space queries.
    ``rotary_pairing``: ``"half"`` (dimension i turns with i + rotary_dim / 2) or ``"neighbours"`` (2i with 2i + 1).  A
    score only sees the rotated parts through their dot product, so for neighbouring pairs the rows of W_q's and W_dkv's
    rotated parts are put into the half layout once, at load, and the same kernel serves both.  ``rotary_scaling`` (factor,
    original, fast, slow): YaRN frequencies and the factor on cosines and sines (``paired_rotary_frequencies``).
    ``head_sinks``: a learned score per head (tensor ``sink``) whose exponential joins every softmax denominator of that
    head and carries no value.

    params: hidden_size, num_heads, head_dim, rot_dim, value_dim, kv_rank, scale, window, gate, eps, rotary_dim (how
    many of the rot_dim dimensions are rotated), theta, rotary_pairing, rotary_scaling, head_sinks, tensors (names of q,
    dkv, dkv_norm, uk, uv, g, o, sink)."""

    graph_capturable = True
    takes_scaled_rows = False

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.d, self.dr = int(p["num_heads"]), int(p["head_dim"]), int(p.get("rot_dim") or 0)
        self.dv, self.rank = int(p["value_dim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.gated = bool(p.get("gate", False))
        self.eps = float(p["eps"])
        self.rotary_dim = int(p.get("rotary_dim", self.dr)) if self.dr else 0
        if self.rotary_dim % 2 or self.rotary_dim > self.dr:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most rot_dim={self.dr}")
        self.row = self.rank + self.dr  # what a token keeps in the cache, and the size of a query in the latent space
        self.inv_freq = None
        self.amp = 1.0
        self.pairing = p.get("rotary_pairing", "half")
        if self.pairing not in ("half", "neighbours"):
            raise ValueError(f"rotary_pairing={self.pairing!r} (half, neighbours)")
        if self.rotary_dim and (p.get("rotary_scaling") or self.pairing == "neighbours"):
            freq, self.amp = paired_rotary_frequencies(self.rotary_dim, float(p["theta"]), p.get("rotary_scaling"))
            self.inv_freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(env.device)
        elif self.rotary_dim:
            from .rotary import inverse_frequencies

            self.inv_freq = inverse_frequencies({"rotary_dim": self.rotary_dim, "theta": float(p["theta"])}).to(env.device)
        self.head_sinks = bool(p.get("head_sinks", False))
        self.sinks = None
        self.names = {role: tensor_name(spec, role, default) for role, default in (
            ("q", "q_proj.weight"), ("dkv", "kv_down_proj.weight"), ("dkv_norm", "kv_norm.weight"), ("uk", "k_up_proj.weight"),
            ("uv", "v_up_proj.weight"), ("g", "g_proj.weight"), ("o", "o_proj.weight"), ("sink", "sinks"))}
        self.q_cols = self.nh * (self.d + self.dr)
        self.gate_col = self.q_cols + self.row
        self.w_in = self.w_uk = self.w_uv = self.wo = self.w_norm = None

    def declare(self):
        H, nm = self.hidden, self.names
        out = {nm["q"]: TensorDecl((self.q_cols, H)), nm["dkv"]: TensorDecl((self.row, H)),
               nm["dkv_norm"]: TensorDecl((self.rank,), "vector32"), nm["uk"]: TensorDecl((self.nh * self.d, self.rank)),
               nm["uv"]: TensorDecl((self.nh * self.dv, self.rank)), nm["o"]: TensorDecl((H, self.nh * self.dv))}
        if self.gated:
            out[nm["g"]] = TensorDecl((self.nh * self.dv, H))
        if self.head_sinks:
            out[nm["sink"]] = TensorDecl((self.nh,), "vector32")
        return out

    def _half_layout(self, w: torch.Tensor, heads: int, plain: int) -> torch.Tensor:
        """Rows of a projection whose heads are [plain | rot_dim]: the first rotary_dim rows of every rotated part, stored as
        neighbouring pairs (2i, 2i + 1), reordered to evens then odds, so that pair i sits at (i, i + rotary_dim / 2)."""
        r = self.rotary_dim
        order = torch.cat([torch.arange(0, r, 2), torch.arange(1, r, 2), torch.arange(r, self.dr)]).to(w.device)
        per = plain + self.dr
        v = w.view(heads, per, w.shape[1]).clone()
        v[:, plain:] = v[:, plain:][:, order]
        return v.view(heads * per, w.shape[1])

    def load(self, tensors):
        nm = self.names
        wq, wd = tensors[nm["q"]], tensors[nm["dkv"]]
        if self.pairing == "neighbours" and self.rotary_dim:
            wq = self._half_layout(wq, self.nh, self.d)
            wd = torch.cat([wd[: self.rank], self._half_layout(wd[self.rank :], 1, 0)], 0)
        rows = [wq, wd] + ([tensors[nm["g"]]] if self.gated else [])
        if self.head_sinks:
            self.sinks = tensors[nm["sink"]]
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_uk = tensors[nm["uk"]].view(self.nh, self.d, self.rank)  # q_latent[a] = q_plain[a] W_uk[a]
        self.w_uv = tensors[nm["uv"]].view(self.nh, self.dv, self.rank).transpose(1, 2).contiguous()  # o[a] = o_latent[a] W_uv[a]^T
        self.wo, self.w_norm = tensors[nm["o"]], tensors[nm["dkv_norm"]]

    def cache_need(self):
        return PagedKVNeed(1, self.row, self.window, values_in_keys=True)

    def decode_launch_key(self, num_seqs: int, max_kv_len: int, page_size: int):
        return attn_kernels.decode_splits(num_seqs, self.nh, 1, self.row, page_size, max_kv_len)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        n = x.shape[0]
        proj = project(x, self.w_in)
        group = batch.group(cache.group)
        # the latent-space queries [n, heads, kv_rank + rot_dim]: the kernel fills the rotated tails, the product the rest
        q = torch.empty((n, self.nh * self.row), dtype=x.dtype, device=x.device)
        ops.latent_prep(q, proj, self.w_norm, self.eps, batch.positions, self.inv_freq, group.slots if cache.writes else None,
                        cache.k if cache.writes else None, self.nh, self.d, self.dr, self.rank, self.rotary_dim, cache.page_size, amp=self.amp)
        heads_product(proj[:, : self.q_cols].view(n, self.nh, self.d + self.dr)[:, :, : self.d], self.w_uk,
                      q.view(n, self.nh, self.row)[:, :, : self.rank])
        latent = torch.empty((n, self.nh * self.row), dtype=x.dtype, device=x.device)
        attn_kernels.paged_attention(latent, q, cache, batch, self.nh, self.scale, self.window, splits=batch.launch_keys.get(id(self)),
                                     sink=self.sinks)
        out = torch.empty((n, self.nh * self.dv), dtype=x.dtype, device=x.device)
        heads_product(latent.view(n, self.nh, self.row)[:, :, : self.rank], self.w_uv, out.view(n, self.nh, self.dv),
                      gate=proj[:, self.gate_col : self.gate_col + self.nh * self.dv] if self.gated else None)
        return project(out, self.wo)


def paired_rotary_frequencies(dims: int, base: float, scaling: dict | None = None) -> tuple[list[float], float]:
    """Frequencies f_i = base^(-2i/dims), i < dims / 2, of a rotation that pairs dimension 2i with 2i + 1, and the factor on its
    cosines and sines.  With ``scaling`` (factor, original, fast, slow) the YaRN correction: dimensions whose wavelength fits
    the original context many times keep their frequency, those that turn less than ``slow`` times in it are divided by
    ``factor``, with a linear ramp between, and cosine and sine are multiplied by 0.1 ln(factor) + 1."""
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_to_dim(turns: float) -> float:  # the (fractional) pair index whose wavelength fits the original context ``turns`` times
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns_to_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@register_part("mixer", "diff_attention")
class DiffAttention(Part):
    """Differential attention: every query head carries two attention maps over the same values, combined by a difference.

    q has heads x 2 x head_dim rows and k kv_heads x 2 x head_dim, head by head as [map 1 | map 2]; v has kv_heads x value_dim.
    Every map of every head of q and k is RMS-normed over head_dim with a weight of that size (one for q, one for k) and then
    rotated on its first ``rotary_dim`` dimensions, dimension 2i paired with 2i + 1 (``paired_rotary_frequencies``).  Causal,
    with an optional sliding ``window`` that always keeps a sequence's first ``keep_first`` tokens.  With a1, a2 the two
    maps' outputs of a head and lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (one number for the layer):

        o = a1 - lambda a2;    o <- o / rms(o) * (1 - diff);    o <- o * sigmoid(W_g x)[head];    out = W_o [o of all heads]

    A layer with ``own_kv`` false has no k and v tensors: its run step reads another step's cache (keys as that layer wrote
    them, normed and rotated) with its own queries, mask and everything else.  A cached token is one key row of
    2 head_dim numbers and one value row of value_dim numbers per KV head.  ``retain_window`` / ``retain_first`` say what the
    cache has to keep (the widest window and most first tokens among the layers that read it).

    One product yields q | k | v | g; one kernel norms, rotates and writes the cache; one kernel attends (both maps, the
    difference, the head's norm and the gate).
    params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window, keep_first, diff, eps, rotary_dim, theta,
    rotary_scaling, own_kv, retain_window, retain_first, tensors (names of q, k, v, g, o, q_norm, k_norm, lq1, lk1, lq2, lk2)."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.d, self.dv = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"]), int(p["value_dim"])
        self.scale, self.diff, self.eps = float(p["scale"]), float(p["diff"]), float(p["eps"])
        self.window = int(p["window"]) if p.get("window") else None
        self.keep_first = int(p.get("keep_first") or 0)
        self.own_kv = bool(p.get("own_kv", True))
        self.retain_window = p.get("retain_window", self.window)
        self.retain_first = int(p.get("retain_first", self.keep_first))
        self.rot = int(p.get("rotary_dim") or 0)
        if self.nh % self.nkv or self.rot % 2 or self.rot > self.d:
            raise ValueError("diff_attention: num_heads must be a multiple of num_kv_heads, rotary_dim even and at most head_dim")
        freq, self.amp = paired_rotary_frequencies(self.rot, float(p["theta"]), p.get("rotary_scaling")) if self.rot else ([0.0], 1.0)
        self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(env.device)
        defaults = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight", "o": "o_proj.weight",
                    "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2",
                    "lk2": "lambda_k2"}
        self.names = {role: tensor_name(spec, role, default) for role, default in defaults.items()}
        self.q_cols = self.nh * 2 * self.d
        self.k_col = self.q_cols if self.own_kv else -1
        self.v_col = self.q_cols + self.nkv * 2 * self.d if self.own_kv else -1
        self.g_col = self.q_cols + (self.nkv * (2 * self.d + self.dv) if self.own_kv else 0)
        self.w_in = self.wo = self.wq_norm = self.wk_norm = None
        self.lam = self.diff

    def declare(self):
        nm, H, d = self.names, self.hidden, self.d
        out = {nm["q"]: TensorDecl((self.q_cols, H)), nm["g"]: TensorDecl((self.nh, H)), nm["o"]: TensorDecl((H, self.nh * self.dv)),
               nm["q_norm"]: TensorDecl((d,), "vector32")}
        out.update({nm[r]: TensorDecl((d,), "vector32") for r in ("lq1", "lk1", "lq2", "lk2")})
        if self.own_kv:
            out.update({nm["k"]: TensorDecl((self.nkv * 2 * d, H)), nm["v"]: TensorDecl((self.nkv * self.dv, H)),
                        nm["k_norm"]: TensorDecl((d,), "vector32")})
        return out

    def load(self, tensors):
        nm = self.names
        rows = [tensors[nm["q"]]] + ([tensors[nm["k"]], tensors[nm["v"]]] if self.own_kv else []) + [tensors[nm["g"]]]
        self.w_in = torch.cat(rows, 0).contiguous()
        self.wo, self.wq_norm = tensors[nm["o"]], tensors[nm["q_norm"]]
        self.wk_norm = tensors[nm["k_norm"]] if self.own_kv else None
        l1 = (tensors[nm["lq1"]].double() * tensors[nm["lk1"]].double()).sum().item()
        l2 = (tensors[nm["lq2"]].double() * tensors[nm["lk2"]].double()).sum().item()
        self.lam = math.exp(l1) - math.exp(l2) + self.diff

    def cache_need(self):
        return PagedKVNeed(self.nkv, 2 * self.d, self.retain_window, value_dim=self.dv,
                           keep_first=self.retain_first if self.retain_window is not None else 0)

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        n = x.shape[0]
        if cache.writes != self.own_kv:
            raise RuntimeError("diff_attention: a layer with keys and values of its own writes its cache, one without reads another's")
        proj = project(x, self.w_in)  # q | k | v | g
        group = batch.group(cache.group)
        q = torch.empty((n, self.q_cols), dtype=x.dtype, device=x.device)
        ops.diff_prep(q, proj, self.k_col, self.v_col, self.wq_norm, self.wk_norm, self.eps, batch.positions, self.freq, self.amp,
                      group.slots if self.own_kv else None, cache.k if self.own_kv else None, cache.v if self.own_kv else None,
                      self.nh, self.nkv, self.d, self.dv, self.rot, cache.page_size)
        out = torch.empty((n, self.nh * self.dv), dtype=x.dtype, device=x.device)
        attn_kernels.diff_attention(out, q, cache, batch, proj[:, self.g_col : self.g_col + self.nh], self.nh, self.scale, self.window,
                                    self.keep_first, self.lam, 1.0 - self.diff, self.eps)
        return project(out, self.wo)
