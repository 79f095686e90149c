"""Stand-ins for the kernels, written with torch on the CPU, for tests of the engine's host side.

The product has no CPU path.  These functions exist only so that the Python above the kernels
(parts and their wiring, batch building, cache pools, the step function, scheduler, engine, the
step launched ahead) can run end to end in the CPU test suite and be compared with the plain
implementation.  Each one restates what its kernel's wrapper documents (kernels/ops.py); none is
used by the GPU tests, which run the real kernels.  ``patched()`` swaps them in.
"""

from __future__ import annotations

import contextlib

import numpy as np
import torch

from dli_b200.engine import graphs as graphs_mod
from dli_b200.engine import runner as runner_mod
from dli_b200.kernels import gemm, ops
from dli_b200.parts import model as model_mod
from tests.plain import llama_plain as plain


def embedding(h, table, ids):
    h.copy_(table[ids.long()].float())


def patch_tokens(ids, source, src):
    pick = src >= 0
    ids[pick] = source[src[pick].long()]


def copy_page(pool, src, dst):
    pool[:, dst] = pool[:, src]


def add_rmsnorm(y, h, delta, weight, eps, rows=None):
    if rows is None:
        if delta is not None:
            h += delta.float()
        x = h
    else:
        x = h[rows.long()] + (delta[rows.long()].float() if delta is not None else 0.0)
    y.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(y.dtype))


def rotary_table(positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], -1)


def rotary_store(qkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size,
                 write_kv=True, table=None):
    n = qkv.shape[0]
    heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)
    if rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        qk = heads[:, : num_heads + num_kv_heads, :rotary_dim].float()
        lo, hi = qk[..., :half].clone(), qk[..., half:].clone()
        heads[:, : num_heads + num_kv_heads, :half] = (lo * cos - hi * sin).to(qkv.dtype)
        heads[:, : num_heads + num_kv_heads, half:rotary_dim] = (hi * cos + lo * sin).to(qkv.dtype)
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = heads[:, num_heads : num_heads + num_kv_heads]
        v_pool[page, :, off, :] = heads[:, num_heads + num_kv_heads :]


def _gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z**3)))


def silu_mul(out, gate_up, tiled=False, activation="silu", limit=0.0, up_shift=0.0):
    n, inter = out.shape
    if tiled:
        blocks = gate_up.view(n, inter // 64, 2, 64)
        gate, up = blocks[:, :, 0].reshape(n, inter), blocks[:, :, 1].reshape(n, inter)
    else:
        gate, up = gate_up[:, :inter], gate_up[:, inter:]
    g, u = gate.float(), up.float()
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    act = {"silu": lambda: g / (1 + torch.exp(-g)), "gelu_tanh": lambda: _gelu_tanh(g), "quick_gelu": lambda: g / (1 + torch.exp(-1.702 * g))}[activation]()
    out.copy_((act * (u + up_shift)).to(out.dtype))


def add_rmsnorm_pair(y1, y2, h, a, b, w1, w2, eps, rows=None):
    idx = slice(None) if rows is None else rows.long()
    x = h[idx]
    if a is not None or b is not None:
        x = x + ((a[idx].float() if a is not None else 0.0) + (b[idx].float() if b is not None else 0.0))
        if rows is None:
            h.copy_(x)
    unit = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    y1.copy_((unit * w1).to(y1.dtype))
    if y2 is not None:
        y2.copy_((unit * w2).to(y2.dtype))


def scale_softcap(logits, scale, cap):
    logits *= scale
    if cap > 0:
        logits.copy_(cap * torch.tanh(logits / cap))


def paged_attention_simt(out, qkv, k_pool, v_pool, block_tables, seq_of_token, positions, num_heads, scale, window=None, sink=None):
    n = out.shape[0]
    _, nkv, page_size, d = k_pool.shape
    fan = num_heads // nkv
    q = qkv[:, : num_heads * d].view(n, num_heads, d).float()
    for t in range(n):
        p = int(positions[t])
        first = max(0, p - window + 1) if window else 0
        keys = torch.arange(first, p + 1)
        table = block_tables[int(seq_of_token[t])]
        pages = table[(keys // page_size).long()].long()
        assert (pages >= 0).all(), "attention reads a page that was given back"
        k = k_pool[pages, :, (keys % page_size).long(), :].float()  # [keys, nkv, d]
        v = v_pool[pages, :, (keys % page_size).long(), :].float()
        k, v = k.repeat_interleave(fan, 1), v.repeat_interleave(fan, 1)  # [keys, nh, d]
        s = torch.einsum("hd,khd->hk", q[t], k) * scale
        if isinstance(sink, torch.Tensor):  # a learned score per head
            s = torch.cat([s, sink.float().view(num_heads, 1)], -1)
        elif sink is not None:  # one more term in the denominator, without a value
            s = torch.cat([s, torch.full((num_heads, 1), float(sink))], -1)
        w = torch.softmax(s, -1)[:, : keys.numel()]
        out[t] = torch.einsum("hk,khd->hd", w, v).reshape(-1).to(out.dtype)


def _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window, sink=None):
    """The bfloat16 attention kernels' common contract: sequences [seq0, seq0 + num_seqs); a sequence's
    tokens sit in rows q_start[s] .. q_start[s + 1] at positions kv_len[s] - q_len .. kv_len[s] - 1."""
    rows, seqs, pos = [], [], []
    for s in range(seq0, seq0 + num_seqs):
        lo, hi = int(q_start[s]), int(q_start[s + 1])
        rows += range(lo, hi)
        seqs += [s] * (hi - lo)
        pos += range(int(kv_len[s]) - (hi - lo), int(kv_len[s]))
    if not rows:
        return
    idx = torch.tensor(rows)
    part = torch.empty((len(rows), out.shape[1]), dtype=out.dtype)
    paged_attention_simt(part, qkv[idx], k_pool, v_pool, block_tables, torch.tensor(seqs, dtype=torch.int32),
                         torch.tensor(pos, dtype=torch.int32), num_heads, scale, window, sink)
    out[idx] = part


def paged_attention_mma(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, max_q_len, first_row, num_heads, scale,
                        window=None, splits=1, scratch=None, sink=None):
    assert splits == 1 or (max_q_len == 1 and scratch is not None)
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window, sink)


def paged_decode_tma(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, first_row, num_heads, scale,
                     window=None, splits=1, scratch=None, max_kv_len=0, sink=None):
    assert splits == 1 or scratch is not None
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window, sink)


def paged_prefill_tc(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, max_q_len, num_heads, scale,
                     window=None, query_tiles=0, sink=None):
    _attend(out, qkv, k_pool, v_pool, block_tables, q_start, kv_len, seq0, num_seqs, num_heads, scale, window, sink)


# ---- layer norm around the residual stream, activations


def _ln(x, eps):
    mu = x.mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(((x - mu) ** 2).mean(-1, keepdim=True) + eps)


def post_add_layernorm(y, h, a, w_post, w_pre, eps_post, eps_pre, rows=None):
    idx = slice(None) if rows is None else rows.long()
    v = h[idx]
    if a is not None:
        v = v + _ln(a[idx].float(), eps_post) * w_post
        if rows is None:
            h.copy_(v)
    if y is not None:
        y.copy_((_ln(v, eps_pre) * w_pre).to(y.dtype))


def stream_reinject(h, table, ids, vec):
    if table is not None:
        h += table[ids.long()].float()
    if vec is not None:
        h += vec


def activation(x, kind):
    z = x.float()
    if kind == "relu2":
        z = torch.relu(z) ** 2
    elif kind == "gelu_tanh":
        z = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z**3)))
    elif kind == "tanh":
        z = torch.tanh(z)
    else:
        z = z / (1 + torch.exp(-z))
    x.copy_(z.to(x.dtype))
    return x


# ---- between an attention mixer's projections and its kernel


def qk_norm_rotary_store(proj, wq, wk, eps, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim,
                         page_size, write_kv=True, values_from_keys=True):
    n = proj.shape[0]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    q, k = proj[:, :nq].float(), proj[:, nq : nq + nk].float()
    v = proj[:, nq : nq + nk] if values_from_keys else proj[:, nq + nk : nq + 2 * nk]
    if wq is not None:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * wq
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * wk
    qk = torch.cat([q, k], -1).view(n, num_heads + num_kv_heads, head_dim).clone()
    if rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        lo, hi = qk[..., :half].clone(), qk[..., half:rotary_dim].clone()
        qk[..., :half] = lo * cos - hi * sin
        qk[..., half:rotary_dim] = hi * cos + lo * sin
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = qk[:, num_heads:].to(k_pool.dtype)
        v_pool[page, :, off, :] = v.reshape(n, num_kv_heads, head_dim).to(v_pool.dtype)
    return qk[:, :num_heads].reshape(n, nq).to(proj.dtype)


def latent_prep(q_out, proj, w_norm, eps, positions, inv_freq, slots, k_pool, num_heads, head_dim, rot_dim, kv_rank, rotary_dim, page_size, amp=1.0):
    n = proj.shape[0]
    qc = num_heads * (head_dim + rot_dim)
    down = proj[:, qc : qc + kv_rank + rot_dim].float()
    c = down[:, :kv_rank]
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * w_norm
    turn = torch.cat([proj[:, :qc].float().view(n, num_heads, head_dim + rot_dim)[:, :, head_dim:], down[:, None, kv_rank:]], 1).clone()
    if rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :] * amp, ang.sin()[:, None, :] * amp
        lo, hi = turn[..., :half].clone(), turn[..., half:rotary_dim].clone()
        turn[..., :half] = lo * cos - hi * sin
        turn[..., half:rotary_dim] = hi * cos + lo * sin
    q_out.view(n, num_heads, kv_rank + rot_dim)[:, :, kv_rank:] = turn[:, :num_heads].to(q_out.dtype)
    if slots is not None:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, 0, off, :] = torch.cat([c, turn[:, num_heads]], -1).to(k_pool.dtype)


def heads_matvec(out, x, weight, gate=None):
    y = torch.einsum("nhi,hif->nhf", x.float(), weight.float())
    if gate is not None:
        y = y * torch.sigmoid(gate.float()).view(y.shape)
    out.copy_(y.to(out.dtype))


def sigmoid_gate(out, gate):
    out.copy_((out.float() * torch.sigmoid(gate.float())).to(out.dtype))


# ---- state-space mixer


def _silu(x):
    return x / (1 + torch.exp(-x))


def causal_conv_silu(out, u, col0, weight, bias, state, seq_of_token, q_start, state_slot, activation=True):
    n, C = out.shape
    taps = weight.shape[0]  # weight [taps, C]
    for t in range(n):
        s = int(seq_of_token[t])
        first, slot = int(q_start[s]), int(state_slot[s])
        acc = bias.clone() if bias is not None else torch.zeros(C)
        for j in range(taps):
            r = t - first - (taps - 1) + j
            x = u[first + r, col0 : col0 + C] if r >= 0 else state[slot, taps - 1 + r]
            acc = acc + weight[j] * x.float()
        out[t] = (_silu(acc) if activation else acc).to(out.dtype)


def conv_state_update(state, u, col0, q_start, state_slot):
    _, keep, C = state.shape
    for s in range(state_slot.numel()):
        first, last, slot = int(q_start[s]), int(q_start[s + 1]), int(state_slot[s])
        seen = torch.cat([state[slot], u[first:last, col0 : col0 + C]], 0)
        state[slot] = seen[seen.shape[0] - keep :]


def ssm_scan(y, xbc, u, dt_col, dt_bias, a_log, d_skip, state, q_start, state_slot, groups, max_len=0):
    _, heads, P, N = state.shape  # the state is kept transposed: [slot, head, p, n]
    inner = heads * P
    for s in range(state_slot.numel()):
        slot = int(state_slot[s])
        for t in range(int(q_start[s]), int(q_start[s + 1])):
            x = xbc[t, :inner].float().view(heads, P)
            B = xbc[t, inner : inner + groups * N].float().view(groups, N).repeat_interleave(heads // groups, 0)
            C = xbc[t, inner + groups * N :].float().view(groups, N).repeat_interleave(heads // groups, 0)
            dt = torch.nn.functional.softplus(u[t, dt_col : dt_col + heads].float() + dt_bias, threshold=20.0)
            decay = torch.exp(-torch.exp(a_log) * dt)
            state[slot] = decay[:, None, None] * state[slot] + x[:, :, None] * (dt[:, None] * B)[:, None, :]
            y[t] = (torch.einsum("hpn,hn->hp", state[slot], C) + d_skip[:, None] * x).reshape(-1)


def gated_group_rmsnorm(out, y, u, z_col, weight, parts, eps, gate_after=False, gate="silu"):
    n, inner = y.shape
    z = u[:, z_col : z_col + inner].float()
    gate = torch.sigmoid(z) if gate == "sigmoid" else _silu(z)
    g = (y if gate_after else y * gate).view(n, parts, inner // parts)
    g = g * torch.rsqrt((g * g).mean(-1, keepdim=True) + eps)
    out.copy_((g.view(n, inner) * weight * (gate if gate_after else 1.0)).to(out.dtype))


def delta_rule_scan(o, qkv, u, b_col, a_col, dt_bias, a_log, state, seq_of_token, q_start, state_slot, kv_heads, head_dim, unit_eps, max_len=0):
    _, heads, dv, d = state.shape  # the state is kept transposed: [slot, head, value column, key row]
    qk = kv_heads * d
    fan = heads // kv_heads
    for s in range(state_slot.numel()):
        slot = int(state_slot[s])
        for t in range(int(q_start[s]), int(q_start[s + 1])):
            q = qkv[t, :qk].float().view(kv_heads, d)
            k = qkv[t, qk : 2 * qk].float().view(kv_heads, d)
            v = qkv[t, 2 * qk :].float().view(heads, dv)
            q = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d**-0.5).repeat_interleave(fan, 0)
            k = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(fan, 0)
            beta = torch.sigmoid(u[t, b_col : b_col + heads].float())
            gamma = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(u[t, a_col : a_col + heads].float() + dt_bias, threshold=20.0))
            S = state[slot] * gamma[:, None, None]
            w = beta[:, None] * (v - torch.einsum("hvd,hd->hv", S, k))
            S = S + w[:, :, None] * k[:, None, :]
            state[slot] = S
            o[t] = torch.einsum("hvd,hd->hv", S, q).reshape(-1)


# ---- the decode matrix product and its epilogues (bfloat16 in, float32 sums)


def _sums(x, weight):
    """float32 sums of x W^T; x may be ops.ScaledRows, whose row factor is applied to the sums."""
    if isinstance(x, ops.ScaledRows):
        factor = torch.rsqrt(x.ssq.sum(-1, keepdim=True) / x.x.shape[1] + x.eps)
        return (x.x.float() @ weight.float().t()) * factor
    return x.float() @ weight.float().t()


def skinny_gemm_slices(tokens, features, in_features):
    return 1


def skinny_gemm(x, weight, out_dtype=torch.bfloat16, slices=None, out=None, max_stages=0):
    y = _sums(x, weight).to(out_dtype)
    if out is None:
        return y
    out.copy_(y)
    return out


def skinny_gemm_residual(x, weight, h, gain, eps, slices=None):
    h += _sums(x, weight)
    tokens, features = h.shape
    tiles = -(-features // 128)
    sq = torch.zeros((tokens, tiles * 128))
    sq[:, :features] = h * h
    return ops.ScaledRows((h * gain).to(torch.bfloat16), sq.view(tokens, tiles, 128).sum(-1), eps)


def skinny_gemm_swiglu(x, weight_tiled, activation="silu", limit=0.0, up_shift=0.0):
    y = _sums(x, weight_tiled)
    out = torch.empty((y.shape[0], y.shape[1] // 2), dtype=torch.bfloat16)
    silu_mul(out, y, True, activation, limit, up_shift)
    return out


def skinny_gemm_act(x, weight, kind):
    return activation(_sums(x, weight).to(torch.bfloat16), kind)


def skinny_gemm_rotary(x, wqkv, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv):
    qkv = _sums(x, wqkv)  # rotated in float32, rounded once (as the kernel's epilogue does)
    pools = (torch.empty_like(k_pool, dtype=torch.float32), torch.empty_like(v_pool, dtype=torch.float32)) if write_kv else (None, None)
    rotary_store(qkv, positions, inv_freq, slots, pools[0], pools[1], num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv)
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = pools[0][page, :, off, :].to(k_pool.dtype)
        v_pool[page, :, off, :] = pools[1][page, :, off, :].to(v_pool.dtype)
    return qkv[:, : num_heads * head_dim].to(torch.bfloat16)


# ---- the product of many tokens and its epilogues


def dense_gemm(x, weight, out=None):
    return skinny_gemm(x, weight, torch.bfloat16, out=out)


def dense_gemm_act(x, weight, kind):
    return skinny_gemm_act(x, weight, kind)


def dense_gemm_swiglu(x, weight_tiled, activation="silu", limit=0.0, up_shift=0.0):
    return skinny_gemm_swiglu(x, weight_tiled, activation, limit, up_shift)


def dense_gemm_rotary(x, wqkv, table, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, rotary_dim, page_size, write_kv):
    qkv = _sums(x, wqkv)
    n = qkv.shape[0]
    heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)
    if rotary_dim:
        half = rotary_dim // 2
        cos, sin = table[:, None, :half], table[:, None, half:]
        qk = heads[:, : num_heads + num_kv_heads, :rotary_dim]
        lo, hi = qk[..., :half].clone(), qk[..., half:].clone()
        heads[:, : num_heads + num_kv_heads, :half] = lo * cos - hi * sin
        heads[:, : num_heads + num_kv_heads, half:rotary_dim] = hi * cos + lo * sin
    if write_kv:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = heads[:, num_heads : num_heads + num_kv_heads].to(k_pool.dtype)
        v_pool[page, :, off, :] = heads[:, num_heads + num_kv_heads :].to(v_pool.dtype)
    return qkv[:, : num_heads * head_dim].to(torch.bfloat16)


def sample(out, logits, temperature=None, top_k=None, top_p=None, seed=None, draw=None):
    rows = logits.shape[0]
    for r in range(rows):
        row = logits[r].numpy()
        if temperature is None:
            out[r] = int(np.argmax(row))
        else:
            out[r] = plain.sample_token(row, float(temperature[r]), int(top_k[r]), float(top_p[r]), int(seed[r]), int(draw[r]))


def linear(x, weight, out=None):
    return torch.matmul(x, weight.t(), out=out)


def logits_product(x, weight):
    return x.float() @ weight.float().t()


class CpuPending:
    def __init__(self, ids: torch.Tensor) -> None:
        self.device_ids = ids
        self.reads = 0

    def result(self) -> list[int]:
        self.reads += 1
        return self.device_ids.tolist()


class CpuSampler:
    """The engine's Sampler without pinned memory and events: same calls, same keys (seed, draw)."""

    def _run(self, logits, params, seeds, draws) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32)
        if all(p.greedy for p in params):
            sample(out, logits)
        else:
            sample(out, logits, [0.0 if p.greedy else p.temperature for p in params], [p.top_k for p in params],
                   [p.top_p for p in params], list(seeds), list(draws))
        return out

    def sample(self, logits, params, seeds, draws) -> list[int]:
        return self._run(logits, params, seeds, draws).tolist() if logits.shape[0] else []

    def sample_async(self, logits, params, seeds, draws) -> CpuPending:
        return CpuPending(self._run(logits, params, seeds, draws))



def pair_embedding(h, table, scale, pair_table, buckets, mul_prev, mul_cur, ids, positions, seq_of_token, q_start, state_slot, prev_state, y=None):
    idl = ids.long()
    x = table[idl].float() * scale
    if pair_table is not None:
        first = q_start.long()[seq_of_token.long()]
        at = torch.arange(ids.numel())
        prev_state = prev_state.view(-1)
        prev = torch.where(at > first, idl[(at - 1).clamp(min=0)], prev_state[state_slot.long()[seq_of_token.long()]].long())
        rows = (prev * mul_prev + idl * mul_cur) % buckets
        rows = torch.where(positions == 0, torch.full_like(rows, buckets), rows)
        x = x + pair_table[rows].float()
        for s in range(state_slot.numel()):
            if q_start[s + 1] > q_start[s]:
                prev_state[state_slot[s].long()] = ids[q_start[s + 1].long() - 1]
    h.copy_(x)
    if y is not None:
        y.copy_(x.to(y.dtype))


def _group_unit(x, groups, eps):
    n, H = x.shape
    parts = x.view(n, groups, H // groups)
    return (parts * torch.rsqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(n, H)


def group_norm_add(h, a, weight, groups, eps, mult, y=None):
    h += mult * (_group_unit(a.float(), groups, eps) * weight)
    if y is not None:
        y.copy_(h.to(y.dtype))


def group_norm_rows(y, h, weight, groups, eps, rows=None):
    x = h if rows is None else h[rows.long()]
    y.copy_((_group_unit(x, groups, eps) * weight).to(y.dtype))


def gelu_mul_rows(g, table, col0, ids):
    e = table[ids.long(), col0 : col0 + g.shape[1]].float()
    g.copy_((_gelu_tanh(g.float()) * e).to(g.dtype))


def depth_average(out, x0, hist, weights, count, y=None):
    out.copy_(weights[0] * x0 + (hist[: count - 1] * weights[1:count, None, None]).sum(0))
    if y is not None:
        y.copy_(out.to(y.dtype))


def mingru_scan(out, p, bz, bx, state, q_start, state_slot, max_len=0):
    W = out.shape[1]
    pf = p.float()
    z = torch.sigmoid(pf[:, :W] + bz)
    u = pf[:, W : 2 * W] + bx
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = pf[:, 2 * W :]
    for s in range(state_slot.numel()):
        slot = int(state_slot[s])
        S = state[slot].clone()
        for r in range(int(q_start[s]), int(q_start[s + 1])):
            S = (1 - z[r]) * S + z[r] * cand[r]
            out[r] = (S * g[r] * torch.sigmoid(g[r])).to(out.dtype)
        state[slot] = S


def diff_prep(q_out, proj, k_col, v_col, wq, wk, eps, positions, freq, amp, slots, k_pool, v_pool, num_heads, num_kv_heads, dim, vdim, rot, page_size):
    n = proj.shape[0]
    ang = positions.float()[:, None] * freq[None, : rot // 2]
    cos, sin = (ang.cos() * amp)[:, None, :], (ang.sin() * amp)[:, None, :]

    def prepare(x, w):  # x [n, units, dim]
        x = x.float()
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
        a, b = x[..., 0:rot:2].clone(), x[..., 1:rot:2].clone()
        x[..., 0:rot:2] = a * cos - b * sin
        x[..., 1:rot:2] = b * cos + a * sin
        return x

    q_out.copy_(prepare(proj[:, : num_heads * 2 * dim].reshape(n, num_heads * 2, dim), wq).reshape(n, -1).to(q_out.dtype))
    if k_col >= 0:
        k = prepare(proj[:, k_col : k_col + num_kv_heads * 2 * dim].reshape(n, num_kv_heads * 2, dim), wk).reshape(n, num_kv_heads, 2 * dim)
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = k.to(k_pool.dtype)
        v_pool[page, :, off, :] = proj[:, v_col : v_col + num_kv_heads * vdim].reshape(n, num_kv_heads, vdim)


def diff_attention_simt(out, q, k_pool, v_pool, block_tables, seq_of_token, positions, gate, num_heads, scale, window, keep_first, lam, post, eps):
    n = q.shape[0]
    _, nkv, page_size, d2 = k_pool.shape
    dim, vdim = d2 // 2, v_pool.shape[3]
    qf = q.float().view(n, num_heads, 2, dim)
    for t in range(n):
        p = int(positions[t])
        table = block_tables[int(seq_of_token[t])].long()
        keys = torch.arange(p + 1)
        if window:
            keys = keys[(p - keys < window) | (keys < keep_first)]
        page, off = table[keys // page_size], keys % page_size
        for h in range(num_heads):
            g = h // (num_heads // nkv)
            k = k_pool[page, g, off].float().view(-1, 2, dim)
            v = v_pool[page, g, off].float()
            a = [torch.softmax((k[:, m] @ qf[t, h, m]) * scale, 0) @ v for m in range(2)]
            o = a[0] - lam * a[1]
            o = o * torch.rsqrt((o * o).mean() + eps) * post
            if gate is not None:
                o = o * torch.sigmoid(gate[t, h].float())
            out[t, h * vdim : (h + 1) * vdim] = o.to(out.dtype)


def diff_attention_tc(out, q, k_pool, v_pool, block_tables, q_start, kv_len, num_seqs, max_q_len, gate, num_heads, scale, window, keep_first, lam,
                      post, eps, splits=1, scratch=None):
    lens = (q_start[1:] - q_start[:-1]).long()
    seq = torch.repeat_interleave(torch.arange(num_seqs), lens)
    at = torch.arange(q.shape[0])
    positions = (kv_len.long() - lens)[seq] + at - q_start.long()[seq]
    diff_attention_simt(out, q, k_pool, v_pool, block_tables, seq, positions, gate, num_heads, scale, window, keep_first, lam, post, eps)


# ---- a stream whose sublayer outputs carry a learned scale per feature; token shift; recurrences with a decay per channel; routed experts


def add_rmsnorm_scaled(y, h, a, fa, b, fb, scale, weight, eps, rows=None):
    delta = None
    if a is not None:
        delta = fa * a.float()
        if b is not None:
            delta = delta + fb * b.float()
        delta = delta * scale
    if rows is None:
        if delta is not None:
            h += delta
        x = h
    else:
        x = h[rows.long()] + (delta[rows.long()] if delta is not None else 0.0)
    if y is not None:
        y.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(y.dtype))


def concat_stream_rows(out, h, table, ids):
    W = h.shape[1]
    out[:, :W] = h.to(out.dtype)
    out[:, W:] = table[ids.long()]


def token_shift_blend(out, x, mu, state, seq_of_token, q_start, state_slot):
    n = x.shape[0]
    for t in range(n):
        s = int(seq_of_token[t])
        before = x[t - 1] if t > int(q_start[s]) else state[int(state_slot[s]), 0]
        c = x[t].float()
        out[:, t] = (c + (before.float() - c) * mu).to(out.dtype)


def rotary_unit_store(q_out, x, positions, inv_freq, slots, k_pool, v_pool, num_heads, num_kv_heads, head_dim, value_dim, rotary_dim, unit_eps, page_size):
    n = x.shape[0]
    d, dv, D = head_dim, value_dim, max(head_dim, value_dim)
    qk = x[:, : (num_heads + num_kv_heads) * d].float().reshape(n, num_heads + num_kv_heads, d).clone()
    if rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        lo, hi = qk[..., :half].clone(), qk[..., half:rotary_dim].clone()
        qk[..., :half] = lo * cos - hi * sin
        qk[..., half:rotary_dim] = hi * cos + lo * sin
    if unit_eps is not None:
        qk = qk * torch.rsqrt((qk * qk).mean(-1, keepdim=True) + unit_eps)
    rows = torch.zeros((n, num_heads + num_kv_heads, D))
    rows[..., :d] = qk
    q_out.copy_(rows[:, :num_heads].reshape(n, num_heads * D).to(q_out.dtype))
    if slots is not None:
        page, off = (slots // page_size).long(), (slots % page_size).long()
        k_pool[page, :, off, :] = rows[:, num_heads:].to(k_pool.dtype)
        v = torch.zeros((n, num_kv_heads, D))
        v[..., :dv] = x[:, (num_heads + num_kv_heads) * d :].float().reshape(n, num_kv_heads, dv)
        v_pool[page, :, off, :] = v.to(v_pool.dtype)


def _row_offsets(kq, heads, d, dv):
    a, k, g = 0, kq * d, 2 * kq * d
    v = g + heads * d
    return a, k, g, v, v + heads * dv


def shift_decay_prep(rows, rkvg, wz, w0, heads, d):
    a, k, g, v, _ = _row_offsets(heads, heads, d, d)
    I = heads * d
    rows[:, a : a + I] = rkvg[0].float()
    rows[:, k : k + I] = rkvg[1].float()
    rows[:, v : v + I] = rkvg[2].float()
    rows[:, g : g + I] = torch.exp(-torch.exp(wz.float() + w0))


def channel_delta_prep(rows, qkv, u, b_col, a, dt_bias, a_log, heads, kv_heads, d, dv, unit_eps):
    n = qkv.shape[0]
    oa, ok, og, ov, ob = _row_offsets(kv_heads, heads, d, dv)
    qk = kv_heads * d
    q = qkv[:, :qk].float().view(n, kv_heads, d)
    k = qkv[:, qk : 2 * qk].float().view(n, kv_heads, d)
    rows[:, oa : oa + qk] = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d**-0.5).reshape(n, qk)
    rows[:, ok : ok + qk] = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + unit_eps)).reshape(n, qk)
    step = torch.nn.functional.softplus(a.float() + dt_bias, threshold=20.0).view(n, heads, d)
    rows[:, og : og + heads * d] = torch.exp(-torch.exp(a_log)[None, :, None] * step).reshape(n, heads * d)
    rows[:, ov : ov + heads * dv] = qkv[:, 2 * qk :].float()
    rows[:, ob : ob + heads] = torch.sigmoid(u[:, b_col : b_col + heads].float())


def decay_recurrence(o, rows, state, q_start, state_slot, kq_heads, mode, bonus=None, max_len=0, rows_per_lane=0):
    _, heads, dv, d = state.shape  # the state is kept transposed: [slot, head, value column, key row]
    oa, ok, og, ov, ob = _row_offsets(kq_heads, heads, d, dv)
    fan = heads // kq_heads
    for s in range(state_slot.numel()):
        slot = int(state_slot[s])
        for t in range(int(q_start[s]), int(q_start[s + 1])):
            a = rows[t, oa : oa + kq_heads * d].view(kq_heads, d).repeat_interleave(fan, 0)
            k = rows[t, ok : ok + kq_heads * d].view(kq_heads, d).repeat_interleave(fan, 0)
            g = rows[t, og : og + heads * d].view(heads, d)
            v = rows[t, ov : ov + heads * dv].view(heads, dv)
            S = state[slot]
            if mode == "bonus":
                kv = v[:, :, None] * k[:, None, :]  # [heads, dv, d]
                o[t] = torch.einsum("hvd,hd->hv", S + kv * bonus[:, None, :], a).reshape(-1)
                state[slot] = S * g[:, None, :] + kv
            else:
                beta = rows[t, ob : ob + heads]
                S = S * g[:, None, :]
                w = beta[:, None] * (v - torch.einsum("hvd,hd->hv", S, k))
                S = S + w[:, :, None] * k[:, None, :]
                state[slot] = S
                o[t] = torch.einsum("hvd,hd->hv", S, a).reshape(-1)


def moe_route(ids, weights, x, router, correction, group_count, group_keep, scale):
    n, top = ids.shape
    E = router.shape[0]
    s = torch.sigmoid(x.float() @ router.t())
    choice = s + correction
    if group_count > 1:
        per = E // group_count
        marks = choice.view(n, group_count, per).topk(min(2, per), -1).values.sum(-1)
        order = torch.sort(-marks, dim=-1, stable=True).indices[:, :group_keep]
        allowed = torch.zeros((n, group_count), dtype=torch.bool)
        allowed.scatter_(1, order, True)
        choice = torch.where(allowed.repeat_interleave(per, 1), choice, torch.full_like(choice, float("-inf")))
    picked = torch.sort(-choice, dim=-1, stable=True).indices[:, :top]
    w = s.gather(1, picked)
    ids.copy_(picked.to(torch.int32))
    weights.copy_(w / (w.sum(-1, keepdim=True) + 1e-20) * scale)


def _glu_act(g, activation):
    if activation == "gelu_tanh":
        return _gelu_tanh(g)
    if activation == "quick_gelu":
        return g * torch.sigmoid(1.702 * g)
    return _silu(g)


def moe_experts(out, x, ids, weights, w_gate_up, w_down, activation="silu", stages=0):
    n, top = ids.shape
    ff = w_gate_up.shape[1] // 2
    acc = torch.zeros((n, x.shape[1]))
    for k in range(top):
        for e in ids[:, k].unique().tolist():
            rows = (ids[:, k] == e).nonzero().flatten()
            gu = _sums(x[rows], w_gate_up[e]).to(x.dtype).float()
            hidden = (_glu_act(gu[:, :ff], activation) * gu[:, ff:]).to(x.dtype)
            acc[rows] += weights[rows, k, None] * _sums(hidden, w_down[e])
    out.copy_(acc.to(out.dtype))


def linear_bias(x, weight, bias):
    return (_sums(x, weight) + bias.float()).to(x.dtype)


def batched_project(x, weight):
    return torch.bmm(x.float(), weight.float()).to(x.dtype)


OPS = {"embedding": embedding, "patch_tokens": patch_tokens, "copy_page": copy_page, "add_rmsnorm": add_rmsnorm,
       "rotary_table": rotary_table, "rotary_store": rotary_store, "silu_mul": silu_mul, "paged_attention_simt": paged_attention_simt,
       "paged_attention_mma": paged_attention_mma, "paged_decode_tma": paged_decode_tma, "paged_prefill_tc": paged_prefill_tc,
       "skinny_gemm_slices": skinny_gemm_slices, "skinny_gemm": skinny_gemm, "skinny_gemm_residual": skinny_gemm_residual,
       "skinny_gemm_swiglu": skinny_gemm_swiglu, "skinny_gemm_act": skinny_gemm_act, "skinny_gemm_rotary": skinny_gemm_rotary, "dense_gemm": dense_gemm,
       "dense_gemm_swiglu": dense_gemm_swiglu, "dense_gemm_act": dense_gemm_act, "dense_gemm_rotary": dense_gemm_rotary,
       "sample": sample, "post_add_layernorm": post_add_layernorm, "stream_reinject": stream_reinject, "activation": activation,
       "qk_norm_rotary_store": qk_norm_rotary_store, "sigmoid_gate": sigmoid_gate, "causal_conv_silu": causal_conv_silu,
       "conv_state_update": conv_state_update, "ssm_scan": ssm_scan, "gated_group_rmsnorm": gated_group_rmsnorm,
       "add_rmsnorm_pair": add_rmsnorm_pair, "scale_softcap": scale_softcap, "latent_prep": latent_prep, "delta_rule_scan": delta_rule_scan,
       "heads_matvec": heads_matvec, "heads_matvec_supported": lambda in_features, features: True,
       "pair_embedding": pair_embedding, "group_norm_add": group_norm_add, "group_norm_rows": group_norm_rows, "gelu_mul_rows": gelu_mul_rows,
       "depth_average": depth_average, "mingru_scan": mingru_scan, "diff_prep": diff_prep, "diff_attention_simt": diff_attention_simt,
       "diff_attention_tc": diff_attention_tc, "add_rmsnorm_scaled": add_rmsnorm_scaled, "concat_stream_rows": concat_stream_rows,
       "token_shift_blend": token_shift_blend, "rotary_unit_store": rotary_unit_store, "shift_decay_prep": shift_decay_prep,
       "moe_grouped_supported": lambda tokens, W, ff, dtype: False, "channel_delta_prep": channel_delta_prep, "decay_recurrence": decay_recurrence, "moe_route": moe_route, "moe_experts": moe_experts}


calls: dict[str, int] = {}  # how often each stand-in ran since patched() was entered


def _counted(name, fn):
    def run(*args, **kwargs):
        calls[name] = calls.get(name, 0) + 1
        return fn(*args, **kwargs)

    return run


@contextlib.contextmanager
def patched():
    """Inside: models on ``device='cpu'`` build, load and step through the stand-ins (float32, and bfloat16
    with the decode products' fused epilogues)."""
    saved = {name: getattr(ops, name) for name in OPS}
    saved_linear, saved_model_linear, saved_require = gemm.linear, model_mod.linear, runner_mod._require_cuda
    saved_logits, saved_need = gemm.logits_product, gemm._need_device
    saved_bias, saved_batched = gemm.linear_bias, gemm.batched_project
    saved_lookup, saved_mixed = graphs_mod.DecodeGraphs.lookup, graphs_mod.DecodeGraphs.lookup_mixed
    try:
        graphs_mod.DecodeGraphs.lookup = graphs_mod.DecodeGraphs.lookup_mixed = lambda self, *a, **k: None  # no captured steps without a device
        calls.clear()
        for name, fn in OPS.items():
            setattr(ops, name, _counted(name, fn))
        gemm.linear = model_mod.linear = linear
        gemm.logits_product, gemm._need_device = logits_product, lambda x, what: None
        gemm.linear_bias, gemm.batched_project = linear_bias, batched_project
        runner_mod._require_cuda = lambda device: None
        yield
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)
        gemm.linear, model_mod.linear, runner_mod._require_cuda = saved_linear, saved_model_linear, saved_require
        gemm.logits_product, gemm._need_device = saved_logits, saved_need
        gemm.linear_bias, gemm.batched_project = saved_bias, saved_batched
        graphs_mod.DecodeGraphs.lookup, graphs_mod.DecodeGraphs.lookup_mixed = saved_lookup, saved_mixed

