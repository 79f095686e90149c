"""The kernels that came with the scaled pre-norm layer, the attention behind short convolutions, the recurrences with a decay per
channel and the routed feed-forward, against plain PyTorch float32 restatements of the same operations (tests/cpu_ops.py), in
float32 and bfloat16, at sizes that take the 16-byte paths and sizes that do not."""

import pytest
import torch

from dli_b200.kernels import ops
from tests import cpu_ops as ref

pytestmark = pytest.mark.gpu

DTYPES = [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)]


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def _close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float()
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"{what}: max error {err}"


def _i32(values):
    return torch.tensor(values, dtype=torch.int32)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("H", [40, 77, 256, 1000, 4096])
def test_add_rmsnorm_scaled(dtype, tol, H):
    n = 7
    h = _rand(n, H, seed=1) * 3 + 0.5
    a, b = (_rand(n, H, seed=2) * 2 + 1).to(dtype), (_rand(n, H, seed=5) - 0.5).to(dtype)
    ls, w = 1 + 0.5 * _rand(H, seed=3), 1 + 0.1 * _rand(H, seed=4)
    for da, db in ((a, b), (a, None), (None, None)):
        for rows in (None, _i32([5, 0, 3])):
            for with_y in (True, False):
                if not with_y and rows is not None:
                    continue
                h_ref, h_dev = h.clone(), h.cuda()
                k = n if rows is None else rows.numel()
                y_ref, y_dev = torch.empty(k, H, dtype=dtype), torch.empty(k, H, dtype=dtype, device="cuda")
                ref.add_rmsnorm_scaled(y_ref if with_y else None, h_ref, da, 0.8, db, -0.6, ls, w, 1e-5, rows)
                ops.add_rmsnorm_scaled(y_dev if with_y else None, h_dev, None if da is None else da.cuda(), 0.8, None if db is None else db.cuda(), -0.6,
                                       ls.cuda(), w.cuda(), 1e-5, None if rows is None else rows.cuda())
                if with_y:
                    _close(y_dev, y_ref, tol, "y")
                _close(h_dev, h_ref, 1e-5, "h")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("W", [52, 64, 1032])
def test_concat_rows_and_token_shift(dtype, tol, W):
    n, V = 9, 30
    h, table, ids = _rand(n, W, seed=1), _rand(V, W, seed=2).to(dtype), _i32([3, 29, 0, 7, 7, 1, 12, 5, 28])
    want, got = torch.empty(n, 2 * W, dtype=dtype), torch.empty(n, 2 * W, dtype=dtype, device="cuda")
    ref.concat_stream_rows(want, h, table, ids)
    ops.concat_stream_rows(got, h.cuda(), table.cuda(), ids.cuda())
    _close(got, want, 0.0, "concat")
    # three sequences of 1, 5 and 3 tokens in slots 2, 0, 3
    x, mu, state = _rand(n, W, seed=3).to(dtype), torch.rand(5, W, generator=torch.Generator().manual_seed(4)), _rand(5, 1, W, seed=5).to(dtype)
    seq_of, q_start, slots = _i32([0, 1, 1, 1, 1, 1, 2, 2, 2]), _i32([0, 1, 6, 9]), _i32([2, 0, 3])
    want, got = torch.empty(5, n, W, dtype=dtype), torch.empty(5, n, W, dtype=dtype, device="cuda")
    ref.token_shift_blend(want, x, mu, state, seq_of, q_start, slots)
    ops.token_shift_blend(got, x.cuda(), mu.cuda(), state.cuda(), seq_of.cuda(), q_start.cuda(), slots.cuda())
    _close(got, want, tol, "blend")
    st_ref, st_dev = state.clone(), state.cuda()
    ref.conv_state_update(st_ref, x, 0, q_start, slots)
    ops.conv_state_update(st_dev, x.cuda(), 0, q_start.cuda(), slots.cuda())
    _close(st_dev, st_ref, 0.0, "carried row")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 8, 8), (3, 3, 10, 7, 6), (8, 2, 64, 16, 32), (2, 1, 24, 40, 0), (2, 2, 128, 128, 32)])
def test_rotary_unit_store(dtype, tol, sizes):
    nh, nkv, d, dv, rot = sizes
    n, page, pages = 11, 4, 6
    D = max(d, dv)
    x = _rand(n, (nh + nkv) * d + nkv * dv, seed=1).to(dtype)
    pos = _i32([0, 1, 2, 300, 301, 5, 6, 7, 8, 9, 1000])
    slots = _i32([20, 1, 7, 3, 12, 13, 14, 15, 0, 9, 23])
    inv = (1.0 / 100.0 ** (torch.arange(0, rot, 2).float() / max(rot, 1))) if rot else None
    for eps in (1e-5, None):
        q_ref, q_dev = torch.zeros(n, nh * D, dtype=dtype), torch.zeros(n, nh * D, dtype=dtype, device="cuda")
        pools_ref = [torch.full((pages, nkv, page, D), 9.0, dtype=dtype) for _ in range(2)]
        pools_dev = [p.cuda() for p in pools_ref]
        ref.rotary_unit_store(q_ref, x, pos, inv, slots, pools_ref[0], pools_ref[1], nh, nkv, d, dv, rot, eps, page)
        ops.rotary_unit_store(q_dev, x.cuda(), pos.cuda(), None if inv is None else inv.cuda(), slots.cuda(), pools_dev[0], pools_dev[1], nh, nkv, d, dv, rot, eps, page)
        _close(q_dev, q_ref, tol, "q")
        _close(pools_dev[0], pools_ref[0], tol, "k")
        _close(pools_dev[1], pools_ref[1], tol, "v")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_convolution_without_activation_and_sigmoid_gate(dtype, tol):
    n, C, taps = 9, 24, 3
    u, w, state = _rand(n, C + 5, seed=1).to(dtype), _rand(taps, C, seed=2), _rand(4, taps - 1, C, seed=3).to(dtype)
    seq_of, q_start, slots = _i32([0, 1, 1, 1, 1, 1, 2, 2, 2]), _i32([0, 1, 6, 9]), _i32([2, 0, 3])
    for act in (True, False):
        want, got = torch.empty(n, C, dtype=dtype), torch.empty(n, C, dtype=dtype, device="cuda")
        ref.causal_conv_silu(want, u, 5, w, None, state, seq_of, q_start, slots, activation=act)
        ops.causal_conv_silu(got, u.cuda(), 5, w.cuda(), None, state.cuda(), seq_of.cuda(), q_start.cuda(), slots.cuda(), activation=act)
        _close(got, want, tol, f"conv act={act}")
    for inner, parts in ((48, 3), (256, 2), (35, 5)):
        y, z, wt = _rand(n, inner, seed=4) * 3, _rand(n, inner, seed=5).to(dtype), 1 + 0.2 * _rand(inner, seed=6)
        for gate in ("silu", "sigmoid"):
            want, got = torch.empty(n, inner, dtype=dtype), torch.empty(n, inner, dtype=dtype, device="cuda")
            ref.gated_group_rmsnorm(want, y, z, 0, wt, parts, 1e-5, gate_after=True, gate=gate)
            ops.gated_group_rmsnorm(got, y.cuda(), z.cuda(), 0, wt.cuda(), parts, 1e-5, gate_after=True, gate=gate)
            _close(got, want, tol, f"norm gate={gate} {inner}")


@pytest.mark.parametrize("lane_rows", [0, 8, 16, 32])
@pytest.mark.parametrize("mode", ["bonus", "delta"])
@pytest.mark.parametrize("sizes", [(4, 2, 12, 10), (2, 2, 32, 32), (3, 1, 9, 7), (2, 1, 64, 48), (2, 2, 128, 128), (1, 1, 136, 40), (2, 1, 72, 72)])
def test_decay_recurrence(mode, sizes, lane_rows):
    """Portions of 1, 19 and 3 tokens from states that are not zero, in scattered slots; the state afterwards; then the same tokens
    one at a time; with 8, 16 and 32 key rows a lane, and with what the launcher chooses."""
    heads, kq, d, dv = sizes
    if mode == "bonus":
        kq, dv = heads, d
    n = 23
    stride = ops.decay_recurrence_row(kq, heads, d, dv)
    g = torch.Generator().manual_seed(7)
    rows = torch.randn(n, stride, generator=g) * 0.3
    rows[:, 2 * kq * d : 2 * kq * d + heads * d] = 0.9 + 0.1 * torch.rand(n, heads * d, generator=g)  # decays
    rows[:, -4:] = torch.rand(n, 4, generator=g)
    if mode == "delta":
        b0 = 2 * kq * d + heads * d + heads * dv
        rows[:, b0 : b0 + heads] = torch.rand(n, heads, generator=g)
    state = torch.randn(5, heads, dv, d, generator=g) * 0.5
    bonus = torch.randn(heads, d, generator=g) if mode == "bonus" else None
    q_start, slots = _i32([0, 1, 20, 23]), _i32([3, 0, 4])
    o_ref, o_dev = torch.zeros(n, heads * dv), torch.zeros(n, heads * dv, device="cuda")
    s_ref, s_dev = state.clone(), state.cuda()
    ref.decay_recurrence(o_ref, rows, s_ref, q_start, slots, kq, mode, bonus)
    ops.decay_recurrence(o_dev, rows.cuda(), s_dev, q_start.cuda(), slots.cuda(), kq, mode, None if bonus is None else bonus.cuda(), rows_per_lane=lane_rows)
    _close(o_dev, o_ref, 1e-4, "o")
    _close(s_dev, s_ref, 1e-4, "state")
    s_one, o_one = state.cuda(), torch.zeros(n, heads * dv, device="cuda")
    for s in range(3):
        for t in range(int(q_start[s]), int(q_start[s + 1])):
            ops.decay_recurrence(o_one[t : t + 1], rows[t : t + 1].cuda(), s_one, _i32([0, 1]).cuda(), slots[s : s + 1].cuda(), kq, mode,
                                 None if bonus is None else bonus.cuda(), rows_per_lane=lane_rows)
    # (equal up to float32 rounding: how many threads share a column, hence the order of a sum, follows the launch's shape)
    _close(o_one, o_dev.cpu(), 1e-5, "token by token against the portion: o")
    _close(s_one, s_dev.cpu(), 1e-5, "token by token against the portion: state")


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_recurrence_rows(dtype, tol):
    n, heads, kq, d, dv = 6, 4, 2, 12, 10
    rkvg, wz, w0 = _rand(4, n, heads * d, seed=1).to(dtype), _rand(n, heads * d, seed=2).to(dtype), _rand(heads * d, seed=3) - 2
    want = torch.zeros(n, ops.decay_recurrence_row(heads, heads, d, d))
    got = torch.zeros_like(want, device="cuda")
    ref.shift_decay_prep(want, rkvg, wz, w0, heads, d)
    ops.shift_decay_prep(got, rkvg.cuda(), wz.cuda(), w0.cuda(), heads, d)
    _close(got, want, 1e-5, "token shift rows")
    qkv, u = _rand(n, 2 * kq * d + heads * dv, seed=4).to(dtype), _rand(n, 2 * kq * d + heads * dv + heads + 3, seed=5).to(dtype)
    a, dt_bias, a_log = _rand(n, heads * d, seed=6).to(dtype), _rand(heads * d, seed=7), _rand(heads, seed=8) - 3
    want = torch.zeros(n, ops.decay_recurrence_row(kq, heads, d, dv))
    got = torch.zeros_like(want, device="cuda")
    b_col = 2 * kq * d + heads * dv
    ref.channel_delta_prep(want, qkv, u, b_col, a, dt_bias, a_log, heads, kq, d, dv, 1e-6)
    ops.channel_delta_prep(got, qkv.cuda(), u.cuda(), b_col, a.cuda(), dt_bias.cuda(), a_log.cuda(), heads, kq, d, dv, 1e-6)
    _close(got, want, 1e-5, "delta rows")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("sizes", [(48, 6, 2, 3, 2, 20), (64, 8, 4, 2, 1, 96), (50, 10, 3, 5, 2, 11), (128, 40, 6, 8, 3, 64), (32, 4, 4, 1, 1, 8), (256, 16, 2, 1, 1, 128)])
def test_routed_feed_forward(dtype, tol, sizes):
    """Routing (exact: the same experts, weights to float32 rounding) and the experts' products, for a few tokens and for many."""
    W, E, top, groups, keep, ff = sizes
    router, corr = _rand(E, W, seed=1, scale=2.0 / W**0.5), _rand(E, seed=2, scale=0.3)
    wgu, wd = _rand(E, 2 * ff, W, seed=3, scale=1 / W**0.5).to(dtype), _rand(E, W, ff, seed=4, scale=1 / ff**0.5).to(dtype)
    for n in (1, 5, 70, 300):
        x = _rand(n, W, seed=10 + n).to(dtype)
        ids_ref, w_ref = torch.zeros(n, top, dtype=torch.int32), torch.zeros(n, top)
        ids_dev, w_dev = ids_ref.cuda(), w_ref.cuda()
        ref.moe_route(ids_ref, w_ref, x, router, corr, groups, keep, 1.5)
        ops.moe_route(ids_dev, w_dev, x.cuda(), router.cuda(), corr.cuda(), groups, keep, 1.5)
        same = (ids_dev.cpu() == ids_ref).all(1)
        assert same.float().mean() > 0.97, "routing differs on more than near ties"
        _close(w_dev.cpu()[same], w_ref[same], 1e-5, "weights")
        out_ref, out_dev = torch.zeros(n, W, dtype=dtype), torch.zeros(n, W, dtype=dtype, device="cuda")
        ref.moe_experts(out_ref, x, ids_dev.cpu(), w_dev.cpu(), wgu, wd, "silu")
        for stages in (0, 2, 3):
            ops.moe_experts(out_dev, x.cuda(), ids_dev, w_dev, wgu.cuda(), wd.cuda(), "silu", stages=stages)
            _close(out_dev, out_ref, tol, f"experts, {n} tokens, copies {stages} deep")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [32, 64, 96, 128])
def test_a_sink_per_head_in_every_attention_kernel(dtype, d):
    """Sinks that differ from head to head, over portions and single tokens, with and without split keys."""
    from dli_b200.kernels import attention as attn

    nh, nkv, page, pages = 4, 2, 16, 40
    if dtype == torch.float32 and d != 32:
        pytest.skip("one size is enough for the float32 kernel")
    g = torch.Generator().manual_seed(d)
    k_pool, v_pool = (torch.randn(pages, nkv, page, d, generator=g) * 0.5).to(dtype), torch.randn(pages, nkv, page, d, generator=g).to(dtype)
    sinks = torch.tensor([3.0, -20.0, 0.5, 1.5])
    lens = [1, 1, 70, 200]  # two single tokens at contexts of 150 and 37, two portions
    kv = [150, 37, 70, 230]
    tables = torch.full((4, 16), -1, dtype=torch.int32)
    perm = torch.randperm(pages, generator=g)
    at = 0
    for s, L in enumerate(kv):
        need = -(-L // page)
        tables[s, :need] = perm[at : at + need].to(torch.int32)
        at += need
    n = sum(lens)
    q = (torch.randn(n, nh * d, generator=g)).to(dtype)
    q_start = _i32([0, 1, 2, 72, 272])
    seq_of = torch.cat([torch.full((L,), s, dtype=torch.int32) for s, L in enumerate(lens)])
    pos = torch.cat([torch.arange(K - L, K, dtype=torch.int32) for K, L in zip(kv, lens)])
    want = torch.zeros(n, nh * d, dtype=dtype)
    ref.paged_attention_simt(want, q, k_pool, v_pool, tables, seq_of, pos, nh, 0.3, 64, sinks)

    class Group:
        block_tables, slots = tables.cuda(), None

    class Batch:
        num_single, num_seqs, max_q_len, max_kv_len_single, max_kv_len = 2, 4, 200, 150, 230
        launch_keys = {}

        def group(self, i):
            return Group

    Batch.q_start, Batch.kv_len, Batch.seq_of_token, Batch.positions = q_start.cuda(), _i32(kv).cuda(), seq_of.cuda(), pos.cuda()

    class Cache:
        k, v, page_size, group = k_pool.cuda(), v_pool.cuda(), page, 0

    for splits in (None, 2):
        got = torch.zeros(n, nh * d, dtype=dtype, device="cuda")
        attn.paged_attention(got, q.cuda(), Cache, Batch(), nh, 0.3, 64, splits=splits, sink=sinks.cuda())
        _close(got, want, 2e-5 if dtype == torch.float32 else 3e-2, f"splits={splits}")
