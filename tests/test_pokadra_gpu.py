"""The Pokadra model on the real kernels, in float32 and bfloat16, against the plain implementation: the cases of
tests/pokadra_suite.py, the new kernels one by one against float32 restatements, trace replay as a child process, and steps
replayed from CUDA graphs."""

import numpy as np
import pytest
import torch

from tests import cpu_ops, pokadra_suite as suite
from tests.plain import pokadra_plain as plain
from tests.util import TraceRun

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, dtype, tmp_path):
    case(tmp_path, "cuda:0", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_with_four_state_slots(dtype, tmp_path):
    """bin/trace_run on a schedule of six requests, four live at most, in a pool that holds three of them."""
    cfg = suite.CONFIGS["mixed"]
    w = suite.make_model(tmp_path / "m", cfg, seed=41)
    seqs = {f"r{i}": suite.tokens_for(cfg, n, seed=80 + i) for i, n in enumerate((40, 33, 21, 38, 27, 30))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    run = TraceRun(tmp_path / "m", dtype, tmp_path / "out", max_tokens=4 * 64, page_size=8)
    at = {r: 0 for r in seqs}
    order = list(seqs)
    live, step = [], 0
    try:
        while order or live:
            while order and len(live) < 4:
                live.append(order.pop(0))
            entries, end = [], []
            for j, r in enumerate(live):
                n = min(len(seqs[r]) - at[r], (13, 1, 2, 5)[(step + j) % 4])
                entries.append((r, seqs[r][at[r] : at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == len(seqs[r]):
                    end.append(r)
            got = run.step(entries, end)
            row = 0
            for r, toks, _ in entries:
                n = len(toks)
                lo = at[r] - n
                suite.close(got[row : row + n].astype(np.float64), want[r][lo : lo + n], dtype, f"{r} at {lo}")
                row += n
            live = [r for r in live if r not in end]
            step += 1
    finally:
        run.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_from_graphs_equal_steps_launched_one_by_one(dtype, tmp_path):
    """Decode steps (and, once their shape has come often enough, small mixed steps) replay CUDA graphs; padding rows
    must not touch a live request's state, pages or previous token."""
    cfg = suite.CONFIGS["mixed"]
    suite.make_model(tmp_path / "m", cfg, seed=51)
    seqs = [suite.tokens_for(cfg, 60, seed=90 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        s = suite.Session(tmp_path / "m", "cuda:0", dtype, pages=40, page_size=8, cuda_graphs=graphs)
        got = [s.step(*[(i, t[:17 + i], [16 + i]) for i, t in enumerate(seqs)])]
        for k in range(40):
            got.append(s.step(*[(i, [t[17 + i + k]], [0]) for i, t in enumerate(seqs)]))
        assert (s.runner.graph_steps > 0) == graphs
        outs.append(np.concatenate(got))
    assert np.abs(outs[0] - outs[1]).max() <= (1e-5 if dtype == "float32" else 2e-2)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,H,groups", [(5, 48, 3), (33, 2048, 2), (3, 45, 5), (1, 256, 1)])
def test_group_norm_kernels(dtype, n, H, groups):
    from dli_b200.kernels import ops

    a, w = _rand((n, H), dtype, 1), _rand((H,), torch.float32, 2) + 1
    h = _rand((n, H), torch.float32, 3)
    h_ref, y_ref = h.cpu().clone(), torch.empty((n, H), dtype=dtype)
    cpu_ops.group_norm_add(h_ref, a.cpu(), w.cpu(), groups, 1e-5, 0.7, y_ref)
    y = torch.empty_like(a)
    ops.group_norm_add(h, a, w, groups, 1e-5, 0.7, y)
    assert torch.allclose(h.cpu(), h_ref, atol=2e-5, rtol=1e-5)
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=2e-5 if dtype == torch.float32 else 4e-2)
    rows = torch.tensor([n - 1, 0], dtype=torch.int32).cuda()
    out, out_ref = torch.empty((2, H), dtype=dtype, device="cuda"), torch.empty((2, H), dtype=dtype)
    ops.group_norm_rows(out, h, w, groups, 1e-5, rows)
    cpu_ops.group_norm_rows(out_ref, h.cpu(), w.cpu(), groups, 1e-5, rows.cpu())
    assert torch.allclose(out.float().cpu(), out_ref.float(), atol=2e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_side_input_and_depth_average_kernels(dtype):
    from dli_b200.kernels import ops

    H, vocab, buckets = 40, 29, 13
    table, pairs = _rand((vocab, H), dtype, 1), _rand((buckets + 1, H), dtype, 2)
    ids = torch.tensor([3, 7, 7, 1, 28, 0, 5], dtype=torch.int32)
    positions = torch.tensor([4, 0, 1, 2, 9, 10, 11], dtype=torch.int32)
    seq = torch.tensor([0, 1, 1, 1, 2, 2, 2], dtype=torch.int32)
    q_start = torch.tensor([0, 1, 4, 7], dtype=torch.int32)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    state = torch.tensor([[11], [12], [13], [14], [15]], dtype=torch.int32)
    h_ref, y_ref, state_ref = torch.empty((7, H)), torch.empty((7, H), dtype=dtype), state.clone()
    cpu_ops.pair_embedding(h_ref, table.cpu(), 1.5, pairs.cpu(), buckets, 5, 3, ids, positions, seq, q_start, slots, state_ref, y_ref)
    h, y, dev_state = torch.empty((7, H), device="cuda"), torch.empty((7, H), dtype=dtype, device="cuda"), state.cuda()
    ops.pair_embedding(h, table, 1.5, pairs, buckets, 5, 3, ids.cuda(), positions.cuda(), seq.cuda(), q_start.cuda(), slots.cuda(), dev_state, y)
    assert torch.allclose(h.cpu(), h_ref, atol=1e-6) and torch.equal(dev_state.cpu(), state_ref) and state_ref.view(-1).tolist() == [1, 12, 3, 5, 15]
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=1e-6 if dtype == torch.float32 else 4e-2)
    g, side = _rand((7, 6), dtype, 4), _rand((vocab, 18), dtype, 5)
    g_ref = g.cpu().clone()
    cpu_ops.gelu_mul_rows(g_ref, side.cpu(), 6, ids)
    ops.gelu_mul_rows(g, side, 6, ids.cuda())
    assert torch.allclose(g.float().cpu(), g_ref.float(), atol=1e-6 if dtype == torch.float32 else 4e-2)
    hist, x0, wts = _rand((4, 7, H), torch.float32, 6), _rand((7, H), torch.float32, 7), _rand((5,), torch.float32, 8)
    ref, ref_y = torch.empty((7, H)), torch.empty((7, H), dtype=dtype)
    cpu_ops.depth_average(ref, x0.cpu(), hist.cpu(), wts.cpu(), 4, ref_y)
    out_y = torch.empty((7, H), dtype=dtype, device="cuda")
    ops.depth_average(hist[3], x0, hist, wts, 4, out_y)
    assert torch.allclose(hist[3].cpu(), ref, atol=1e-5) and torch.allclose(out_y.float().cpu(), ref_y.float(), atol=1e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,lens", [(40, (1, 1, 1)), (7, (5, 1, 300)), (256, (700, 2)), (130, (64, 65, 257))])
def test_mingru_kernel(dtype, W, lens):
    """Single tokens, short portions (the plain walk) and long ones (chunks walked side by side), each from its own slot."""
    from dli_b200.kernels import ops

    n = sum(lens)
    p, bz, bx = _rand((n, 3 * W), dtype, 1, 1.5), _rand((W,), torch.float32, 2) - 1.0, _rand((W,), torch.float32, 3)
    q_start = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    slots = torch.tensor(list(range(len(lens), 0, -1)), dtype=torch.int32)
    state = _rand((len(lens) + 1, W), torch.float32, 4)
    out_ref, state_ref = torch.empty((n, W), dtype=dtype), state.cpu().clone()
    cpu_ops.mingru_scan(out_ref, p.cpu(), bz.cpu(), bx.cpu(), state_ref, q_start, slots)
    out = torch.empty((n, W), dtype=dtype, device="cuda")
    ops.mingru_scan(out, p, bz, bx, state, q_start.cuda(), slots.cuda(), max_len=max(lens))
    assert torch.allclose(state.cpu(), state_ref, atol=2e-5, rtol=1e-5)
    assert torch.allclose(out.float().cpu(), out_ref.float(), atol=2e-5 if dtype == torch.float32 else 4e-2, rtol=1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dim,vdim,rot,page,window,keep", [(4, 2, 16, 24, 8, 8, 13, 3), (3, 1, 6, 5, 2, 4, 3, 1), (8, 2, 64, 128, 64, 16, 0, 0),
                                                                 (6, 2, 48, 80, 16, 16, 40, 6), (2, 2, 32, 16, 0, 8, 9, 20)])
def test_diff_attention_kernels(dtype, nh, nkv, dim, vdim, rot, page, window, keep):
    """Preparation (norm, rotation, cache write) and attention (both maps, difference, norm, gate) against the float32
    restatement, over a prompt portion, a later portion of the same sequence and single tokens of another, with pages in
    scrambled order and unused pages poisoned."""
    from dli_b200.kernels import attention as attn
    from dli_b200.kernels import ops

    lens, starts = (37, 1, 9), (0, 50, 37)  # sequence 0 twice: a first portion, later nine more tokens; sequence 1 decodes at position 50
    per_seq = -(-52 // page)
    pages = 2 * per_seq
    order = np.random.default_rng(0).permutation(pages)
    k_pool = torch.full((pages, nkv, page, 2 * dim), float("nan"), dtype=dtype, device="cuda")
    v_pool = torch.full((pages, nkv, page, vdim), float("nan"), dtype=dtype, device="cuda")
    tables = torch.tensor(np.stack([order[:per_seq], order[per_seq:]]), dtype=torch.int32)
    cols = nh * 2 * dim + nkv * (2 * dim + vdim) + nh
    wq, wk = _rand((dim,), torch.float32, 1) + 1.5, _rand((dim,), torch.float32, 2) + 1.5
    freq = torch.tensor([10000.0 ** (-2 * i / max(rot, 2)) for i in range(max(rot // 2, 1))], dtype=torch.float32).cuda()
    pools_ref = [k_pool.cpu().clone(), v_pool.cpu().clone()]

    def run(seq_ids, firsts, counts, seed):
        n = sum(counts)
        proj = _rand((n, cols), dtype, seed)
        seq = torch.tensor(np.repeat(np.arange(len(counts)), counts), dtype=torch.int32)
        pos = torch.tensor(np.concatenate([np.arange(f, f + c) for f, c in zip(firsts, counts)]), dtype=torch.int32)
        tab = tables[list(seq_ids)]
        slots = torch.tensor([int(tab[s, p // page]) * page + p % page for s, p in zip(seq.tolist(), pos.tolist())], dtype=torch.int32)
        q, q_ref = torch.empty((n, nh * 2 * dim), dtype=dtype, device="cuda"), torch.empty((n, nh * 2 * dim), dtype=dtype)
        args = (nh * 2 * dim, nh * 2 * dim + nkv * 2 * dim)
        ops.diff_prep(q, proj, *args, wq, wk, 1e-5, pos.cuda(), freq, 1.07, slots.cuda(), k_pool, v_pool, nh, nkv, dim, vdim, rot, page)
        cpu_ops.diff_prep(q_ref, proj.cpu(), *args, wq.cpu(), wk.cpu(), 1e-5, pos, freq.cpu(), 1.07, slots, pools_ref[0], pools_ref[1], nh, nkv, dim, vdim, rot, page)
        tol = 2e-5 if dtype == torch.float32 else 6e-2
        assert torch.allclose(q.float().cpu(), q_ref.float(), atol=tol, rtol=1e-2)
        gate = proj[:, cols - nh :]
        out, out_ref = torch.empty((n, nh * vdim), dtype=dtype, device="cuda"), torch.empty((n, nh * vdim), dtype=dtype)
        ops.diff_attention_simt(out, q, k_pool, v_pool, tab.cuda(), seq.cuda(), pos.cuda(), gate, nh, 0.4, window or None, keep, 0.37, 0.6, 1e-5)
        cpu_ops.diff_attention_simt(out_ref, q_ref, pools_ref[0], pools_ref[1], tab, seq, pos, gate.cpu(), nh, 0.4, window or None, keep, 0.37, 0.6, 1e-5)
        assert not torch.isnan(out).any()
        assert torch.allclose(out.float().cpu(), out_ref.float(), atol=1e-4 if dtype == torch.float32 else 6e-2, rtol=1e-2)
        return q, tab, seq, pos, gate, out_ref

    run((0, 1), (0, 0), (37, 50), 10)
    q, tab, seq, pos, gate, out_ref = run((0, 1), (37, 50), (9, 1), 11)
    keys = torch.isnan(k_pool.float()).any(-1).sum().item()
    assert keys == (pages * page - 46 - 51) * nkv  # nothing was written beside the tokens' own slots
    # the kernels the engine chooses for this dtype and these sizes give the same
    from types import SimpleNamespace

    cache = SimpleNamespace(k=k_pool, v=v_pool, group=0, page_size=page)
    batch = SimpleNamespace(group=lambda g: SimpleNamespace(block_tables=tab.cuda()), seq_of_token=seq.cuda(), positions=pos.cuda(), num_single=0,
                            num_seqs=2, q_start=torch.tensor([0, 9, 10], dtype=torch.int32).cuda(), kv_len=torch.tensor([46, 51], dtype=torch.int32).cuda(),
                            max_q_len=9, max_kv_len=51, max_kv_len_single=0, launch_keys={})
    out = torch.empty((10, nh * vdim), dtype=dtype, device="cuda")
    attn.diff_attention(out, q, cache, batch, gate, nh, 0.4, window or None, keep, 0.37, 0.6, 1e-5)
    assert torch.allclose(out.float().cpu(), out_ref.float(), atol=1e-4 if dtype == torch.float32 else 6e-2, rtol=1e-2)


@pytest.mark.parametrize("nh,nkv,dim,vdim,window,keep", [(8, 2, 64, 128, 100, 4), (2, 2, 32, 64, 0, 0), (3, 1, 48, 80, 70, 130), (12, 1, 16, 32, 65, 1)])
def test_diff_attention_on_tensor_cores_over_many_key_tiles(nh, nkv, dim, vdim, window, keep):
    """The tensor-core kernel against the CUDA-core kernel (bfloat16 both) where a row walks several tiles of keys: a long
    portion, a short one behind a long context, single tokens at contexts on both sides of a tile's edge; row counts that
    divide a map's warps by rows, by keys and both ways."""
    from dli_b200.kernels import ops

    page, dtype = 16, torch.bfloat16
    q_lens, kv_lens = (150, 7, 1, 1, 1, 20), (150, 300, 257, 64, 65, 21)
    S, n = len(q_lens), sum(q_lens)
    per_seq = -(-max(kv_lens) // page)
    order = torch.tensor(np.random.default_rng(1).permutation(S * per_seq), dtype=torch.int32).view(S, per_seq).cuda()
    k_pool = _rand((S * per_seq, nkv, page, 2 * dim), dtype, 21)
    v_pool = _rand((S * per_seq, nkv, page, vdim), dtype, 22)
    q = _rand((n, nh * 2 * dim), dtype, 23) * 3.0
    gate = _rand((n, nh), dtype, 24)
    seq = torch.tensor(np.repeat(np.arange(S), q_lens), dtype=torch.int32).cuda()
    pos = torch.tensor(np.concatenate([np.arange(k - c, k) for c, k in zip(q_lens, kv_lens)]), dtype=torch.int32).cuda()
    q_start = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32).cuda()
    kv = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    ref, out = torch.empty((n, nh * vdim), dtype=dtype, device="cuda"), torch.empty((n, nh * vdim), dtype=dtype, device="cuda")
    ops.diff_attention_simt(ref, q, k_pool, v_pool, order, seq, pos, gate, nh, dim**-0.5, window or None, keep, 0.45, 0.7, 1e-5)
    assert ops.diff_attention_tc_supported(dim, vdim)
    ops.diff_attention_tc(out, q, k_pool, v_pool, order, q_start, kv, S, max(q_lens), gate, nh, dim**-0.5, window or None, keep, 0.45, 0.7, 1e-5)
    assert not torch.isnan(out).any()
    assert torch.allclose(out.float(), ref.float(), atol=4e-2, rtol=2e-2)
    # single tokens alone, their key tiles divided between CTAs (more CTAs than the shortest context has tiles)
    singles = [i for i, c in enumerate(q_lens) if c == 1]
    rows = torch.tensor([int(q_start[i]) for i in singles]).cuda()
    for splits in (2, 3, 7):
        part = torch.full((len(singles), nh * vdim), float("nan"), dtype=dtype, device="cuda")
        scratch = torch.full((ops.diff_attention_scratch(len(singles), nh, vdim, splits),), float("nan"), dtype=torch.float32, device="cuda")
        ops.diff_attention_tc(part, q[rows].contiguous(), k_pool, v_pool, order[singles].contiguous(), torch.arange(len(singles) + 1, dtype=torch.int32).cuda(),
                              kv[singles].contiguous(), len(singles), 1, gate[rows].contiguous(), nh, dim**-0.5, window or None, keep, 0.45, 0.7, 1e-5, splits, scratch)
        assert torch.allclose(part.float(), out[rows].float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bounded_gate_times_shifted_up_kernel(dtype):
    from dli_b200.kernels import ops

    for n, inter, tiled in ((5, 37, False), (3, 128, True), (70, 64, False)):
        gu = _rand((n, 2 * inter), dtype, 3, 2.0)
        out, ref = torch.empty((n, inter), dtype=dtype, device="cuda"), torch.empty((n, inter), dtype=dtype)
        ops.silu_mul(out, gu, tiled, "quick_gelu", 1.2, 1.0)
        cpu_ops.silu_mul(ref, gu.cpu(), tiled, "quick_gelu", 1.2, 1.0)
        assert torch.allclose(out.float().cpu(), ref.float(), atol=1e-5 if dtype == torch.float32 else 3e-2)
    # the same in the epilogues of the two products that yield gate and up (bfloat16): a decode step's few tokens and a long portion,
    # with sums large enough for both bounds to act
    if dtype == torch.bfloat16:
        for tokens in (3, 700):
            x, wt = _rand((tokens, 256), dtype, 6, 0.5), _rand((384, 256), dtype, 7, 0.3)
            want = cpu_ops.skinny_gemm_swiglu(x.cpu(), wt.cpu(), "quick_gelu", 1.2, 1.0)
            got = (ops.skinny_gemm_swiglu if tokens <= 8 else ops.dense_gemm_swiglu)(x, wt, "quick_gelu", 1.2, 1.0)
            assert (want.float().abs() > 1.9).any()  # some gate and up at their bounds: 1.2 sigmoid(1.702 * 1.2) * 2.2 = 2.3
            assert torch.allclose(got.float().cpu(), want.float(), atol=3e-2, rtol=2e-2)
