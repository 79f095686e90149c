"""The Lokolorn model on the real kernels, in float32 and bfloat16, against the plain implementation: the cases of
tests/lokolorn_suite.py, trace replay as a child process, and steps replayed from CUDA graphs."""

import numpy as np
import pytest

from tests import lokolorn_suite as suite
from tests.plain import lokolorn_plain as plain
from tests.util import TraceRun

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, dtype, tmp_path):
    case(tmp_path, "cuda:0", dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_with_four_state_slots(dtype, tmp_path):
    """bin/trace_run on a schedule of six requests, four live at most, in a pool that holds three of them."""
    cfg = suite.pick("mixed_loop", dtype)
    w = suite.make_model(tmp_path / "m", cfg, seed=41)
    seqs = {f"r{i}": suite.tokens_for(cfg, n, seed=80 + i) for i, n in enumerate((40, 33, 21, 38, 27, 30))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    rounding = {r: suite.rounding_error(tmp_path / "m", "cuda:0", dtype, t, want[r]) for r, t in seqs.items()}
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
                suite.close(got[row : row + n].astype(np.float64), want[r][lo : lo + n], dtype, f"{r} at {lo}", rounding[r])
                row += n
            live = [r for r in live if r not in end]
            step += 1
    finally:
        run.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_from_graphs(dtype, tmp_path):
    """Steps of single tokens replay a CUDA graph; a step shape that keeps coming (a short portion of one request beside single
    tokens of two others) is captured after 32 sightings.  Padding rows use the scratch page and the scratch state slot.  Logits
    before and after the capture equal the plain model's."""
    cfg = suite.pick("mixed_loop", dtype)
    w = suite.make_model(tmp_path / "m", cfg, seed=43)
    s = suite.Session(tmp_path / "m", "cuda:0", dtype, pages=120, page_size=8)
    assert s.runner.graphs is not None
    long = suite.tokens_for(cfg, 3 * 48 + 1, seed=90)
    b, c = suite.tokens_for(cfg, 60, seed=91), suite.tokens_for(cfg, 60, seed=92)
    want = {"a": plain.forward(cfg, w, long), "b": plain.forward(cfg, w, b), "c": plain.forward(cfg, w, c)}
    s.step(("b", b[:10], []), ("c", c[:9], []))
    got = {"a": [], "b": [], "c": []}
    at = {"a": 0, "b": 10, "c": 9}
    for _ in range(48):
        out = s.step(("a", long[at["a"] : at["a"] + 3], [0, 1, 2]), ("b", [b[at["b"]]], [0]), ("c", [c[at["c"]]], [0]))
        got["a"].append(out[0:3]), got["b"].append(out[3:4]), got["c"].append(out[4:5])
        at["a"] += 3
        at["b"] += 1
        at["c"] += 1
    assert s.runner.mixed_graph_steps >= 10, s.runner.graphs.mixed_failure
    before = s.runner.graph_steps
    out = s.step(("a", [long[at["a"]]], [0]), ("b", [b[at["b"]]], [0]), ("c", [c[at["c"]]], [0]))  # three single tokens: a decode graph
    assert s.runner.graph_steps == before + 1
    got["a"].append(out[0:1]), got["b"].append(out[1:2]), got["c"].append(out[2:3])
    at = {r: at[r] + 1 for r in at}
    for r, first in (("a", 0), ("b", 10), ("c", 9)):
        seq = {"a": long, "b": b, "c": c}[r]
        suite.close(np.concatenate(got[r]), want[r][first : at[r]], dtype, f"request {r}",
                    suite.rounding_error(tmp_path / "m", "cuda:0", dtype, seq, want[r]))
