"""Cases that compare the engine's Pokadra model with the plain implementation (tests/plain/pokadra_plain.py).

Each case takes (tmp_path, device, dtype) and builds its own small configuration and weights.  The CPU tests run them on
torch stand-ins for the kernels (float32), the GPU tests on the real kernels in both dtypes.  Weights are drawn so that
faults show: sharp attention (one missing key changes the logits), update gates that are mostly closed (a lost state
changes later tokens), depth weights and pair rows of order one.
"""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import dli_b200
from dli_b200.config.registry import resolve_architecture
from dli_b200.engine import ModelRunner
from dli_b200.parts.model import declared_tensors
from dli_b200.weights import write_safetensors
from tests.pazenex_suite import TOL, Session, close
from tests.plain import pokadra_plain as plain

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.5, diff=0.3, rot_dims=8, base=10000.0, scaling=YARN, window=13, keep_first=3, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def mingru(width=40):
    return {"type": "mingru", "mixer": {"width": width}}


def config(layers, width=48, vocab=83, ff=56, limit=1.2, eps=1e-5, groups=3, mult=0.7, scale=2.0, pair=(101, 7, 13), side=6, no_mlp=()):
    out = {"architecture": "Pokadra", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "residual_mult": mult,
           "embedding": {"scale": scale}, "layers": []}
    if pair:
        out["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), pair))
    if side:
        out["token_side"] = {"dim": side}
    for i, layer in enumerate(layers):
        out["layers"].append({**layer, "mlp": None if i in no_mlp else {"kind": "dense", "ff": ff, "limit": limit}})
    return out


# sizes that differ from one another in every respect: head counts, one and several KV heads, key and value sizes that are
# and are not equal or a multiple of 8, whole and partial rotation, with and without scaling of the frequencies, windows that
# differ between layers, kept first tokens from none to more than a page, a reader of another layer's keys with a wider and
# with a narrower mask than its owner's, norm groups 1 to 4, factors of 1, no pair table, no token input, no feed-forward
CONFIGS = {
    "mixed": config([attention(), mingru(), attention(heads=2, kv_heads=1, dim=8, vdim=8, window=9, keep_first=0, rot_dims=8, scaling=None), mingru(24),
                     attention(kv_from=0, window=21, keep_first=5), mingru()]),
    "readers": config([attention(heads=3, kv_heads=3, dim=12, vdim=20, window=17, keep_first=10, rot_dims=4), attention(heads=3, kv_heads=3, dim=12, vdim=20, rot_dims=4,
                                                                                                                    window=6, keep_first=1, kv_from=0),
                       mingru(16), attention(heads=3, kv_heads=3, dim=12, vdim=20, rot_dims=4, window=None, kv_from=0)],
                      width=36, vocab=61, ff=64, groups=1, mult=1.0, scale=1.0, side=4, no_mlp=(1,)),
    "only_attention": config([attention(heads=2, kv_heads=2, dim=32, vdim=16, window=None, rot_dims=32), attention(heads=6, kv_heads=2, dim=8, vdim=40, window=5,
                                                                                                                   keep_first=2, rot_dims=0)],
                             width=64, vocab=130, ff=128, groups=4, pair=None),
    "only_mingru": config([mingru(48), mingru(10)], side=None, groups=2, no_mlp=(0,)),
    # nothing a multiple of 4 or 8
    "odd_sizes": config([mingru(7), attention(heads=3, kv_heads=1, dim=6, vdim=5, rot_dims=2, window=3, keep_first=1), attention(heads=3, kv_heads=1, dim=6, vdim=5,
                                                                                                                               rot_dims=2, window=7, keep_first=0, kv_from=1)],
                        width=45, vocab=59, ff=37, groups=5, pair=(53, 3, 1), side=3, eps=1e-6),
}


def make_model(path: Path, cfg: dict, seed: int = 0, sharp: float = 1.0) -> dict:
    """Writes the folder; returns the tensors as float64 arrays (as stored: values a bfloat16 engine reads unchanged)."""
    arch = resolve_architecture(cfg)
    decls = declared_tensors(arch.model_spec(arch.parse_config(cfg)))
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=g) * std

    tensors = {}
    for name, decl in sorted(decls.items()):
        shape = tuple(decl.shape)
        if name.endswith("q.norm") or name.endswith("k.norm"):
            t = sharp * (1.6 + normal(shape, 0.3))  # sharp attention: single keys matter
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = normal(shape, 0.25)
        elif name.endswith(".dwa"):
            t = 1.0 / shape[0] + normal(shape, 0.3)
        elif name.endswith("z.b"):
            t = -1.5 + normal(shape, 1.0)  # update gates mostly closed: the state remembers
        elif name.endswith("x.b"):
            t = normal(shape, 0.5)
        elif len(shape) == 1:
            t = 1.0 + normal(shape, 0.2)
        elif name in ("embed", "bigram", "side.embed"):
            t = normal(shape, 1.0)
        else:
            t = normal(shape, 1.0 / shape[1] ** 0.5)
        tensors[name] = t.to(torch.bfloat16).float()
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", tensors)
    return {k: v.double().numpy() for k, v in tensors.items()}


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def rounding_error(path, device, dtype, toks, want, **session):
    """What rounding alone does to this sequence in bfloat16: the error of the whole prompt, alone, in a fresh engine."""
    if dtype == "float32":
        return 0.0
    return float(np.abs(Session(path, device, dtype, **session).whole("alone", toks) - want).max())


# ----------------------------------------------------------------------------- cases


def case_every_configuration_whole_prompt_and_layers(tmp_path, device, dtype):
    """Whole prompts in every configuration: logits, and the stream behind every layer (in float32)."""
    for name, cfg in CONFIGS.items():
        w = make_model(tmp_path / name, cfg, seed=3)
        toks = tokens_for(cfg, 45, seed=1)
        layers = []
        want = plain.forward(cfg, w, toks, layers)
        s = Session(tmp_path / name, device, dtype)
        s.model.trace_layers = []
        got = s.whole("a", toks)
        close(got, want, dtype, name)
        assert len(s.model.trace_layers) == len(layers)
        if dtype == "float32":
            for i, (mine, theirs) in enumerate(zip(s.model.trace_layers, layers)):
                err = np.abs(mine.double().cpu().numpy() - theirs).max()
                assert err < 2e-4 * max(1.0, np.abs(theirs).max()), f"{name}: stream behind layer {i} differs by {err:.3g}"


def case_each_mixer_alone(tmp_path, device, dtype):
    for name, layer in (("attention", attention(heads=2, kv_heads=1, dim=16, vdim=16)), ("mingru", mingru(32))):
        cfg = config([layer], width=32, vocab=40, pair=None, side=None, groups=1, mult=1.0, scale=1.0, no_mlp=(0,))
        w = make_model(tmp_path / name, cfg, seed=5)
        toks = tokens_for(cfg, 30, seed=2)
        close(Session(tmp_path / name, device, dtype).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)


def case_prefill_then_token_by_token(tmp_path, device, dtype):
    """A prompt in one step and 40 tokens one by one (windows pass over decoded tokens, pages are given back while the
    kept first tokens stay), and a sequence token by token from its first token."""
    cfg = CONFIGS["mixed"]
    w = make_model(tmp_path / "m", cfg, seed=7)
    toks = tokens_for(cfg, 70, seed=3)
    want = plain.forward(cfg, w, toks)
    noise = rounding_error(tmp_path / "m", device, dtype, toks, want)
    s = Session(tmp_path / "m", device, dtype, pages=12, page_size=8)
    got = [s.step(("a", toks[:30], list(range(30))))] + [s.step(("a", [t], [0])) for t in toks[30:]]
    close(np.concatenate(got), want, dtype, "prompt then tokens", noise)
    s.manager.check_invariants()
    s.free("a")
    got = [s.step(("b", [t], [0])) for t in toks[:40]]
    close(np.concatenate(got), want[:40], dtype, "token by token", noise)


def case_portions_of_many_sizes(tmp_path, device, dtype):
    """Portions of 2 to 17 tokens, cut inside pages and windows."""
    for name in ("mixed", "odd_sizes", "readers"):
        cfg = CONFIGS[name]
        w = make_model(tmp_path / name, cfg, seed=11)
        toks = tokens_for(cfg, 75, seed=4)
        want = plain.forward(cfg, w, toks)
        noise = rounding_error(tmp_path / name, device, dtype, toks, want)
        for sizes in ((2, 2, 3, 17, 5, 2, 9, 1, 1, 2, 13, 2, 7, 2, 7), (16, 8, 24, 3, 24), (1, 2, 64, 8)):
            s = Session(tmp_path / name, device, dtype, pages=14, page_size=8)
            at, got = 0, []
            for n in sizes:
                got.append(s.step(("a", toks[at : at + n], list(range(n)))))
                at += n
            close(np.concatenate(got), want[:at], dtype, f"{name} in portions {sizes}", noise)
            s.manager.check_invariants()


def case_batches_of_unequal_requests(tmp_path, device, dtype):
    """Four live requests, portions of some beside single tokens of others, against each alone."""
    cfg = CONFIGS["mixed"]
    w = make_model(tmp_path / "m", cfg, seed=13)
    seqs = {r: tokens_for(cfg, n, seed=20 + i) for i, (r, n) in enumerate((("a", 50), ("b", 23), ("c", 37), ("d", 9)))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    noise = max(rounding_error(tmp_path / "m", device, dtype, seqs[r], want[r]) for r in seqs)
    s = Session(tmp_path / "m", device, dtype, pages=30, page_size=8)
    at = {r: 0 for r in seqs}
    plan = {"a": (11, 1, 1, 20, 1, 2, 14), "b": (1, 1, 1, 5, 15), "c": (30, 1, 1, 1, 1, 3), "d": (2, 1, 2, 1, 1, 2)}
    got = {r: [] for r in seqs}
    for step in range(8):
        parts = []
        for r in seqs:
            if step < len(plan[r]):
                n = plan[r][step]
                parts.append((r, seqs[r][at[r] : at[r] + n], list(range(n))))
        if not parts:
            break
        out = s.step(*parts)
        row = 0
        for r, t, _ in parts:
            got[r].append(out[row : row + len(t)])
            row += len(t)
            at[r] += len(t)
    for r in seqs:
        assert at[r] == len(seqs[r])
        close(np.concatenate(got[r]), want[r], dtype, f"request {r} in a batch", noise)
    s.manager.check_invariants()


def case_pages_and_slots_used_again(tmp_path, device, dtype):
    """Eight requests through a pool that holds two of them and two state slots: pages, recurrent state and the previous token
    of a finished request must not leak into the next."""
    cfg = CONFIGS["mixed"]
    w = make_model(tmp_path / "m", cfg, seed=17)
    s = Session(tmp_path / "m", device, dtype, pages=16, page_size=8, max_requests=2)
    live = []
    for i in range(8):
        toks = tokens_for(cfg, 30 + 3 * i, seed=40 + i)
        if len(live) == 2:
            s.free(live.pop(0))
        cut = len(toks) // 2
        a = s.step((i, toks[:cut], list(range(cut))))
        b = s.step((i, toks[cut:], list(range(len(toks) - cut))))
        want = plain.forward(cfg, w, toks)
        close(np.concatenate([a, b]), want, dtype, f"request {i}", rounding_error(tmp_path / "m", device, dtype, toks, want))
        live.append(i)
    s.manager.check_invariants()


def _deciding_pair(cfg, w, margin=8.0):
    """(asker, key, noise tokens) for a first layer of attention without rotation and a model without pair table: map 1 of
    the asker's first head puts nearly all its mass on ``key`` among the noise tokens."""
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    x = plain.embed(cfg, w, np.arange(cfg["vocab"]))
    d = m["dim"]
    q = (plain.rms_unit((x @ w["l0.mix.q"].T)[:, :d], eps) * w["l0.mix.q.norm"])
    k = (plain.rms_unit((x @ w["l0.mix.k"].T)[:, :d], eps) * w["l0.mix.k.norm"])
    scores = (q @ k.T) * m["scale"]
    asker = next(t for t in range(cfg["vocab"]) if scores[t].argmax() != t and np.sort(scores[t])[-1] - np.sort(scores[t])[-2] > margin)
    key = int(scores[asker].argmax())
    noise = [t for t in range(cfg["vocab"]) if scores[asker, t] < scores[asker, key] - margin and t != asker]
    assert len(noise) > 15
    return asker, key, noise


def case_one_far_key_decides(tmp_path, device, dtype):
    """Attention without a window, and a sequence made so that one map of the last token's first head puts nearly all its mass
    on ONE key far back — at a page border, beside one, at the very start: a kernel that skips or misplaces that key changes
    the logits by far more than the tolerance.  In a prompt portion and decoded."""
    cfg = config([attention(heads=2, kv_heads=1, dim=16, vdim=24, rot_dims=0, scale=6.0, window=None)], width=32, vocab=50, pair=None, side=None, groups=2, no_mlp=(0,))
    w = make_model(tmp_path / "far", cfg, seed=19, sharp=2.0)
    asker, key, noise = _deciding_pair(cfg, w)
    s = Session(tmp_path / "far", device, dtype, pages=48, page_size=8)
    for far in (8, 15, 16, 1, 0, 100, 263):
        toks = [noise[i] for i in np.random.default_rng(far).integers(0, len(noise), 330)]
        toks[far] = key
        toks[-1] = asker
        want = plain.forward(cfg, w, toks)
        without = list(toks)
        without[far] = noise[0]
        assert np.abs(plain.forward(cfg, w, without)[-1] - want[-1]).max() > 0.2, "the far key does not matter enough for this test"
        close(s.whole("p", toks)[-1], want[-1], dtype, f"far key {far} in a prompt")
        s.free("p")
        s.step(("d", toks[:-1], []))
        close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"far key {far} decoded")
        s.free("d")


def case_keys_at_the_edges_of_the_mask(tmp_path, device, dtype):
    """The deciding key on the last place the window still holds (it decides) and one place beyond (unseen); on the last of
    the kept first tokens (it decides although the window passed it long ago) and on the first token that is not kept
    (unseen).  In a prompt, decoded alone, and inside a last portion; edges inside a page and on a page border."""
    window, keep = 24, 5
    cfg = config([attention(heads=2, kv_heads=1, dim=16, vdim=24, rot_dims=0, scale=6.0, window=window, keep_first=keep)], width=32, vocab=50, pair=None,
                 side=None, groups=2, no_mlp=(0,))
    w = make_model(tmp_path / "edge", cfg, seed=19, sharp=2.0)
    asker, key, noise = _deciding_pair(cfg, w)
    s = Session(tmp_path / "edge", device, dtype, pages=24, page_size=8)
    for length in (60, 57, 100):
        last = length - 1
        places = {"window_in": last - window + 1, "window_out": last - window, "first_in": keep - 1, "first_out": keep}
        logits = {}
        for name, place in places.items():
            toks = [noise[i] for i in np.random.default_rng(length).integers(0, len(noise), length)]
            toks[place] = key
            toks[last] = asker
            want = plain.forward(cfg, w, toks)
            logits[name] = want[-1]
            close(s.whole("p", toks)[-1], want[-1], dtype, f"key {name} at {place}, prompt of {length}")
            s.free("p")
            s.step(("d", toks[:-1], []))
            close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"key {name} at {place}, decoded at {last}")
            s.free("d")
            s.step(("c", toks[:-3], []))
            close(s.step(("c", toks[-3:], [2]))[0], want[-1], dtype, f"key {name} at {place}, in a last portion of 3")
            s.free("c")
            s.manager.check_invariants()
        matters = min(np.abs(logits["window_in"] - logits["window_out"]).max(), np.abs(logits["first_in"] - logits["first_out"]).max())
        assert matters > 0.2, "the keys at the mask's edges do not matter enough for this test"


def case_the_token_in_front(tmp_path, device, dtype):
    """The pair table reads the token in front: inside a portion, across a cut (from the state slot), and not at all for a
    sequence's first token; a slot that another request used before must not hand on its last token."""
    cfg = config([mingru(16)], width=32, vocab=30, pair=(17, 5, 3), side=None, groups=4, no_mlp=(0,))
    w = make_model(tmp_path / "p", cfg, seed=37)
    a, b = tokens_for(cfg, 12, seed=5), tokens_for(cfg, 9, seed=6)
    swapped = list(a)
    swapped[4] = (a[4] + 1) % cfg["vocab"]
    assert np.abs(plain.forward(cfg, w, swapped)[5] - plain.forward(cfg, w, a)[5]).max() > 0.05, "the token in front does not matter enough for this test"
    s = Session(tmp_path / "p", device, dtype, max_requests=1)
    got = np.concatenate([s.step(("a", a[:5], list(range(5)))), s.step(("a", a[5:6], [0])), s.step(("a", a[6:], list(range(6))))])
    close(got, plain.forward(cfg, w, a), dtype, "cuts behind token 4 and 5")
    s.free("a")
    close(s.whole("b", b), plain.forward(cfg, w, b), dtype, "the same slot, another request")
    s.free("b")
    for n in (1, 2, 3):
        close(s.whole("c", a[:n]), plain.forward(cfg, w, a[:n]), dtype, f"a sequence of {n}")
        s.free("c")


def case_long_decoding(tmp_path, device, dtype):
    """300 decoded tokens through minGRU layers, windows and kept first tokens, in a pool that only holds what the masks keep."""
    cfg = CONFIGS["mixed"]
    w = make_model(tmp_path / "m", cfg, seed=43)
    toks = tokens_for(cfg, 320, seed=8)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "m", device, dtype, pages=48, page_size=8)
    got = [s.step(("a", toks[:20], [19]))] + [s.step(("a", [t], [0])) for t in toks[20:]]
    close(np.concatenate(got), want[19:], dtype, "long decoding", rounding_error(tmp_path / "m", device, dtype, toks, want, pages=48))
    s.manager.check_invariants()


def case_long_portions(tmp_path, device, dtype):
    """Portions long enough for the recurrence's two-level walk (several chunks of a sequence, beside a short one)."""
    cfg = config([mingru(40), attention(window=40, keep_first=2)], no_mlp=(0,))
    w = make_model(tmp_path / "l", cfg, seed=47)
    a, b = tokens_for(cfg, 700, seed=9), tokens_for(cfg, 41, seed=10)
    wa, wb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    s = Session(tmp_path / "l", device, dtype, pages=120, page_size=8)
    s.step(("b", b[:40], []))
    first = s.step(("a", a[:333], [0, 100, 332]), ("b", b[40:], [0]))
    close(first[:3], wa[[0, 100, 332]], dtype, "a long portion", rounding_error(tmp_path / "l", device, dtype, a, wa, pages=120))
    close(first[3], wb[40], dtype, "a single token beside it")
    second = s.step(("a", a[333:], [0, 200, 366]))
    close(second, wa[[333, 533, 699]], dtype, "the second long portion", rounding_error(tmp_path / "l", device, dtype, a, wa, pages=120))


def case_greedy_generation_through_the_engine(tmp_path, device, dtype):
    """LLMEngine.generate (scheduler, batching, sampler) against greedy decoding with the plain model."""
    from dli_b200 import LLMEngine, SamplingParams, SchedulerConfig

    cfg = CONFIGS["mixed"]
    w = make_model(tmp_path / "g", cfg, seed=31)
    prompts = [tokens_for(cfg, n, seed=60 + n) for n in (5, 19, 1, 11, 8)]
    if device == "cpu":
        from tests import cpu_ops

        model = dli_b200.load_model(tmp_path / "g", dtype, device)
        runner = ModelRunner(model, num_pages=32, page_size=8, max_requests=4, cuda_graphs=False)
        engine = LLMEngine(runner, SchedulerConfig(4, 24), sampler=cpu_ops.CpuSampler())
    else:
        engine = LLMEngine.from_model_dir(tmp_path / "g", dtype=dtype, device=device, num_blocks=32, block_size=8, config=SchedulerConfig(4, 24))
    outs = engine.generate(prompts, SamplingParams(max_tokens=10))
    tol = TOL[dtype]
    compared = 0
    for p, got in zip(prompts, outs):
        toks = list(p)
        for t in got:
            row = plain.forward(cfg, w, toks)[-1]
            top = np.sort(row)[-2:]
            if int(np.argmax(row)) != t:
                assert top[1] - top[0] < 2 * tol * max(1.0, np.abs(row).max()), "a generated token differs from the plain model's"
                break
            toks.append(t)
            compared += 1
    assert compared >= 25


CASES = [v for k, v in sorted(globals().items()) if k.startswith("case_")]
