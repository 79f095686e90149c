"""Cases that compare the engine's Lokolorn model with the plain implementation (tests/plain/lokolorn_plain.py).

Each case takes (tmp_path, device, dtype) and builds its own small configuration and weights.  The CPU tests run them on
torch stand-ins for the kernels (float32), the GPU tests on the real kernels in both dtypes.  Weights are drawn so that
faults show: decays close to one (a lost state changes later tokens), sharp attention (one missing key changes the
logits), convolution taps, layer scales and token-shift blends of order one, corrections that change the routing.
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
from tests.plain import lokolorn_plain as plain


def parallel(heads=4, kv_heads=2, dim=16, vdim=8, conv=3, scale=0.7, rot_dims=8, base=100.0, r_heads=2, r_dim=12, rank=6, left_scale=0.9, right_scale=0.6):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "decay_rank": rank}, "left_scale": left_scale,
                                          "right_scale": right_scale}}


def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, decay_rank=5, gate_rank=7):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
                                               "gate_rank": gate_rank}}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.6, base=1000.0, window=13, scaling=(4.0, 32, 8.0, 1.0)):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        m["rot_dim"] = rot_dim
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def moe(ff=20, experts=6, top=2, scale=1.25, groups=(3, 2)):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(layers, width=48, vocab=89, mlp=None, loop=None, eps=1e-5, no_mlp=()):
    out = {"architecture": "Lokolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for i, layer in enumerate(layers):
        out["layers"].append({**layer, "mlp": None if i in no_mlp else (mlp or moe())})
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# sizes that differ from one another in every respect: head counts, key and value sizes equal and unequal (values longer and
# shorter than keys), partial, full and no rotation, one to four taps, several heads per key/value head and one, cache rows
# that are and are not multiples of 16, with and without windows and frequency scaling, experts in groups and not, one
# choice and several, loops over a middle span, from the first layer, once, three times, absent; layers without feed-forward
CONFIGS = {
    "mixed_loop": config([parallel(), delta(), latent(), delta(heads=2, kv_heads=2, dim=8, vdim=20, conv=4)], loop=(1, 3, 3)),
    "loop_from_start": config([delta(heads=3, kv_heads=1, dim=20, vdim=10, conv=2), parallel(heads=2, kv_heads=1, dim=8, vdim=24, conv=2, rot_dims=8, r_heads=3, r_dim=8)],
                              width=40, mlp=moe(ff=16, experts=4, top=1, groups=None), loop=(0, 2, 2), no_mlp=(0,)),
    "no_loop": config([latent(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=96, scale=0.3, window=None), parallel(heads=4, kv_heads=4, dim=16, vdim=16, conv=1, rot_dims=0),
                       delta(heads=2, kv_heads=1, dim=64, vdim=32, conv=1)], width=64, vocab=130, mlp=moe(ff=64, experts=12, top=4, groups=(3, 1)), no_mlp=(2,)),
    "loop_once": config([delta(), latent(heads=1, dim=16, rot_dim=0, vdim=48, kv_rank=20, window=5)], loop=(1, 2, 1), eps=1e-6,
                        mlp=moe(ff=24, experts=5, top=5, groups=None, scale=1.0)),
    "only_parallel": config([parallel(), parallel(heads=3, kv_heads=1, dim=32, vdim=32, conv=4, rot_dims=32, r_heads=1, r_dim=40)], loop=(0, 2, 2)),
    "only_latent": config([latent(), latent(heads=5, dim=8, rot_dim=16, vdim=8, kv_rank=112, window=36, scaling=None)], loop=(0, 2, 2), mlp=moe(experts=9, top=3, groups=(3, 1))),
    # nothing a multiple of 4 or 8
    "odd_sizes": config([latent(heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=13), delta(heads=3, kv_heads=1, dim=9, vdim=7, conv=5, decay_rank=3, gate_rank=2),
                         parallel(heads=3, kv_heads=3, dim=10, vdim=7, conv=2, rot_dims=6, r_heads=3, r_dim=5, rank=3)], width=50, vocab=61,
                        mlp=moe(ff=11, experts=10, top=3, groups=(5, 2)), loop=(1, 3, 2)),
}


def make_model(path: Path, cfg: dict, seed: int = 0, sharp: float = 1.0, edit=None) -> dict:
    """Writes the folder; returns the tensors as float64 arrays (as stored: values a bfloat16 engine reads unchanged).
    ``edit(tensors)`` may change the tensors before they are written."""
    arch = resolve_architecture(cfg)
    decls = declared_tensors(arch.model_spec(arch.parse_config(cfg)))
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std):
        return torch.randn(shape, generator=g) * std

    def uniform(shape, lo, hi):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    tensors = {}
    for name, decl in sorted(decls.items()):
        shape = tuple(decl.shape)
        if name.endswith("A_log"):
            t = uniform(shape, -5.0, -2.0)  # decays close to one: the state remembers
        elif name.endswith("dt_bias"):
            t = uniform(shape, -2.0, 0.5)
        elif name.endswith(".w0"):
            t = uniform(shape, -5.0, -2.0)  # exp(-exp(w0)) close to one
        elif name.endswith(".conv"):
            t = normal(shape, 0.6)
        elif ".mu." in name:
            t = uniform(shape, 0.0, 1.0)
        elif name.endswith("ls1") or name.endswith("ls2"):
            t = uniform(shape, 0.5, 1.5)
        elif name.endswith("right.u"):
            t = normal(shape, 0.5)
        elif name.endswith("correction"):
            t = normal(shape, 0.3)
        elif name.endswith("sink"):
            t = normal(shape, 1.0)
        elif name.endswith("dkv.norm"):
            t = sharp * (1.5 + normal(shape, 0.3))  # sharp attention: single keys matter
        elif name.endswith("mix.norm") or name.endswith("right.norm"):
            t = 1.0 + normal(shape, 0.2)
        elif name.endswith(".b"):
            t = normal(shape, 0.3) if len(shape) == 1 else normal(shape, 1.0 / shape[1] ** 0.5)
        elif len(shape) == 1:
            t = normal(shape, 0.2)  # norm weights are stored as the deviation from one
        elif name == "embed":
            t = normal(shape, 1.0)
        elif name == "loop.in":
            t = normal(shape, 1.0 / (shape[1] / 2) ** 0.5)
        elif name.endswith("router"):
            t = normal(shape, 2.0 / shape[1] ** 0.5)
        else:
            t = normal(shape, 1.0 / shape[1] ** 0.5)
        tensors[name] = t.to(torch.bfloat16).float()
    if edit is not None:
        edit(tensors)
        tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", tensors)
    return {k: v.double().numpy() for k, v in tensors.items()}


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def rounding_error(path, device, dtype, toks, want):
    """What rounding alone does to this sequence in bfloat16: the error of the whole prompt, alone, in a fresh engine."""
    if dtype == "float32":
        return 0.0
    return float(np.abs(Session(path, device, dtype, pages=len(toks) // 8 + 2).whole("alone", toks) - want).max())


def forward_with_layers(cfg, w, toks):
    trace = []
    return plain.forward(cfg, w, toks, trace), np.stack(trace)


def all_experts_chosen(cfg):
    """The same configuration with every expert chosen.  In bfloat16 a token whose choice between two experts is a close call may take
    the other one than the float64 model, and over hundreds of (token, layer run) pairs some call is always close; with nothing to
    choose only the weights remain.  (Choices are compared exactly in float32, and kernel by kernel on equal inputs.)"""
    out = json.loads(json.dumps(cfg))
    for layer in out["layers"]:
        if layer.get("mlp"):
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
            layer["mlp"]["router"].pop("groups", None)
    return out


def steady(cfg, dtype):
    """``cfg`` as a case runs it in ``dtype``: as it is in float32, with every expert chosen in bfloat16."""
    return all_experts_chosen(cfg) if dtype == "bfloat16" else cfg


def pick(name, dtype):
    return steady(CONFIGS[name], dtype)


# ----------------------------------------------------------------------------- cases


def case_every_configuration_whole_prompt_and_layers(tmp_path, device, dtype):
    """Whole prompts in every configuration: logits, and the stream after every layer run (in float32)."""
    for name, cfg in CONFIGS.items():
        cfg = steady(cfg, dtype)
        w = make_model(tmp_path / name, cfg, seed=3)
        toks = tokens_for(cfg, 77, seed=1)
        want, layers = forward_with_layers(cfg, w, toks)
        s = Session(tmp_path / name, device, dtype)
        s.model.trace_layers = []
        got = s.whole("a", toks)
        close(got, want, dtype, name)
        assert len(s.model.trace_layers) == layers.shape[0] == len(plain.layer_runs(cfg)), name
        if dtype == "float32":
            for i, h in enumerate(s.model.trace_layers):
                close(h.double().cpu().numpy(), layers[i], dtype, f"{name}: stream after layer run {i}")
        s.model.trace_layers = None


def case_each_mechanism_alone(tmp_path, device, dtype):
    """One layer, no loop: each mixer with nothing beside it (each half of the parallel mixer with the other's factor at zero), each
    mixer's variants, and the routed feed-forward's variants beside the simplest mixer; cache rows of 64 and 128 numbers (which the
    TMA-fed attention kernels take in bfloat16) and of a size that is no multiple of 16."""
    layers = {
        "attention_half": parallel(right_scale=0.0),
        "recurrence_half": parallel(left_scale=0.0, r_heads=3, r_dim=20),
        "attention_rows_64": parallel(heads=4, kv_heads=2, dim=64, vdim=48, conv=3, rot_dims=64, right_scale=0.1),
        "attention_values_longer": parallel(heads=2, kv_heads=2, dim=16, vdim=48, conv=2, rot_dims=4),
        "attention_rows_128": parallel(heads=2, kv_heads=1, dim=128, vdim=128, conv=3, rot_dims=32, r_heads=1, r_dim=64),
        "recurrence_wide": parallel(left_scale=0.2, r_heads=2, r_dim=72, rank=8),
        "delta": delta(heads=6, kv_heads=2, dim=12, vdim=10, conv=3),
        "delta_one_tap": delta(heads=1, kv_heads=1, dim=32, vdim=64, conv=1),
        "delta_wide": delta(heads=2, kv_heads=2, dim=136, vdim=40, conv=4),
        "latent": latent(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=24, scale=0.9),
        "latent_no_rotation_no_window": latent(heads=2, dim=16, rot_dim=0, vdim=8, kv_rank=24, window=None),
        "latent_row_64": latent(heads=8, dim=16, rot_dim=16, vdim=32, kv_rank=48, window=20),
        "latent_row_128": latent(heads=5, dim=24, rot_dim=32, vdim=16, kv_rank=96, window=30),
        "latent_row_odd": latent(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=21, window=9),
    }
    for name, layer in layers.items():
        cfg = config([layer], no_mlp=(0,))
        w = make_model(tmp_path / name, cfg, seed=5)
        toks = tokens_for(cfg, 45, seed=2)
        close(Session(tmp_path / name, device, dtype, pages=12).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)
    routed = {"no_groups": moe(ff=16, experts=7, top=3, groups=None), "one_choice": moe(ff=24, experts=4, top=1, groups=(2, 1)),
              "all_chosen": moe(ff=8, experts=4, top=4, groups=(2, 2)), "groups_of_one": moe(ff=64, experts=6, top=2, groups=(6, 3)),
              "many": moe(ff=32, experts=40, top=6, groups=(8, 3), scale=2.5)}
    for name, mlp in routed.items():
        cfg = config([latent(heads=1, dim=8, rot_dim=0, vdim=8, kv_rank=16, window=3)], mlp=mlp)
        w = make_model(tmp_path / name, cfg, seed=6)
        toks = tokens_for(cfg, 30, seed=3)
        close(Session(tmp_path / name, device, dtype).whole("a", toks), plain.forward(cfg, w, toks), dtype, name)


def case_routing_follows_the_correction_and_the_groups(tmp_path, device, dtype):
    """A correction that lifts one expert far above the rest makes every token choose it, weighted by its score WITHOUT the
    correction; a correction that sinks a group's second-best expert makes the group lose although it holds the best one."""
    mlp = moe(ff=16, experts=6, top=2, groups=(3, 1))
    cfg = config([latent(heads=1, dim=8, rot_dim=0, vdim=8, kv_rank=16, window=3)], mlp=mlp)

    def lift(t):
        t["l0.mlp.correction"] = torch.tensor([5.0, -9.0, 0.0, 0.0, 0.1, 0.1])  # group 0 holds the best expert and a hopeless one

    w = make_model(tmp_path / "r", cfg, seed=8, edit=lift)
    toks = tokens_for(cfg, 25, seed=4)
    ids, weights = plain.route(plain.offset_norm(np.random.default_rng(0).normal(size=(50, 48)), w["l0.norm2"], 1e-5), w, "l0.mlp.", mlp["router"])
    assert (ids >= 2).all(), "the group with the best expert should lose on the sum of its two best"
    close(Session(tmp_path / "r", device, dtype).whole("a", toks), plain.forward(cfg, w, toks), dtype, "routing")


def case_prefill_then_token_by_token(tmp_path, device, dtype):
    """A prompt in one step, then 60 tokens one at a time (the windows pass over decoded tokens), against the whole sequence at once;
    and a sequence fed token by token from its very first token."""
    cfg = pick("mixed_loop", dtype)
    w = make_model(tmp_path / "m", cfg, seed=7)
    toks = tokens_for(cfg, 95, seed=3)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "m", device, dtype, pages=40)
    got = [s.step(("a", toks[:35], list(range(35))))]
    got += [s.step(("a", [t], [0])) for t in toks[35:]]
    close(np.concatenate(got), want, dtype, "prompt then decode", rounding_error(tmp_path / "m", device, dtype, toks, want))
    s.free("a")
    got = [s.step(("b", [t], [0])) for t in toks[:20]]
    close(np.concatenate(got), want[:20], dtype, "token by token from the start")


def case_long_decoding(tmp_path, device, dtype):
    """A short prompt and 300 decoded tokens: the states are carried through hundreds of steps, pages behind the windows are given back."""
    cfg = config([delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=4), parallel(heads=2, kv_heads=1, dim=8, vdim=8, r_heads=2, r_dim=8),
                  latent(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=21)], loop=(0, 2, 2), width=32, mlp=moe(ff=16, experts=4, top=2, groups=(2, 1)))
    cfg = steady(cfg, dtype)
    w = make_model(tmp_path / "l", cfg, seed=9)
    toks = tokens_for(cfg, 310, seed=4)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "l", device, dtype, pages=88, page_size=8)
    s.step(("a", toks[:10], []))
    got = np.concatenate([s.step(("a", [t], [0])) for t in toks[10:]])
    close(got, want[10:], dtype, "long decoding", rounding_error(tmp_path / "l", device, dtype, toks, want))
    forgot = plain.forward(cfg, w, toks[200:])
    assert np.abs(forgot[-1] - want[-1]).max() > 0.05, "the state does not remember enough for this test"


def case_portions_of_many_sizes(tmp_path, device, dtype):
    """Portions down to two tokens and single tokens between them, cut inside pages and windows and shorter than the convolution's
    reach; the token in front of a portion's first one comes from the state."""
    for name in ("mixed_loop", "loop_from_start", "no_loop", "odd_sizes"):
        cfg = pick(name, dtype)
        w = make_model(tmp_path / name, cfg, seed=11)
        toks = tokens_for(cfg, 64, seed=5)
        want = plain.forward(cfg, w, toks)
        s = Session(tmp_path / name, device, dtype)
        got, at = [], 0
        for n in (2, 1, 2, 3, 1, 1, 9, 2, 16, 1, 7, 2, 2, 15):
            got.append(s.step(("a", toks[at : at + n], list(range(n)))))
            at += n
        assert at == 64
        close(np.concatenate(got), want, dtype, name, rounding_error(tmp_path / name, device, dtype, toks, want))


def case_batches_of_unequal_requests(tmp_path, device, dtype):
    """Up to four live requests: portions of some beside single tokens of others; a request sits out a step; the logits of each equal
    those of the request alone."""
    cfg = pick("mixed_loop", dtype)
    w = make_model(tmp_path / "m", cfg, seed=13)
    seqs = {r: tokens_for(cfg, n, seed=20 + i) for i, (r, n) in enumerate((("a", 50), ("b", 33), ("c", 9), ("d", 41)))}
    want = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    s = Session(tmp_path / "m", device, dtype, pages=40)
    at = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}
    plan = [{"a": 17, "b": 2}, {"a": 1, "b": 20, "c": 3}, {"a": 1, "c": 1, "d": 30}, {"b": 1, "c": 1, "d": 1, "a": 9}, {"a": 2, "b": 2, "c": 2, "d": 2},
            {"a": 1, "b": 1, "c": 1, "d": 1}, {"d": 1, "c": 1}, {"a": 19, "b": 7, "d": 7}]
    for step in plan:
        parts = []
        for r, n in step.items():
            n = min(n, len(seqs[r]) - at[r])
            parts.append((r, seqs[r][at[r] : at[r] + n], list(range(n))))
        out = s.step(*parts)
        row = 0
        for r, t, _ in parts:
            got[r].append(out[row : row + len(t)])
            row += len(t)
            at[r] += len(t)
    for r in seqs:
        close(np.concatenate(got[r]), want[r][: at[r]], dtype, f"request {r}", rounding_error(tmp_path / "m", device, dtype, seqs[r], want[r]))


def case_pages_and_slots_used_again(tmp_path, device, dtype):
    """A pool for two short requests and two state slots: request after request takes the pages and the slot a finished one gave
    back, and computes what it would compute in a fresh engine."""
    cfg = pick("mixed_loop", dtype)
    w = make_model(tmp_path / "m", cfg, seed=17)
    s = Session(tmp_path / "m", device, dtype, pages=8, page_size=8, max_requests=2)
    seqs = [tokens_for(cfg, n, seed=40 + i) for i, n in enumerate((30, 25, 31, 12, 28))]
    live = []
    for i, toks in enumerate(seqs):
        if len(live) == 2:
            s.free(live.pop(0))
        cut = len(toks) // 2
        a = s.step((i, toks[:cut], list(range(cut))))
        b = s.step((i, toks[cut:], list(range(len(toks) - cut))))
        want = plain.forward(cfg, w, toks)
        close(np.concatenate([a, b]), want, dtype, f"request {i}", rounding_error(tmp_path / "m", device, dtype, toks, want))
        live.append(i)
    s.manager.check_invariants()


def _quiet_sink(t):
    for k in t:
        if k.endswith("sink"):
            t[k] = torch.full_like(t[k], -30.0)


def _latent_pair(cfg, w):
    """In a model of one latent layer without positions a score depends on the two tokens alone.  Returns a token whose first head
    gives one other token's key a score far above every other's, that token, and tokens whose keys it scores far below."""
    mix, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    h = plain.offset_norm(w["embed"], w["l0.norm1"], eps)
    q = (h @ w["l0.mix.q"].T)[:, : mix["dim"]]
    c = plain.rms_unit(h @ w["l0.mix.dkv"].T, eps) * w["l0.mix.dkv.norm"]
    k = (c @ w["l0.mix.uk"].T)[:, : mix["dim"]]
    return _pick(q @ k.T * mix["scale"], cfg["vocab"])


def _pick(scores, V):
    asker = next(t for t in range(V) if scores[t].argmax() != t and np.sort(scores[t])[-1] - np.sort(scores[t])[-2] > 8)
    key = int(scores[asker].argmax())
    noise = [t for t in range(V) if scores[asker, t] < scores[asker, key] - 8 and t != asker]
    assert len(noise) > 20
    return asker, key, noise


def _far_key_rounds(tmp_path, device, dtype, cfg, w, asker, key, noise, name):
    s = Session(tmp_path / name, device, dtype, pages=48, page_size=8)
    for far in (8, 15, 16, 1, 0, 100, 263):
        toks = [noise[i] for i in np.random.default_rng(far).integers(0, len(noise), 330)]
        toks[far] = key
        toks[-1] = asker
        want = plain.forward(cfg, w, toks)
        without = list(toks)
        without[far] = noise[0]
        assert np.abs(plain.forward(cfg, w, without)[-1] - want[-1]).max() > 0.5, "the far key does not matter enough for this test"
        close(s.whole("p", toks)[-1], want[-1], dtype, f"{name}: far key {far} in a prompt")
        s.free("p")
        s.step(("d", toks[:-1], []))
        close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"{name}: far key {far} decoded")
        s.free("d")


def case_one_far_key_decides(tmp_path, device, dtype):
    """Sequences made so that the last token's first head puts nearly all its mass on ONE key among hundreds — at a page border,
    beside one, at the very start: a kernel that skips or misplaces that key changes the logits by far more than the tolerance.
    In a prompt portion and decoded; over the latent (no window, no positions, a sink that stays out of the way) and in the
    attention half of a parallel mixer (no rotation, a convolution that passes the token itself, a large scale)."""
    cfg = config([latent(heads=2, dim=16, rot_dim=0, vdim=16, kv_rank=24, scale=3.0, window=None)], width=32, vocab=50, no_mlp=(0,))
    w = make_model(tmp_path / "far_latent", cfg, seed=19, edit=_quiet_sink)
    _far_key_rounds(tmp_path, device, dtype, cfg, w, *_latent_pair(cfg, w), "far_latent")

    cfg = config([parallel(heads=2, kv_heads=1, dim=16, vdim=24, conv=3, scale=9.0, rot_dims=0, right_scale=0.0)], width=32, vocab=50, no_mlp=(0,))

    def pass_through(t):
        for k in t:
            if k.endswith(".conv") and ".left." in k:
                t[k] = torch.zeros_like(t[k])
                t[k][:, -1] = 1.0

    w = make_model(tmp_path / "far_left", cfg, seed=21, edit=pass_through)
    eps = cfg["norm"]["eps"]
    h = plain.offset_norm(w["embed"], w["l0.norm1"], eps)
    q = plain.rms_unit((h @ w["l0.mix.left.q"].T + w["l0.mix.left.q.b"])[:, :16], eps)
    k = plain.rms_unit(h @ w["l0.mix.left.k"].T + w["l0.mix.left.k.b"], eps)
    _far_key_rounds(tmp_path, device, dtype, cfg, w, *_pick(q @ k.T * 9.0, 50), "far_left")


def case_one_key_at_the_window_s_edge(tmp_path, device, dtype):
    """The same construction over the latent with a window of 24 keys: the deciding key sits on the last place the window still
    holds (it decides), and one place further back (it must not be seen); in a prompt, decoded alone and inside a last portion, with
    the window's edge inside a page and on a page border."""
    window = 24
    cfg = config([latent(heads=2, dim=16, rot_dim=0, vdim=16, kv_rank=24, scale=3.0, window=window)], width=32, vocab=50, no_mlp=(0,))
    w = make_model(tmp_path / "edge", cfg, seed=19, edit=_quiet_sink)
    asker, key, noise = _latent_pair(cfg, w)
    s = Session(tmp_path / "edge", device, dtype, pages=24, page_size=8)
    for length in (60, 57):
        last = length - 1
        inside, outside = last - window + 1, last - window
        logits = {}
        for name, place in (("inside", inside), ("outside", outside)):
            toks = [noise[i] for i in np.random.default_rng(length).integers(0, len(noise), length)]
            toks[place] = key
            toks[last] = asker
            want = plain.forward(cfg, w, toks)
            logits[name] = want[-1]
            close(s.whole("p", toks)[-1], want[-1], dtype, f"key {name} the window, prompt of {length}")
            s.free("p")
            s.step(("d", toks[:-1], []))
            close(s.step(("d", toks[-1:], [0]))[0], want[-1], dtype, f"key {name} the window, decoded at {last}")
            s.free("d")
            s.step(("c", toks[: last - 5], []))
            close(s.step(("c", toks[last - 5 :], [5]))[0], want[-1], dtype, f"key {name} the window, in a last portion of 6")
            s.free("c")
        assert np.abs(logits["inside"] - logits["outside"]).max() > 0.5, "the key at the window's edge does not matter enough for this test"


def case_a_sink_takes_the_mass(tmp_path, device, dtype):
    """Sinks far above every score in some heads and far below in others: the first heads' outputs all but vanish, the others' do not
    notice; left out, the logits move by far more than the tolerance."""
    cfg = config([latent(heads=4, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=11)], width=32, vocab=40, no_mlp=(0,))

    def sinks(t):
        t["l0.mix.sink"] = torch.tensor([12.0, -12.0, 3.0, 0.0])

    w = make_model(tmp_path / "sink", cfg, seed=29, edit=sinks)
    toks = tokens_for(cfg, 40, seed=8)
    want = plain.forward(cfg, w, toks)
    none = {k: v for k, v in w.items() if not k.endswith("sink")}
    assert np.abs(plain.forward(cfg, none, toks) - want).max() > 0.3
    s = Session(tmp_path / "sink", device, dtype)
    got = [s.step(("a", toks[:30], list(range(30))))] + [s.step(("a", [t], [0])) for t in toks[30:]]
    close(np.concatenate(got), want, dtype, "sink")


def case_rotation_far_back(tmp_path, device, dtype):
    """Rotations over 300 positions, whole and with the last 40 tokens decoded: scaled frequencies of neighbouring pairs over the
    latent, plain frequencies of distant pairs in the attention half; keys of every distance matter."""
    layers = {"latent": latent(heads=2, dim=8, rot_dim=16, vdim=16, kv_rank=16, scale=0.3, base=50.0, window=None, scaling=(4.0, 64, 4.0, 1.0)),
              "attention": parallel(heads=2, kv_heads=2, dim=16, vdim=16, conv=2, scale=1.5, rot_dims=16, base=50.0, right_scale=0.1)}
    for name, layer in layers.items():
        cfg = config([layer], width=32, vocab=60, no_mlp=(0,))
        w = make_model(tmp_path / name, cfg, seed=23)
        toks = tokens_for(cfg, 300, seed=6)
        want = plain.forward(cfg, w, toks)
        assert np.abs(plain.forward(cfg, w, toks[100:])[-1] - want[-1]).max() > 0.05, "far keys do not matter enough for this test"
        s = Session(tmp_path / name, device, dtype, pages=44, page_size=8)
        rounding = rounding_error(tmp_path / name, device, dtype, toks, want)
        got = [s.step(("a", toks[:260], list(range(260))))] + [s.step(("a", [t], [0])) for t in toks[260:]]
        close(np.concatenate(got), want, dtype, name, rounding)


def case_the_first_tokens(tmp_path, device, dtype):
    """Sequences of one, two and three tokens, and a first step of one token followed by portions: the convolution's zeros and the
    token shift's zero row before the start, states that start from zero, windows and pages that are not full."""
    cfg = pick("mixed_loop", dtype)
    w = make_model(tmp_path / "m", cfg, seed=27)
    s = Session(tmp_path / "m", device, dtype)
    for n in (1, 2, 3):
        toks = tokens_for(cfg, n, seed=70 + n)
        close(s.whole("a", toks), plain.forward(cfg, w, toks), dtype, f"{n} tokens")
        s.free("a")
    toks = tokens_for(cfg, 12, seed=75)
    got = np.concatenate([s.step(("b", toks[:1], [0])), s.step(("b", toks[1:3], [0, 1])), s.step(("b", toks[3:], list(range(9))))])
    close(got, plain.forward(cfg, w, toks), dtype, "one token, then portions")


def case_layer_sizes_of_a_larger_model(tmp_path, device, dtype):
    """Heads of 128 x 128 in both recurrences, attention rows of 128 and cache rows of 128 numbers (which the TMA-fed and tcgen05
    attention kernels take in bfloat16, with several tiles of queries and keys), experts of 128 x 256, a prompt of 300 tokens in two
    portions (many tokens per expert), then decoding."""
    cfg = config([parallel(heads=8, kv_heads=2, dim=128, vdim=128, conv=4, scale=0.5, rot_dims=64, base=10000.0, r_heads=2, r_dim=128, rank=16),
                  delta(heads=4, kv_heads=2, dim=128, vdim=128, conv=4, decay_rank=16, gate_rank=16),
                  latent(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=0.2, window=150)], width=256, vocab=300,
                 mlp=moe(ff=128, experts=8, top=2, groups=(4, 2)), loop=(0, 2, 2))
    cfg = steady(cfg, dtype)
    w = make_model(tmp_path / "big", cfg, seed=37)
    toks = tokens_for(cfg, 320, seed=12)
    want = plain.forward(cfg, w, toks)
    s = Session(tmp_path / "big", device, dtype, pages=48, page_size=16)
    rows = [0, 1, 15, 16, 127, 128, 129, 149, 150, 151, 199]
    got = [s.step(("a", toks[:200], rows)), s.step(("a", toks[200:300], list(range(100))))]
    got += [s.step(("a", [t], [0])) for t in toks[300:]]
    rounding = rounding_error(tmp_path / "big", device, dtype, toks, want)
    close(np.concatenate(got), np.concatenate([want[rows], want[200:]]), dtype, "larger sizes", rounding)


def case_greedy_generation_through_the_engine(tmp_path, device, dtype):
    """LLMEngine.generate (scheduler, batching, sampler) against greedy decoding with the plain model."""
    from dli_b200 import LLMEngine, SamplingParams, SchedulerConfig

    cfg = pick("mixed_loop", dtype)
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
