"""Typed configuration of the Lokolorn decoder, and its model as parts.

A Lokolorn layer is pre-norm, x <- x + s1 * mixer(N1(x)), x <- x + s2 * ff(N2(x)), with RMS norms whose weight is
stored as the deviation from one and a learned scale per feature (s1, s2) on each sublayer's output.  The mixer is
``parallel`` (softmax attention with short convolutions and unit-RMS queries and keys, and a decayed linear recurrence
with token shift, side by side on the same input, their outputs added with two constants), ``channel_delta`` (a delta
rule whose state decays per head and key channel) or ``latent_attention`` (attention over a cached latent with a
rotation of neighbouring pairs, YaRN-scaled frequencies, a sliding window and a learned sink per head).  The
feed-forward is a routed mixture of small gated feed-forwards (sigmoid scores, a correction that only steers the choice,
groups of experts), or absent.  A span of the layers may run several times in a row with the same weights, each pass
with a cache and state of its own and entered through a product that reads the stream and the embedding output side
by side.  config.json gives every size and constant; nothing here is fixed to one model.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .llama import UnsupportedModelError
from .pazenex import LoopConfig, _positive
from .spec import LayerSpec, ModelSpec, PartSpec, looped_run_order
from .sugonex import _keys


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: tuple[float, float, float, float] | None = None  # factor, original, fast, slow


@dataclass(frozen=True)
class ConvAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    rot: RotationConfig | None


@dataclass(frozen=True)
class ShiftRecurrenceConfig:
    heads: int
    dim: int
    decay_rank: int | None = None  # inner size of the decay's low-rank product; None: the checkpoint's tensor shapes give it


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ConvAttentionConfig
    right: ShiftRecurrenceConfig
    left_scale: float
    right_scale: float

    kind = "parallel"


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int | None = None  # inner sizes of the decay's and the gate's low-rank products; None: the checkpoint's
    gate_rank: int | None = None

    kind = "channel_delta"


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig | None
    window: int | None

    kind = "latent_attention"


@dataclass(frozen=True)
class RoutedMlpConfig:
    ff: int
    experts: int
    top: int
    scale: float
    group_count: int
    group_keep: int


@dataclass(frozen=True)
class LokolornLayerConfig:
    mixer: ParallelMixerConfig | ChannelDeltaConfig | LatentMixerConfig
    mlp: RoutedMlpConfig | None


def _rotation(m: dict | None, where: str, limit: int) -> RotationConfig | None:
    if m is None:
        return None
    _keys(m, where, ("base", "dims"), ("scaling",))
    dims = int(m["dims"])
    if dims % 2 or not 0 <= dims <= limit:
        raise UnsupportedModelError(f"{where}.dims={dims} must be even and at most {limit}")
    scaling = None
    if m.get("scaling") is not None:
        s = m["scaling"]
        _keys(s, where + ".scaling", ("factor", "original", "fast", "slow"))
        scaling = (float(s["factor"]), float(s["original"]), float(s["fast"]), float(s["slow"]))
        if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
            raise UnsupportedModelError(f"{where}.scaling: factor, original, fast and slow must be positive")
    return RotationConfig(float(m["base"]), dims, scaling)


def _parse_parallel(m: dict, where: str) -> ParallelMixerConfig:
    _keys(m, where, ("left", "right", "left_scale", "right_scale"))
    l, r = m["left"], m["right"]
    _keys(l, where + ".left", ("heads", "kv_heads", "dim", "vdim", "conv", "scale"), ("rot",))
    _keys(r, where + ".right", ("heads", "dim"), ("decay_rank",))
    heads, kv, dim, vdim, conv = (_positive(l[k], f"{where}.left.{k}") for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
    if heads % kv:
        raise UnsupportedModelError(f"{where}.left.heads={heads} is not a multiple of kv_heads={kv}")
    left = ConvAttentionConfig(heads, kv, dim, vdim, conv, float(l["scale"]), _rotation(l.get("rot"), where + ".left.rot", dim))
    right = ShiftRecurrenceConfig(_positive(r["heads"], where + ".right.heads"), _positive(r["dim"], where + ".right.dim"),
                                  None if r.get("decay_rank") is None else _positive(r["decay_rank"], where + ".right.decay_rank"))
    return ParallelMixerConfig(left, right, float(m["left_scale"]), float(m["right_scale"]))


def _parse_channel_delta(m: dict, where: str) -> ChannelDeltaConfig:
    _keys(m, where, ("heads", "kv_heads", "dim", "vdim", "conv"), ("decay_rank", "gate_rank"))
    out = ChannelDeltaConfig(*(_positive(m[k], f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim", "conv")),
                             *(None if m.get(k) is None else _positive(m[k], f"{where}.{k}") for k in ("decay_rank", "gate_rank")))
    if out.heads % out.kv_heads:
        raise UnsupportedModelError(f"{where}.heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
    return out


def _parse_latent(m: dict, where: str) -> LatentMixerConfig:
    _keys(m, where, ("heads", "dim", "vdim", "kv_rank", "scale"), ("rot_dim", "rot", "mask"))
    rot_dim = int(m.get("rot_dim") or 0)
    rot = None
    if rot_dim:
        if rot_dim < 0 or rot_dim % 2 or m.get("rot") is None:
            raise UnsupportedModelError(f"{where}.rot_dim={rot_dim} must be even and needs a rot object")
        rot = _rotation(m["rot"], where + ".rot", rot_dim)
    window = None
    if m.get("mask") is not None:
        _keys(m["mask"], where + ".mask", ("size",))
        window = _positive(m["mask"]["size"], where + ".mask.size")
    return LatentMixerConfig(_positive(m["heads"], where + ".heads"), _positive(m["dim"], where + ".dim"), rot_dim,
                             _positive(m["vdim"], where + ".vdim"), _positive(m["kv_rank"], where + ".kv_rank"), float(m["scale"]), rot, window)


def _parse_mlp(m: dict, where: str) -> RoutedMlpConfig:
    _keys(m, where, ("kind", "expert", "router"))
    if m["kind"] != "moe":
        raise UnsupportedModelError(f"{where}.kind={m['kind']!r} (known: moe)")
    _keys(m["expert"], where + ".expert", ("ff",))
    r = m["router"]
    _keys(r, where + ".router", ("experts", "top", "scale"), ("groups",))
    experts, top = _positive(r["experts"], where + ".router.experts"), _positive(r["top"], where + ".router.top")
    count, keep = 1, 1
    if r.get("groups") is not None:
        _keys(r["groups"], where + ".router.groups", ("count", "keep"))
        count, keep = _positive(r["groups"]["count"], where + ".router.groups.count"), _positive(r["groups"]["keep"], where + ".router.groups.keep")
    if experts % count or keep > count or top > keep * (experts // count):
        raise UnsupportedModelError(f"{where}.router: {experts} experts in {count} groups, {keep} kept, cannot yield {top} choices")
    return RoutedMlpConfig(_positive(m["expert"]["ff"], where + ".expert.ff"), experts, top, float(r["scale"]), count, keep)


_MIXERS = {"parallel": "_parse_parallel", "channel_delta": "_parse_channel_delta", "latent_attention": "_parse_latent"}  # looked up by name at every call


@dataclass(frozen=True)
class LokolornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[LokolornLayerConfig, ...]
    loop: LoopConfig | None

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "LokolornConfig":
        _keys(cfg, "config", ("architecture", "layers", "norm", "vocab", "width"), ("loop",))
        _keys(cfg["norm"], "norm", ("eps",))
        if not isinstance(cfg["layers"], list) or not cfg["layers"]:
            raise UnsupportedModelError("layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(cfg["layers"]):
            where = f"layers[{i}]"
            _keys(entry, where, ("type", "mixer"), ("mlp",))
            if entry["type"] not in _MIXERS:
                raise UnsupportedModelError(f"{where}.type={entry['type']!r} (known: {', '.join(_MIXERS)})")
            mixer = globals()[_MIXERS[entry["type"]]](entry["mixer"], where + ".mixer")
            layers.append(LokolornLayerConfig(mixer, None if entry.get("mlp") is None else _parse_mlp(entry["mlp"], where + ".mlp")))
        loop = None
        if cfg.get("loop") is not None:
            _keys(cfg["loop"], "loop", ("start", "stop", "times"))
            loop = LoopConfig(int(cfg["loop"]["start"]), int(cfg["loop"]["stop"]), int(cfg["loop"]["times"]))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise UnsupportedModelError(f"loop {cfg['loop']} does not name a span of the {len(layers)} layers run at least once")
        return cls(_positive(cfg["vocab"], "vocab"), _positive(cfg["width"], "width"), float(cfg["norm"]["eps"]), tuple(layers), loop)


def lokolorn_run_order(cfg: LokolornConfig):
    loop = cfg.loop
    return looped_run_order(len(cfg.layers), None if loop is None else (loop.start, loop.stop, loop.times))


def _scaling_dict(rot: RotationConfig | None):
    if rot is None or rot.scaling is None:
        return None
    return dict(zip(("factor", "original", "fast", "slow"), rot.scaling))


def lokolorn_model_spec(cfg: LokolornConfig) -> ModelSpec:
    """Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``; layer i's tensors start with ``l<i>.``: ``norm1``, ``norm2``,
    ``ls1``, ``ls2``, ``mix.*`` (``mix.left.*`` and ``mix.right.*`` in a parallel layer), ``mlp.router``, ``mlp.correction``, ``mlp.e<j>.*``."""
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "tensor": name, "offset": 1.0})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, ParallelMixerConfig):
            lp, rp = p + "mix.left.", p + "mix.right."
            a = m.left
            left = PartSpec("conv_attention", {
                "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim, "conv_taps": a.conv,
                "scale": a.scale, "bias": True, "qk_unit_eps": cfg.eps, "rotary_dim": a.rot.dims if a.rot else 0, "theta": a.rot.base if a.rot else 1.0,
                "tensors": {"q": lp + "q", "k": lp + "k", "v": lp + "v", "o": lp + "o", "q_bias": lp + "q.b", "k_bias": lp + "k.b", "v_bias": lp + "v.b",
                            "o_bias": lp + "o.b", "q_conv": lp + "q.conv", "k_conv": lp + "k.conv", "v_conv": lp + "v.conv"}}, lp)
            names = {role: rp + role for role in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
            names.update({"mu_" + s: rp + "mu." + s for s in "rkvgw"})
            right = PartSpec("shift_decay_recurrence", {"hidden_size": W, "num_heads": m.right.heads, "head_dim": m.right.dim, "eps": cfg.eps,
                                                        "decay_rank": m.right.decay_rank, "tensors": names}, rp)
            mixer = PartSpec("weighted_pair", {"first": left, "second": right, "first_scale": m.left_scale, "second_scale": m.right_scale}, p + "mix.")
        elif isinstance(m, ChannelDeltaConfig):
            names = {role: p + "mix." + role for role in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o", "A_log", "dt_bias", "norm")}
            names.update({"q_conv": p + "mix.q.conv", "k_conv": p + "mix.k.conv", "v_conv": p + "mix.v.conv"})
            mixer = PartSpec("channel_delta", {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                                               "conv_taps": m.conv, "eps": cfg.eps, "unit_eps": 1e-6, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank,
                                               "tensors": names}, p + "mix.")
        else:
            names = {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv", "o": p + "mix.o",
                     "sink": p + "mix.sink"}
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "window": m.window, "gate": False, "eps": cfg.eps, "rotary_dim": m.rot.dims if m.rot else 0,
                "theta": m.rot.base if m.rot else 1.0, "rotary_pairing": "neighbours", "rotary_scaling": _scaling_dict(m.rot), "head_sinks": True,
                "tensors": names}, p + "mix.")
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer}
        params = {"mixer_scale": p + "ls1", "size": W}
        if layer.mlp is not None:
            f = layer.mlp
            parts["ffn_norm"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("routed_glu", {
                "hidden_size": W, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top, "route_scale": f.scale,
                "group_count": f.group_count, "group_keep": f.group_keep, "activation": "silu", "score": "sigmoid",
                "tensors": {"router": p + "mlp.router", "correction": p + "mlp.correction", "gate": p + "mlp.e{}.gate", "up": p + "mlp.e{}.up",
                            "down": p + "mlp.e{}.down"}}, p + "mlp.")
            params["ffn_scale"] = p + "ls2"
        layers.append(LayerSpec("prenorm_scaled", parts, params))
    entries = ()
    if cfg.loop is not None:
        entries = tuple(PartSpec("concat_project", {"size": W, "vocab_size": cfg.vocab, "table": "embed", "tensor": "loop.in"}) for _ in range(cfg.loop.times))
    return ModelSpec(
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "tensor": "embed"}),
        layers=tuple(layers),
        run_order=lokolorn_run_order(cfg),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tensor": "head"}),
        entries=entries,
    )
