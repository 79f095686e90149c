"""Typed configuration of the Pokadra decoder, and its model as parts.

A Pokadra layer reads the residual stream itself and norms only what its sublayers return: x <- x + m * norm(mixer(x)), then
x <- x + m * norm(ff(x)) (an RMS norm in groups; the feed-forward may be absent), then a small input from the token itself,
and at the end the stream becomes a learned mixture of the embedding output and of all layers' results so far.  The mixer
is differential attention (two softmax maps per head over shared values, with q/k norm, a paired rotation with YaRN
scaling, a sliding window that keeps the first tokens, a per-head norm and gate; a layer may read an earlier layer's keys
and values) or a minGRU recurrence.  The embedding adds a row of a second table chosen by a hash of the token and the one
in front of it.  config.json gives every size and constant; nothing here is fixed to one model.
"""

from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any

from .llama import UnsupportedModelError
from .pazenex import _positive
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep


def _keys(d: dict, where: str, required: tuple[str, ...], optional: tuple[str, ...] = ()) -> None:
    """Required keys must be there; a key this parser does not know is reported and ignored."""
    if not isinstance(d, dict):
        raise UnsupportedModelError(f"{where} must be an object")
    for k in required:
        if k not in d:
            raise KeyError(f"{where}.{k}")
    for k in d:
        if k not in required and k not in optional:
            warnings.warn(f"{where}.{k} is not a key of this architecture and is ignored", stacklevel=3)


@dataclass(frozen=True)
class YarnConfig:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int  # per-head, per-map size of queries and keys
    vdim: int
    scale: float
    diff: float
    rot_base: float
    rot_dims: int
    yarn: YarnConfig | None
    window: int | None
    keep_first: int
    kv_from: int | None  # the layer whose keys and values this one reads (None: its own)

    kind = "attention"


@dataclass(frozen=True)
class MinGRUConfig:
    width: int

    kind = "mingru"


@dataclass(frozen=True)
class ClippedGLUConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class PokadraLayerConfig:
    mixer: DiffAttentionConfig | MinGRUConfig
    mlp: ClippedGLUConfig | None


@dataclass(frozen=True)
class PairTableConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class PokadraConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    residual_mult: float
    embedding_scale: float
    pair_table: PairTableConfig | None
    token_side_dim: int | None
    layers: tuple[PokadraLayerConfig, ...]

    @classmethod
    def from_dict(cls, cfg: dict[str, Any]) -> "PokadraConfig":
        _keys(cfg, "config", ("architecture", "layers", "norm", "vocab", "width"), ("embedding", "residual_mult", "token_side"))
        _keys(cfg["norm"], "norm", ("eps",), ("groups",))
        width = _positive(cfg["width"], "width")
        groups = _positive(cfg["norm"].get("groups", 1), "norm.groups")
        if width % groups:
            raise UnsupportedModelError(f"width={width} is not a multiple of norm.groups={groups}")
        emb = cfg.get("embedding") or {}
        _keys(emb, "embedding", (), ("scale", "bigram"))
        pair = None
        if emb.get("bigram") is not None:
            _keys(emb["bigram"], "embedding.bigram", ("buckets", "mul_prev", "mul_cur"))
            b = emb["bigram"]
            pair = PairTableConfig(_positive(b["buckets"], "embedding.bigram.buckets"), int(b["mul_prev"]), int(b["mul_cur"]))
            if pair.mul_prev < 0 or pair.mul_cur < 0:
                raise UnsupportedModelError("embedding.bigram: the multipliers must not be negative")
        side = None
        if cfg.get("token_side") is not None:
            _keys(cfg["token_side"], "token_side", ("dim",))
            side = _positive(cfg["token_side"]["dim"], "token_side.dim")
        if not isinstance(cfg["layers"], list) or not cfg["layers"]:
            raise UnsupportedModelError("layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(cfg["layers"]):
            where = f"layers[{i}]"
            _keys(entry, where, ("type", "mixer"), ("mlp",))
            if entry["type"] == "attention":
                mixer = _parse_attention(entry["mixer"], where + ".mixer")
            elif entry["type"] == "mingru":
                _keys(entry["mixer"], where + ".mixer", ("width",))
                mixer = MinGRUConfig(_positive(entry["mixer"]["width"], where + ".mixer.width"))
            else:
                raise UnsupportedModelError(f"{where}.type={entry['type']!r} (known: attention, mingru)")
            mlp = None
            if entry.get("mlp") is not None:
                _keys(entry["mlp"], where + ".mlp", ("kind", "ff", "limit"))
                if entry["mlp"]["kind"] != "dense":
                    raise UnsupportedModelError(f"{where}.mlp.kind={entry['mlp']['kind']!r} (known: dense)")
                limit = float(entry["mlp"]["limit"])
                if not limit > 0:
                    raise UnsupportedModelError(f"{where}.mlp.limit={limit} must be positive")
                mlp = ClippedGLUConfig(_positive(entry["mlp"]["ff"], where + ".mlp.ff"), limit)
            layers.append(PokadraLayerConfig(mixer, mlp))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, DiffAttentionConfig) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if 0 <= m.kv_from < i else None
                if not isinstance(src, DiffAttentionConfig) or src.kv_from is not None:
                    raise UnsupportedModelError(f"layers[{i}].mixer.kv_from={m.kv_from} must name an earlier attention layer with keys and values of its own")
                if (src.heads, src.kv_heads, src.dim, src.vdim, src.rot_base, src.rot_dims, src.yarn) != \
                        (m.heads, m.kv_heads, m.dim, m.vdim, m.rot_base, m.rot_dims, m.yarn):
                    raise UnsupportedModelError(f"layers[{i}].mixer reads layer {m.kv_from}'s keys and values, but its heads, sizes or rotation differ")
        return cls(_positive(cfg["vocab"], "vocab"), width, float(cfg["norm"]["eps"]), groups, float(cfg.get("residual_mult", 1.0)),
                   float(emb.get("scale", 1.0)), pair, side, tuple(layers))


def _parse_attention(m: dict, where: str) -> DiffAttentionConfig:
    _keys(m, where, ("heads", "kv_heads", "dim", "vdim", "scale", "diff"), ("rot", "mask", "kv_from"))
    heads, kv_heads = _positive(m["heads"], where + ".heads"), _positive(m["kv_heads"], where + ".kv_heads")
    dim, vdim = _positive(m["dim"], where + ".dim"), _positive(m["vdim"], where + ".vdim")
    if heads % kv_heads:
        raise UnsupportedModelError(f"{where}.heads={heads} is not a multiple of kv_heads={kv_heads}")
    base, dims, yarn = 10000.0, 0, None
    if m.get("rot") is not None:
        _keys(m["rot"], where + ".rot", ("base", "dims"), ("scaling",))
        base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
        if dims % 2 or not 0 <= dims <= dim:
            raise UnsupportedModelError(f"{where}.rot.dims={dims} must be even and at most dim={dim}")
        if m["rot"].get("scaling") is not None:
            _keys(m["rot"]["scaling"], where + ".rot.scaling", ("factor", "original", "fast", "slow"))
            sc = m["rot"]["scaling"]
            yarn = YarnConfig(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
    window, keep = None, 0
    if m.get("mask") is not None:
        _keys(m["mask"], where + ".mask", ("size",), ("keep_first",))
        window = _positive(m["mask"]["size"], where + ".mask.size")
        keep = int(m["mask"].get("keep_first") or 0)
        if keep < 0:
            raise UnsupportedModelError(f"{where}.mask.keep_first={keep} must not be negative")
    kv_from = m.get("kv_from")
    return DiffAttentionConfig(heads, kv_heads, dim, vdim, float(m["scale"]), float(m["diff"]), base, dims, yarn, window, keep,
                               None if kv_from is None else int(kv_from))


def pokadra_run_order(cfg: PokadraConfig) -> tuple[RunStep, ...]:
    """Every layer once; a layer that reads another layer's keys and values reads that run step's cache."""
    return tuple(RunStep(i, cache_of=layer.mixer.kv_from if isinstance(layer.mixer, DiffAttentionConfig) else None)
                 for i, layer in enumerate(cfg.layers))


def pokadra_model_spec(cfg: PokadraConfig) -> ModelSpec:
    """Tensor names: ``embed``, ``bigram``, ``side.embed``, ``final.norm``, ``head``; layer i's tensors start with ``l<i>.``:
    ``norm1`` (behind the mixer), ``norm2`` (behind the feed-forward), ``mix.*``, ``mlp.*``, ``side.gate``, ``side.proj``,
    ``side.norm``, ``dwa``."""
    W, L = cfg.width, len(cfg.layers)

    def out_norm(name: str, groups: int) -> PartSpec:
        return PartSpec("group_rmsnorm", {"size": W, "eps": cfg.eps, "groups": groups, "mult": cfg.residual_mult, "tensor": name})

    # what the cache of a layer with keys and values has to keep: the widest mask among the layers that read it
    retain: dict[int, tuple[int | None, int]] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, DiffAttentionConfig):
            owner = i if m.kv_from is None else m.kv_from
            window, first = retain.get(owner, (m.window, m.keep_first))
            window = None if window is None or m.window is None else max(window, m.window)
            retain[owner] = (window, max(first, m.keep_first))

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, DiffAttentionConfig):
            owner = i if m.kv_from is None else m.kv_from
            names = {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "g": p + "mix.g", "o": p + "mix.o", "q_norm": p + "mix.q.norm",
                     "k_norm": p + "mix.k.norm", "lq1": p + "mix.lq1", "lk1": p + "mix.lk1", "lq2": p + "mix.lq2", "lk2": p + "mix.lk2"}
            yarn = None if m.yarn is None else {"factor": m.yarn.factor, "original": m.yarn.original, "fast": m.yarn.fast, "slow": m.yarn.slow}
            mixer = PartSpec("diff_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
                "window": m.window, "keep_first": m.keep_first, "diff": m.diff, "eps": cfg.eps, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                "rotary_scaling": yarn, "own_kv": m.kv_from is None, "retain_window": retain[owner][0], "retain_first": retain[owner][1],
                "tensors": names}, p + "mix.")
        else:
            mixer = PartSpec("mingru", {"hidden_size": W, "width": m.width,
                                        "tensors": {"z": p + "mix.z", "z_bias": p + "mix.z.b", "x": p + "mix.x", "x_bias": p + "mix.x.b",
                                                    "g": p + "mix.g", "o": p + "mix.o"}}, p + "mix.")
        parts = {"mixer": mixer, "mixer_post_norm": out_norm(p + "norm1", cfg.norm_groups)}
        if layer.mlp is not None:
            parts["ffn"] = PartSpec("glu", {"hidden_size": W, "intermediate_size": layer.mlp.ff, "activation": "quick_gelu",
                                            "limit": layer.mlp.limit, "up_shift": 1.0,
                                            "tensors": {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"}}, p + "mlp.")
            parts["ffn_post_norm"] = out_norm(p + "norm2", cfg.norm_groups)
        after = []
        if cfg.token_side_dim is not None:
            after.append(PartSpec("token_gated_input", {
                "hidden_size": W, "vocab_size": cfg.vocab, "dim": cfg.token_side_dim, "col0": i * cfg.token_side_dim,
                "table_cols": L * cfg.token_side_dim, "norm": out_norm(p + "side.norm", 1),
                "tensors": {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj"}}, p + "side."))
        after.append(PartSpec("depth_average", {"size": W, "index": i, "layers": L, "tensor": p + "dwa"}))
        for j, part in enumerate(after):
            parts[f"after_{j + 1}"] = part
        layers.append(LayerSpec("outnorm", parts))
    pair = None
    if cfg.pair_table is not None:
        pair = {"tensor": "bigram", "buckets": cfg.pair_table.buckets, "mul_prev": cfg.pair_table.mul_prev, "mul_cur": cfg.pair_table.mul_cur}
    return ModelSpec(
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("pair_hash_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "tensor": "embed", "scale": cfg.embedding_scale,
                                                   "pair": pair}),
        layers=tuple(layers),
        run_order=pokadra_run_order(cfg),
        final_norm=PartSpec("group_rmsnorm", {"size": W, "eps": cfg.eps, "groups": cfg.norm_groups, "tensor": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": None, "tensor": "head"}),
    )
