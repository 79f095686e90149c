"""Arrangements: how a layer's norms, mixer and feed-forward sit around the residual."""

from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import BuildEnv, Part, PendingNormed, PendingScaled, PendingSum, ResidualStream, build_part, can_fuse, normed_input, register_part


@register_part("arrangement", "prenorm")
class PreNormBlock(Part):
    """x = x + mixer(norm(x)); x = x + ffn(norm(x)) (src/dli/model/llama.py:211-212).
    Roles: mixer_norm, mixer, ffn_norm, ffn.  The feed-forward's output stays pending on the
    stream; the next norm adds it."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
        self.ffn = build_part("feed_forward", spec.parts["ffn"], env)

        if hasattr(self.mixer, "defer_output"):
            self.mixer.defer_output = can_fuse(self.ffn_norm, self.ffn)

    def children(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_need(self):
        """What this layer's run step keeps between steps: whatever its one mixer needs."""
        return self.mixer.cache_need()

    def first_consumer(self):
        """The norm that takes the stream's pending delta, and the part that reads its output."""
        return self.mixer_norm, self.mixer

    def defer_last_product(self, flag: bool) -> None:
        """Whether whoever runs after this layer can take the feed-forward's last product uncomputed."""
        if hasattr(self.ffn, "defer_output"):
            self.ffn.defer_output = bool(flag)

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        y = normed_input(self.mixer_norm, stream.h, stream.take_pending(), self.mixer)
        a = self.mixer.forward(y, batch, cache)
        y = normed_input(self.ffn_norm, stream.h, a, self.ffn)
        stream.pending = self.ffn.forward(y)


@register_part("arrangement", "prenorm_scaled")
class ScaledPreNormBlock(Part):
    """x <- x + s1 * mixer(norm(x)); x <- x + s2 * ffn(norm(x)): pre-norm with a learned float32 scale per feature on each
    sublayer's output (s1, s2: tensors of the arrangement itself, named by the layer's ``mixer_scale`` and ``ffn_scale``).
    Roles: mixer_norm, mixer, and — a layer may have no feed-forward — ffn_norm, ffn.  A sublayer's output stays pending
    with its scale (``PendingScaled``), so the next norm multiplies, adds and norms in one kernel; a mixer may return a
    ``WeightedPair`` (two mixers side by side), whose sum is formed in that kernel as well."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.size = int(spec.params["size"])
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.has_ffn = "ffn" in spec.parts
        if self.has_ffn:
            self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
            self.ffn = build_part("feed_forward", spec.parts["ffn"], env)
        self.names = [spec.params["mixer_scale"]] + ([spec.params["ffn_scale"]] if self.has_ffn else [])
        self.scales: list[torch.Tensor] = []

    def children(self):
        return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.has_ffn else [])

    def declare(self):
        return {name: TensorDecl((self.size,), "vector32") for name in self.names}

    def load(self, tensors):
        self.scales = [tensors[name] for name in self.names]

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        y = normed_input(self.mixer_norm, stream.h, stream.take_pending(), self.mixer)
        pending = PendingScaled(self.mixer.forward(y, batch, cache), self.scales[0])
        if self.has_ffn:
            y = normed_input(self.ffn_norm, stream.h, pending, self.ffn)
            pending = PendingScaled(self.ffn.forward(y), self.scales[1])
        stream.pending = pending


@register_part("arrangement", "sandwich")
class SandwichBlock(Part):
    """x = x + post_a(mixer(pre_a(x))); x = x + post_f(ffn(pre_f(x))): every sublayer between two norms, the second
    one on its output before the residual addition.  Roles: mixer_norm, mixer, mixer_post_norm, and — a layer
    may have no feed-forward — ffn_norm, ffn, ffn_post_norm.  A sublayer's output stays pending with its norm
    (``PendingNormed``), so the norm in front of the next sublayer norms it, adds it and norms the sum in one
    kernel."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.mixer_post_norm = build_part("norm", spec.parts["mixer_post_norm"], env)
        self.has_ffn = "ffn" in spec.parts
        if self.has_ffn:
            self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
            self.ffn = build_part("feed_forward", spec.parts["ffn"], env)
            self.ffn_post_norm = build_part("norm", spec.parts["ffn_post_norm"], env)
        for norm in (self.mixer_post_norm, *([self.ffn_post_norm] if self.has_ffn else [])):
            if not hasattr(norm, "add_into"):
                raise ValueError("sandwich: the norm behind a sublayer must offer add_into(h, a)")

    def children(self):
        out = [self.mixer_norm, self.mixer, self.mixer_post_norm]
        return out + ([self.ffn_norm, self.ffn, self.ffn_post_norm] if self.has_ffn else [])

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        y = normed_input(self.mixer_norm, stream.h, stream.take_pending(), self.mixer)
        pending = PendingNormed(self.mixer.forward(y, batch, cache), self.mixer_post_norm)
        if self.has_ffn:
            y = normed_input(self.ffn_norm, stream.h, pending, self.ffn)
            pending = PendingNormed(self.ffn.forward(y), self.ffn_post_norm)
        stream.pending = pending


@register_part("arrangement", "parallel")
class ParallelBlock(Part):
    """x = x + (mixer(norm_a(x)) + ffn(norm_f(x))): both branches read the same x, each behind a norm of its own, and
    their outputs are added to the stream together.  Roles: mixer_norm, mixer, and — a layer may have no
    feed-forward — ffn_norm, ffn.  The two outputs stay pending on the stream as a ``PendingSum``; the norm in front
    of the next layer's branches adds them, and where both norms divide by the same root mean square
    (``add_norm_pair``) one kernel adds the pending outputs and writes both branches' inputs."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.mixer_norm = build_part("norm", spec.parts["mixer_norm"], env)
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.has_ffn = "ffn" in spec.parts
        if self.has_ffn:
            self.ffn_norm = build_part("norm", spec.parts["ffn_norm"], env)
            self.ffn = build_part("feed_forward", spec.parts["ffn"], env)

    def children(self):
        return [self.mixer_norm, self.mixer] + ([self.ffn_norm, self.ffn] if self.has_ffn else [])

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        pair = getattr(self.mixer_norm, "add_norm_pair", None) if self.has_ffn else None
        if pair is not None and not isinstance(stream.take_pending(), (PendingSum, torch.Tensor, type(None))):
            stream.settle()
        ys = pair(stream.h, stream.take_pending(), self.ffn_norm) if pair is not None else None
        if ys is not None:
            stream.pending = None
            ya, yf = ys
        else:
            ya = normed_input(self.mixer_norm, stream.h, stream.take_pending(), self.mixer)
            stream.pending = None  # the norm has added it; the second norm reads the same sum
            yf = normed_input(self.ffn_norm, stream.h, None, self.ffn) if self.has_ffn else None
        a = self.mixer.forward(ya, batch, cache)
        stream.pending = PendingSum(a, self.ffn.forward(yf) if self.has_ffn else None)


@register_part("arrangement", "outnorm")
class OutNormBlock(Part):
    """x <- x + post_a(mixer(x)); x <- x + post_f(ffn(x)): the sublayers read the stream itself, and only their OUTPUT is normed
    (by a norm with ``add_scaled_into``, which also carries the factor of the addition).  Roles: mixer, mixer_post_norm, and —
    a layer may have no feed-forward — ffn, ffn_post_norm; then, optionally, ``after_1`` and ``after_2``: stream_entry parts
    that act on the stream behind the sublayers, in that order (a part with ``begin(stream, batch)`` is also told when the
    layer starts).  In a 16-bit dtype the kernel that adds to the float32 stream also writes it in that dtype, which is what
    the next product reads; nothing else is rounded."""

    graph_capturable = True

    def __init__(self, spec, env: BuildEnv) -> None:
        self.spec, self.env = spec, env
        self.mixer = build_part("mixer", spec.parts["mixer"], env)
        self.mixer_post_norm = build_part("norm", spec.parts["mixer_post_norm"], env)
        self.has_ffn = "ffn" in spec.parts
        if self.has_ffn:
            self.ffn = build_part("feed_forward", spec.parts["ffn"], env)
            self.ffn_post_norm = build_part("norm", spec.parts["ffn_post_norm"], env)
        self.after = [build_part("stream_entry", spec.parts[role], env) for role in ("after_1", "after_2") if role in spec.parts]
        for norm in (self.mixer_post_norm, *([self.ffn_post_norm] if self.has_ffn else [])):
            if not hasattr(norm, "add_scaled_into"):
                raise ValueError("outnorm: the norm behind a sublayer must offer add_scaled_into(h, a, want_cast)")

    def children(self):
        return [self.mixer, self.mixer_post_norm] + ([self.ffn, self.ffn_post_norm] if self.has_ffn else []) + self.after

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, stream: ResidualStream, batch, cache) -> None:
        for part in self.after:
            begin = getattr(part, "begin", None)
            if begin is not None:
                begin(stream, batch)
        h = stream.settle()
        dtype = self.env.dtype
        a = self.mixer.forward(stream.activation(dtype), batch, cache)
        stream.cast = self.mixer_post_norm.add_scaled_into(h, a, want_cast=self.has_ffn or bool(self.after))
        if self.has_ffn:
            f = self.ffn.forward(stream.activation(dtype))
            stream.cast = self.ffn_post_norm.add_scaled_into(h, f, want_cast=bool(self.after))
        for i, part in enumerate(self.after):
            part.apply(stream, batch, want_cast=True)
