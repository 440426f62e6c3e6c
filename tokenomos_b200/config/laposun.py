"""Typed configuration of the Laposun decoder, read from ``config.json``.

The file gives every size and every constant that differs between models of the design:

- ``vocab``, ``width``, ``norm.eps``, ``streams`` (copies of the residual stream; absent: one,
  without connection weights), ``canon.taps`` (taps of the input convolution; absent: none),
  ``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``; absent: no bigram table);
- ``layers``: a list; each entry has ``type`` (``latent_attention``), ``mixer`` (``heads``,
  ``dim``, ``rot_dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``mask.size``, ``rot.base``,
  ``rot.dims``) and ``mlp``: null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"},
  "router": {"experts", "top", "scale"}, "shared": {"ff"} or absent}``.

``from_dict`` lists every fault it finds in one ``ConfigError``.
"""

from __future__ import annotations

from dataclasses import dataclass

from tokenomos_b200.config.lfm3 import ConfigError

MIXER_KINDS = ("latent_attention",)


@dataclass(frozen=True)
class LatentParams:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int | None
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class FeedForwardParams:
    kind: str                # "dense" or "moe"
    ff: int                  # dense: the hidden size; moe: an expert's
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    shared_ff: int = 0       # 0: no shared expert


@dataclass(frozen=True)
class LayerParams:
    mixer: LatentParams
    mlp: FeedForwardParams | None


@dataclass(frozen=True)
class BigramParams:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LaposunConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int | None      # None: a single stream without connection weights
    taps: int | None         # None: no input convolution
    bigram: BigramParams | None
    layers: tuple[LayerParams, ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict) -> "LaposunConfig":
        errors: list[str] = []

        def number(where: str, d, key: str, kind, positive: bool = True):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                errors.append(f"{where}: missing key {key!r}")
                return None
            v = d[key]
            if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and int(v) != v):
                errors.append(f"{where}.{key} must be {'an integer' if kind is int else 'a number'}, got {v!r}")
                return None
            if positive and not v > 0:
                errors.append(f"{where}.{key} = {v!r} must be positive")
                return None
            return kind(v)

        vocab = number("config", raw, "vocab", int)
        width = number("config", raw, "width", int)
        eps = number("norm", raw.get("norm"), "eps", float)
        streams = number("config", raw, "streams", int) if raw.get("streams") is not None else None
        taps = None
        if raw.get("canon") is not None:
            taps = number("canon", raw.get("canon"), "taps", int)
        bigram = None
        bg = (raw.get("embedding") or {}).get("bigram") if isinstance(raw.get("embedding"), dict) else None
        if bg is not None:
            buckets = number("embedding.bigram", bg, "buckets", int)
            mul_prev = number("embedding.bigram", bg, "mul_prev", int, positive=False)
            mul_cur = number("embedding.bigram", bg, "mul_cur", int, positive=False)
            if None not in (buckets, mul_prev, mul_cur):
                bigram = BigramParams(buckets, mul_prev, mul_cur)
        layers = []
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            errors.append("'layers' must be a non-empty list")
            entries = []
        for i, entry in enumerate(entries):
            at = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_KINDS:
                errors.append(f"{at}.type = {kind!r}: known mixers are {list(MIXER_KINDS)}")
                continue
            m = entry.get("mixer")
            if not isinstance(m, dict):
                errors.append(f"{at}: missing 'mixer'")
                continue
            w = f"{at}.mixer"
            heads, dim = number(w, m, "heads", int), number(w, m, "dim", int)
            rot_dim, vdim = number(w, m, "rot_dim", int), number(w, m, "vdim", int)
            q_rank, kv_rank = number(w, m, "q_rank", int), number(w, m, "kv_rank", int)
            scale = number(w, m, "scale", float)
            window = None
            if m.get("mask") is not None:
                window = number(f"{w}.mask", m.get("mask"), "size", int)
                if window is None:
                    continue
            base = number(f"{w}.rot", m.get("rot"), "base", float)
            dims = number(f"{w}.rot", m.get("rot"), "dims", int)
            if None not in (dims, rot_dim) and (dims % 2 or dims > rot_dim):
                errors.append(f"{w}.rot.dims = {dims}: an even number of at most rot_dim = {rot_dim}")
            mlp = None
            f = entry.get("mlp")
            if f is not None:
                fk = f.get("kind") if isinstance(f, dict) else None
                if fk == "dense":
                    ff = number(f"{at}.mlp", f, "ff", int)
                    mlp = FeedForwardParams("dense", ff) if ff is not None else None
                elif fk == "moe":
                    ff = number(f"{at}.mlp.expert", f.get("expert"), "ff", int)
                    r = f.get("router")
                    experts = number(f"{at}.mlp.router", r, "experts", int)
                    top = number(f"{at}.mlp.router", r, "top", int)
                    rscale = number(f"{at}.mlp.router", r, "scale", float)
                    shared_ff = 0
                    if f.get("shared") is not None:
                        shared_ff = number(f"{at}.mlp.shared", f.get("shared"), "ff", int)
                    if None not in (experts, top) and top > experts:
                        errors.append(f"{at}.mlp.router: top = {top} of {experts} experts")
                    if None not in (ff, experts, top, rscale, shared_ff):
                        mlp = FeedForwardParams("moe", ff, experts, top, rscale, shared_ff)
                else:
                    errors.append(f"{at}.mlp.kind = {fk!r}: 'dense', 'moe' or null")
            if None in (heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims):
                continue
            layers.append(LayerParams(LatentParams(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window,
                                                   base, dims), mlp))
        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        return cls(str(raw.get("architecture") or "Laposun"), vocab, width, eps, streams, taps, bigram,
                   tuple(layers))
