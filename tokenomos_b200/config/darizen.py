"""Typed configuration of the Darizen decoder, read from ``config.json``.

The file gives every size and every constant that differs between models of the design:

- ``vocab``, ``width``, ``norm.eps``;
- ``layers``: a list; each entry has ``type`` (``attention`` or ``attention_2``), ``mixer``
  (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, for ``attention_2`` also
  ``mask.keep_first``, ``rot.base``, ``rot.dims`` and ``rot.scaling``: ``factor, original, fast,
  slow`` for ``attention``, ``factor`` for ``attention_2``) and ``mlp`` (null, or ``kind``
  ``dense`` with ``ff`` and ``limit``);
- ``loop`` (optional): ``start``, ``stop``, ``times``: the layers ``start .. stop-1`` run ``times``
  times in a row with the same weights.

``from_dict`` lists every fault it finds in one ``ConfigError``.
"""

from __future__ import annotations

from dataclasses import dataclass

from tokenomos_b200.config.lfm3 import ConfigError

MIXER_KINDS = ("attention", "attention_2")


@dataclass(frozen=True)
class RotaryParams:
    base: float
    dims: int
    # None, {"kind": "yarn", factor, original, fast, slow} or {"kind": "linear", factor}
    scaling: dict | None


@dataclass(frozen=True)
class MixerParams:
    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot: RotaryParams


@dataclass(frozen=True)
class MlpParams:
    kind: str
    ff: int
    limit: float


@dataclass(frozen=True)
class LayerParams:
    mixer: MixerParams
    mlp: MlpParams | None


@dataclass(frozen=True)
class LoopParams:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class DarizenConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[LayerParams, ...]
    loop: LoopParams | None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict) -> "DarizenConfig":
        errors: list[str] = []

        def number(where: str, d, key: str, kind, positive: bool = True, default=None):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                if default is not None:
                    return default
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
            heads = number(f"{at}.mixer", m, "heads", int)
            kv_heads = number(f"{at}.mixer", m, "kv_heads", int)
            dim = number(f"{at}.mixer", m, "dim", int)
            vdim = number(f"{at}.mixer", m, "vdim", int)
            scale = number(f"{at}.mixer", m, "scale", float)
            mask = m.get("mask")
            window = number(f"{at}.mixer.mask", mask, "size", int)
            keep = 0
            if kind == "attention_2" and isinstance(mask, dict) and mask.get("keep_first") is not None:
                keep = number(f"{at}.mixer.mask", mask, "keep_first", int, positive=False)
                if keep is not None and keep < 0:
                    errors.append(f"{at}.mixer.mask.keep_first = {keep} must not be negative")
            rot = m.get("rot")
            base = number(f"{at}.mixer.rot", rot, "base", float)
            dims = number(f"{at}.mixer.rot", rot, "dims", int)
            scaling = None
            sc = rot.get("scaling") if isinstance(rot, dict) else None
            if sc is not None:
                factor = number(f"{at}.mixer.rot.scaling", sc, "factor", float)
                if kind == "attention":
                    scaling = {"kind": "yarn", "factor": factor,
                               "original": number(f"{at}.mixer.rot.scaling", sc, "original", float),
                               "fast": number(f"{at}.mixer.rot.scaling", sc, "fast", float),
                               "slow": number(f"{at}.mixer.rot.scaling", sc, "slow", float)}
                else:
                    scaling = {"kind": "linear", "factor": factor}
            if None not in (heads, kv_heads) and heads % kv_heads:
                errors.append(f"{at}.mixer: {heads} heads over {kv_heads} kv_heads")
            if None not in (dims, dim) and (dims % 2 or dims > dim):
                errors.append(f"{at}.mixer.rot.dims = {dims}: an even number of at most dim = {dim}")
            if kind == "attention" and None not in (dim, vdim) and dim != vdim:
                errors.append(f"{at}.mixer: the values of 'attention' are its keys, so vdim = dim; got {vdim}, {dim}")
            if base is not None and base == 1.0:
                errors.append(f"{at}.mixer.rot.base must not be 1")
            mlp = None
            f = entry.get("mlp")
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "dense":
                    errors.append(f"{at}.mlp.kind = {f.get('kind') if isinstance(f, dict) else f!r}: 'dense' or null")
                else:
                    ff = number(f"{at}.mlp", f, "ff", int)
                    limit = number(f"{at}.mlp", f, "limit", float)
                    if None not in (ff, limit):
                        mlp = MlpParams("dense", ff, limit)
            if None in (heads, kv_heads, dim, vdim, scale, window, keep, base, dims) or (
                    scaling is not None and None in scaling.values()):
                continue
            layers.append(LayerParams(MixerParams(kind, heads, kv_heads, dim, vdim, scale, window, keep,
                                                  RotaryParams(base, dims, scaling)), mlp))
        loop = None
        lp = raw.get("loop")
        if lp is not None:
            start = number("loop", lp, "start", int, positive=False)
            stop = number("loop", lp, "stop", int)
            times = number("loop", lp, "times", int)
            if None not in (start, stop, times):
                if not 0 <= start < stop <= len(entries):
                    errors.append(f"loop: layers {start} .. {stop - 1} of {len(entries)}")
                else:
                    loop = LoopParams(start, stop, times)
        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        return cls(str(raw.get("architecture") or "Darizen"), vocab, width, eps, tuple(layers), loop)
