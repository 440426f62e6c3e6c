"""A plain, slow Darizen in PyTorch on the CPU: the oracle of the Darizen tests.

One function per mechanism, whole sequences only (no cache, no batching), any float type
(float64 by default). It shares no code with ``tokenomos_b200``: the configuration is read
from the raw dictionary, weights come as a name -> tensor dictionary.

Notation. ``x`` [T, width] is the residual stream of one sequence, positions ``0 .. T-1``.
A layer is ``x += mixer(norm1(x)); x += ff(norm2(x))`` with ``norm(x) = x / sqrt(mean(x^2) +
eps) * (1 + w)``. The layers ``loop.start .. loop.stop-1`` run ``loop.times`` times with the
same weights; pass ``t`` first adds the embedding output (``t > 0`` only) and row ``t`` of
``loop.step``.
"""

from __future__ import annotations

import math

import torch


def unit_offset_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1 + w.to(x.dtype))


def rotary_table(kind: str, rot: dict, dtype=torch.float64) -> tuple[torch.Tensor, float]:
    """(frequency of each of ``dims / 2`` pairs, the factor cos and sin are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    scaling = rot.get("scaling")
    freqs, mult = [], 1.0
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling and kind == "attention":
            factor, original = float(scaling["factor"]), float(scaling["original"])

            def turn(t):
                return dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(base))

            lo = max(math.floor(turn(float(scaling["fast"]))), 0)
            hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / factor * ramp + f * (1 - ramp)
            mult = 0.1 * math.log(factor) + 1.0
        elif scaling and kind == "attention_2":
            f = f / float(scaling["factor"])
        freqs.append(f)
    return torch.tensor(freqs, dtype=dtype), mult


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, mult: float,
           interleaved: bool) -> torch.Tensor:
    """``x`` [T, heads, dim]: the first ``2 * len(freqs)`` columns of every head are rotated,
    pair (2i, 2i+1) when ``interleaved`` else pair (i, i + dims/2); the rest pass."""
    half = freqs.numel()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]            # [T, half]
    cos = (torch.cos(ang) * mult).to(x.dtype)[:, None, :]
    sin = (torch.sin(ang) * mult).to(x.dtype)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = u * cos - v * sin
        out[..., 1:2 * half:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:2 * half]
        out[..., :half] = u * cos - v * sin
        out[..., half:2 * half] = v * cos + u * sin
    return out


def visible(T: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def sink_softmax_attention(q, k, v, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; head h reads key/value head
    ``h // (H / G)``; weights ``exp(s_j) / (1 + sum_j exp(s_j))``."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(-1, keepdim=True))
        out[:, h] = p @ v[:, g]
    return out


def mixer(kind: str, h: torch.Tensor, w: dict, pre: str, c: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D, Dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    dt = h.dtype

    def lin(name):
        y = h @ w[pre + name].to(dt).T
        if pre + name + ".b" in w:
            y = y + w[pre + name + ".b"].to(dt)
        return y

    q = lin("q").view(T, H, D)
    k = lin("k").view(T, G, D)
    v = lin("v").view(T, G, Dv) if kind == "attention_2" else k
    pos = torch.arange(T)
    freqs, mult = rotary_table(kind, c["rot"], torch.float64 if dt == torch.float64 else torch.float32)
    q = rotate(q, pos, freqs, mult, interleaved=(kind == "attention"))
    k = rotate(k, pos, freqs, mult, interleaved=(kind == "attention"))
    mask = visible(T, int(c["mask"]["size"]), int(c["mask"].get("keep_first", 0)) if kind == "attention_2" else 0)
    o = sink_softmax_attention(q, k, v, float(c["scale"]), mask).reshape(T, H * Dv)
    o = o * torch.sigmoid(h @ w[pre + "g"].to(dt).T)
    return o @ w[pre + "o"].to(dt).T


def feed_forward(h: torch.Tensor, w: dict, pre: str, c: dict) -> torch.Tensor:
    dt = h.dtype
    limit = float(c["limit"])
    g = h @ w[pre + "gate"].to(dt).T + w[pre + "gate.b"].to(dt)
    u = h @ w[pre + "up"].to(dt).T + w[pre + "up.b"].to(dt)
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1)
    return y @ w[pre + "down"].to(dt).T + w[pre + "down.b"].to(dt)


def layer_runs(config: dict) -> list[tuple[int, int | None]]:
    """The order the layers run in: (layer, pass number if the run opens a pass else None)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(config: dict, w: dict, tokens: list[int], dtype=torch.float64):
    """Logits [T, vocab] and the residual stream after every layer run [runs, T, width]."""
    eps = float(config["norm"]["eps"])
    x0 = w["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    streams = []
    for i, opens in layer_runs(config):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"].to(dtype)[opens]
        layer = config["layers"][i]
        p = f"l{i}."
        x = x + mixer(layer["type"], unit_offset_rms_norm(x, w[p + "norm1"], eps), w, p + "mix.",
                      layer["mixer"])
        if layer.get("mlp"):
            x = x + feed_forward(unit_offset_rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        streams.append(x.clone())
    logits = unit_offset_rms_norm(x, w["final.norm"], eps) @ w["head"].to(dtype).T
    return logits, torch.stack(streams)
