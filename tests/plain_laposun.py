"""A plain, slow implementation of the Laposun decoder: whole sequences, float64, one function
per mechanism, written from the design's equations. It shares no code with the package and is
the oracle of ``test_laposun.py``.

Notation: ``x`` [T, width] rows of one sequence, positions 0 .. T-1; linear weights [out, in]
applied as ``W x``; ``w`` maps tensor names to float64 tensors.
"""

from __future__ import annotations

import math

import torch

ROUTER_FLOOR = 1e-20


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def bigram_rows(tokens: list[int], buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """Row of the bigram table for every token: the table's last row for the first token."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return rows


def embedding(config: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    bg = (config.get("embedding") or {}).get("bigram")
    if bg is not None:
        rows = bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])
        x = x + w["bigram"][torch.tensor(rows, dtype=torch.long)]
    return rms_norm(x, w["embed.norm"], config["norm"]["eps"])


def input_conv(h: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``h + conv(h)``, ``conv(h)_t = sum_j taps[:, j] * h_(t - K + 1 + j)``, zeros before the start."""
    T, K = h.shape[0], taps.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(K):
            src = t - K + 1 + j
            if src >= 0:
                out[t] += taps[:, j] * h[src]
    return out


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Columns (2i, 2i + 1), i < dims / 2, of the last axis turned by ``position * base^(-2i/dims)``;
    ``x`` [T, ..., D], the other columns unchanged."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.double() * base ** (-2.0 * i / dims)
        shape = (-1,) + (1,) * (x.dim() - 2)
        c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def window_mask(T: int, window: int | None) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff 0 <= i - j (< window)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = i >= j
    if window is not None:
        vis &= (i - j) < window
    return vis


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The mixer, naively: keys and values of every head are up-projected from the latent."""
    T = h.shape[0]
    H, D, Dr, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    c_q = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (c_q @ w[p + "uq"].T).view(T, H, D + Dr)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :R], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(kv[:, R:], pos, m["rot"]["base"], m["rot"]["dims"])           # [T, Dr], all heads
    q_rot = rotate_pairs(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])           # [T, H, Dr]
    k = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, Dv)
    window = (m.get("mask") or {}).get("size")
    vis = window_mask(T, window)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                               # [T, H]
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for head in range(H):
        s = (q[:, head, :D] @ k[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        s = s.masked_fill(~vis, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, head] * gate[:, head:head + 1]
    return out.reshape(T, H * Dv) @ w[p + "o"].T


def swiglu(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def relu2_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ up.T) ** 2 @ down.T


def route(z: torch.Tensor, top: int, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """Router rows -> (chosen experts [T, top], their weights)."""
    s = torch.softmax(z, dim=-1)
    best, idx = torch.topk(s, top, dim=-1)
    return idx, best / (best.sum(dim=-1, keepdim=True) + ROUTER_FLOOR) * scale


def routed_experts(h: torch.Tensor, w: dict, p: str, f: dict) -> torch.Tensor:
    r = f["router"]
    idx, weight = route(h @ w[p + "router"].T, r["top"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(r["top"]):
            e = int(idx[t, k])
            out[t] += weight[t, k] * relu2_expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if f.get("shared") is not None:
        shared = relu2_expert(h, w[p + "shared.up"], w[p + "shared.down"])
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * shared
    return out


def hyper_read(xs: list[torch.Tensor], w_in: torch.Tensor | None) -> torch.Tensor:
    return sum(xs) if w_in is None else sum(w_in[s] * x for s, x in enumerate(xs))


def hyper_write(xs: list[torch.Tensor], y: torch.Tensor, mix: torch.Tensor | None,
                out: torch.Tensor | None) -> list[torch.Tensor]:
    """All streams at once from the old ones; ``mix`` is indexed [from, to]."""
    if mix is None:
        return [x + y for x in xs]
    S = len(xs)
    return [sum(mix[s, t] * xs[s] for s in range(S)) + out[t] * y for t in range(S)]


def forward(config: dict, w: dict, tokens: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
    """(logits [T, vocab], the sum of the streams after every layer [layers, T, width])."""
    eps = config["norm"]["eps"]
    x = embedding(config, w, tokens)
    has_hc = config.get("streams") is not None
    xs = [x.clone() for _ in range(config.get("streams") or 1)]
    taps = (config.get("canon") or {}).get("taps")
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            h = rms_norm(hyper_read(xs, w[f"{p}hc{q}.in"] if has_hc else None), w[f"{p}norm{q}"], eps)
            if taps is not None:
                h = input_conv(h, w[f"{p}canon{q}"])
            if q == 1:
                y = latent_attention(h, w, p + "mix.", layer["mixer"], eps)
            elif layer["mlp"]["kind"] == "dense":
                y = swiglu(h, w, p + "mlp.")
            else:
                y = routed_experts(h, w, p + "mlp.", layer["mlp"])
            xs = hyper_write(xs, y, w[f"{p}hc{q}.mix"] if has_hc else None, w[f"{p}hc{q}.out"] if has_hc else None)
        after.append(sum(xs))
    logits = rms_norm(sum(xs), w["final.norm"], eps) @ w["embed"].T
    return logits, torch.stack(after)
