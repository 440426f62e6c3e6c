"""Rotary position encoding, rotate-half (neox) layout.

Frequencies ``inv_i = theta ** (-2 i / dim)`` for ``i < angles``, zero for the rest of
``dim / 2`` (a zero-tail partial rotation: those dims pass through with cos 1, sin 0), computed
once on the CPU in float32; the angle of a token is ``float(position) * inv_i`` and cos / sin are
rounded to the storage type (Tokenomos models/blocks/rope.py:33-35,51-59). One kernel norms the
q and k heads, rotates them by angles it computes from ``inv_freq`` and the positions, and
writes the new keys and values into the cache.
"""

from __future__ import annotations

import math

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class Rope:
    capture_safe = True

    def __init__(self, head_dim: int, angles: int, theta: float, device, dim: int | None = None):
        dim = dim or head_dim
        if dim % 2 or dim > head_dim:
            raise ValueError(f"rotary width {dim} of head size {head_dim}")
        if not 0 <= angles <= dim // 2:
            raise ValueError(f"{angles} rotary angles of width {dim}")
        idx = torch.arange(0, 2 * angles, 2, dtype=torch.float32)
        inv = 1.0 / (theta ** (idx / dim))
        inv = torch.cat((inv, torch.zeros(dim // 2 - angles, dtype=torch.float32)))
        self.inv_freq = inv.to(device).contiguous()
        self.dim = dim

    def rotate_half_frequencies(self) -> torch.Tensor:
        return self.inv_freq

    def encode_qk(self, qkv: torch.Tensor, ctx: StepContext, heads: HeadLayout,
                  pool: torch.Tensor | None, table: torch.Tensor | None) -> torch.Tensor:
        if self.dim > heads.head_dim:
            raise ValueError(f"rotary width {self.dim} above the head size {heads.head_dim}")
        return ops.qk_norm_rope_write(
            qkv, pool, heads.q_norm, heads.k_norm if heads.kv_heads else None, heads.eps,
            self.inv_freq, ctx.positions, ctx.tok_seq, table, heads.heads, heads.kv_heads,
            heads.head_dim, ctx.page_size)


@register("position", "rope")
def build_rope(params: dict, tensors: dict, rt: Runtime) -> Rope:
    return Rope(params["head_dim"], params["angles"], params["theta"], rt.device,
                params.get("dim"))


class Rotary:
    """Rotary encoding in its general form: the first ``dims`` columns of every q and k head are
    rotated by ``position * freq_i``, pairs ``(2i, 2i + 1)`` (``layout`` "interleaved") or
    ``(i, i + dims / 2)`` ("half"), ``freq_i = base ** (-2 i / dims)`` changed by ``scaling``:

    - ``{"kind": "linear", "factor": s}``: every frequency divided by ``s``;
    - ``{"kind": "yarn", "factor": s, "original": L, "fast": a, "slow": b}``: with ``turn(t) =
      dims * ln(L / (2 pi t)) / (2 ln base)``, ``lo = max(floor(turn(a)), 0)``, ``hi =
      min(ceil(turn(b)), dims - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``
      the frequency is ``freq_i / s * ramp_i + freq_i * (1 - ramp_i)``, and cos and sin are
      multiplied by ``0.1 * ln(s) + 1``.

    The table is computed once in float64 and kept in float32; angles, cos and sin are 32-bit
    and not rounded. The kernel also writes the new keys and values into the cache; the head
    layout may say that a value is its key before the rotation."""

    capture_safe = True

    def __init__(self, head_dim: int, dims: int, base: float, layout: str, scaling: dict | None, device):
        if dims % 2 or not 0 <= dims <= head_dim:
            raise ValueError(f"{dims} rotated columns of a head of {head_dim}")
        if layout not in ("interleaved", "half"):
            raise ValueError(f"rotary layout {layout!r}: 'interleaved' or 'half'")
        self.head_dim, self.dims, self.interleaved = head_dim, dims, layout == "interleaved"
        freqs, self.cs_mult = self.table(dims, float(base), scaling)
        self.freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device).contiguous()

    @staticmethod
    def table(dims: int, base: float, scaling: dict | None) -> tuple[list[float], float]:
        """(the ``dims / 2`` frequencies in double precision, the factor on cos and sin)."""
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        kind = (scaling or {}).get("kind")
        if kind is None:
            return freqs, 1.0
        factor = float(scaling["factor"])
        if kind == "linear":
            return [f / factor for f in freqs], 1.0
        if kind != "yarn":
            raise ValueError(f"rotary scaling {kind!r}: 'linear' or 'yarn'")

        def turn(t: float) -> float:
            return dims * math.log(float(scaling["original"]) / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
        out = []
        for i, f in enumerate(freqs):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return out, 0.1 * math.log(factor) + 1.0

    def plain_rotation(self) -> tuple[torch.Tensor, float, bool]:
        """(frequencies [dims / 2] float32, the factor on cos and sin, whether columns pair
        (2i, 2i + 1)): all there is to this encoding, for a mixer that applies it inside a kernel
        of its own (attention does, in steps where every sequence brings one token)."""
        return self.freq, self.cs_mult, self.interleaved

    def encode_qk(self, qkv: torch.Tensor, ctx: StepContext, heads: HeadLayout,
                  pool: torch.Tensor | None, table: torch.Tensor | None) -> torch.Tensor:
        if heads.q_norm is not None or heads.k_norm is not None:
            raise ValueError("Rotary: per-head q/k norms are the 'rope' encoding's")
        return ops.rotary_write(qkv, pool, self.freq, self.cs_mult, ctx.positions, ctx.tok_seq, table,
                                heads.heads, heads.kv_heads, heads.head_dim,
                                heads.v_dim if heads.v_dim is not None else heads.head_dim, ctx.page_size,
                                self.interleaved, heads.v_is_k)


@register("position", "rotary")
def build_rotary(params: dict, tensors: dict, rt: Runtime) -> Rotary:
    return Rotary(params["head_dim"], params["dims"], params["base"], params["layout"],
                  params.get("scaling"), rt.device)
