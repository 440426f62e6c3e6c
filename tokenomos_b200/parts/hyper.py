"""Hyper-connections: a residual stream in ``S`` copies, and the block arrangement that uses it.

Instead of ``x <- x + f(norm(x))`` a sublayer reads a weighted sum of the copies and writes into
all of them:

    u = sum_s in[s] x_s;   y = f(conv(norm(u)));   x_t <- sum_s mix[s, t] x_s + out[t] y

``StreamReader`` (family ``norm``, kind ``hyper_norm``) owns one sublayer's ``in``, ``mix``,
``out``, its RMS norm and, optionally, a short causal convolution over time on what the sublayer
reads (``h <- h + conv(h)``, the last taps - 1 rows of ``h`` kept per request). The write of a
sublayer is done by the reader of the next one, in the same kernel as its read and norm, as a
plain pre-norm block leaves its add to the next norm; the model's final norm is a reader without
weights on the copies (their plain sum) and without a convolution. The stream is float32
``[T, S * width]`` whatever the storage type; ``S`` = 1 with no ``in / mix / out`` is the plain
residual stream in 32-bit.

``HyperBlock`` (kind ``hyper``): mixer and feed-forward (or none), each behind its reader.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SlotState, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class StreamReader:
    capture_safe = True
    stream_dtype = torch.float32

    def __init__(self, weight: torch.Tensor, eps: float, streams: int, store: torch.dtype,
                 hc_in: torch.Tensor | None = None, hc_mix: torch.Tensor | None = None,
                 hc_out: torch.Tensor | None = None, taps: torch.Tensor | None = None, tile: int = 16):
        self.weight = weight.float().contiguous()
        self.eps, self.streams, self.store = float(eps), int(streams), store
        self.width = weight.numel()
        if not 1 <= self.streams <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"hyper-connections: {self.streams} streams; 1..{ops.HYPER_MAX_STREAMS} are built")
        S = self.streams
        for name, t, shape in (("in", hc_in, (S,)), ("mix", hc_mix, (S, S)), ("out", hc_out, (S,))):
            if t is not None and tuple(t.shape) != shape:
                raise ValueError(f"hyper-connections: '{name}' of shape {tuple(t.shape)} for {S} streams")
        self.hc_in = hc_in.float().contiguous() if hc_in is not None else None
        self.hc_mix = hc_mix.float().contiguous().view(-1) if hc_mix is not None else None    # [from, to]
        self.hc_out = hc_out.float().contiguous() if hc_out is not None else None
        self.taps = None
        if taps is not None:
            self.taps = taps.float().reshape(self.width, -1).contiguous()
            k = self.taps.shape[1]
            if not 1 <= k <= ops.CANON_MAX_TAPS:
                raise ValueError(f"input convolution: {k} taps; 1..{ops.CANON_MAX_TAPS} are built")
            self.tile = max(int(tile), k - 1, 1)

    def state_shape(self) -> tuple | None:
        """Shape of the rows this reader keeps per request (None: it keeps nothing)."""
        if self.taps is None or self.taps.shape[1] < 2:
            return None
        return (self.taps.shape[1] - 1, self.width)

    def read(self, streams: torch.Tensor, y: torch.Tensor | None, writer: "StreamReader | None",
             ctx: StepContext | None, state: torch.Tensor | None) -> torch.Tensor:
        """Apply ``writer``'s write of ``y`` to ``streams`` (in place), then this sublayer's read:
        what the sublayer gets, in the storage type."""
        mix = writer.hc_mix if writer is not None else None
        out = writer.hc_out if writer is not None else None
        if self.taps is not None and ctx.host.decode_only:
            # every sequence brings one token: the convolution and its state ride in the same kernel
            return ops.hc_mix_norm(streams, y, mix, out, self.hc_in, self.weight, self.eps, self.streams, self.store,
                                   keep32=False, conv=(self.taps, state, ctx.seq_ctx, ctx.seq_slot))
        h = ops.hc_mix_norm(streams, y, mix, out, self.hc_in, self.weight, self.eps, self.streams, self.store,
                            keep32=self.taps is not None)
        if self.taps is None:
            return h
        return ops.canon_conv(h, self.taps, state, ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot,
                              ctx.tiles(self.tile), self.store)

    # the norm contract, for the place of a model's final norm: the last sublayer's write, the sum
    # of the copies, the norm
    def add_norm(self, x: torch.Tensor, residual: torch.Tensor | None, pre=None):
        if self.taps is not None:
            raise ValueError("a stream reader with an input convolution needs the step's context: it is a "
                             "block's reader, not a final norm")
        if residual is None:
            streams, y = x, None
        else:
            streams, y = residual, x
        return self.read(streams, y, pre, None, None), streams

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)[0]


@register("norm", "hyper_norm")
def build_stream_reader(params: dict, tensors: dict, rt: Runtime) -> StreamReader:
    return StreamReader(tensors["weight"], params["eps"], params.get("streams", 1), rt.dtype,
                        tensors.get("in"), tensors.get("mix"), tensors.get("out"), tensors.get("taps"),
                        tile=rt.tuning.conv_tile)


class HyperBlock:
    """``mixer`` and ``ffn`` (or None) behind their readers. The stream it carries between blocks
    is ``(y, streams, writer)``: the last sublayer's output, not yet written, and the reader that
    holds its ``mix`` and ``out``."""

    def __init__(self, mixer, ffn, read_mixer: StreamReader, read_ffn: StreamReader | None):
        if (ffn is None) != (read_ffn is None):
            raise ValueError("a block's feed-forward and its reader come together or not at all")
        self.mixer, self.ffn, self.read_mixer, self.read_ffn = mixer, ffn, read_mixer, read_ffn
        self.capture_safe = all(getattr(p, "capture_safe", False)
                                for p in (mixer, ffn, read_mixer, read_ffn) if p is not None)

    def state_specs(self) -> dict:
        specs = dict(self.mixer.state_specs())
        for name, reader in (("canon_mixer", self.read_mixer), ("canon_ffn", self.read_ffn)):
            shape = reader.state_shape() if reader is not None else None
            if shape is not None:
                specs[name] = SlotState(shape, torch.float32)
        return specs

    def forward(self, h, residual, pending, ctx: StepContext, call: int):
        if residual is None:                 # the first block: ``h`` is the stream as the embedding left it
            streams, y = h, None
        else:
            streams, y = residual, h
        x = self.read_mixer.read(streams, y, pending, ctx, ctx.states.get((call, "canon_mixer")))
        y = self.mixer.forward(x, ctx, call)
        if self.ffn is None:
            return y, streams, self.read_mixer
        x = self.read_ffn.read(streams, y, self.read_mixer, ctx, ctx.states.get((call, "canon_ffn")))
        return self.ffn.forward(x), streams, self.read_ffn


@register("block", "hyper")
def build_hyper_block(parts: dict) -> HyperBlock:
    return HyperBlock(parts["mixer"], parts.get("ffn"), parts["pre_mixer_norm"], parts.get("pre_ffn_norm"))
