"""Embedding parts: what turns a step's token ids into the rows the layer list starts from.

A model without an embedding part gathers rows of its embedding table (``Stack.embed``). A part
of the ``embedding`` family may do more, keep state per request, and start the stream in a form
of its own; it is called with the ids, the step's context and, in recorded steps, the triple
``(use_prev, last_token, tok_slot)`` that says which ids are still on the device.

``HashedBigram``: ``e = norm(table[id] + bigram[(prev * mul_prev + id * mul_cur) mod buckets])``
with the bigram table's last row for a sequence's first token, an RMS norm in 32-bit, and the
result written ``copies`` times side by side as a float32 stream ``[T, copies * width]``. The
previous token of a portion's first token is the request's state (one int32).
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import EMBED_CALL, SlotState, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class HashedBigram:
    capture_safe = True
    stream_dtype = torch.float32

    def __init__(self, table: torch.Tensor, bigram: torch.Tensor | None, norm: torch.Tensor | None, eps: float,
                 buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0, copies: int = 1):
        self.table = table.contiguous()
        self.bigram = bigram.contiguous() if bigram is not None else None
        self.norm = norm.float().contiguous() if norm is not None else None
        self.eps, self.copies = float(eps), int(copies)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.bigram is not None and self.bigram.shape[0] != self.buckets + 1:
            raise ValueError(f"bigram embedding: {self.bigram.shape[0]} rows for {self.buckets} buckets and the "
                             "row of a sequence's first token")
        if not 1 <= self.copies <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"embedding: {self.copies} copies of the stream; 1..{ops.HYPER_MAX_STREAMS} are built")

    def state_specs(self) -> dict:
        return {"prev": SlotState((1,), torch.int32)} if self.bigram is not None else {}

    def forward(self, ids: torch.Tensor, ctx: StepContext, select: tuple | None = None) -> torch.Tensor:
        prev = ctx.states[(EMBED_CALL, "prev")] if self.bigram is not None else None
        return ops.embed_bigram_norm(self.table, self.bigram, self.norm, self.eps, ids, select, ctx.tok_seq,
                                     ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot, prev, self.copies, self.buckets,
                                     self.mul_prev, self.mul_cur)


@register("embedding", "bigram_hash")
def build_hashed_bigram(params: dict, tensors: dict, rt: Runtime) -> HashedBigram:
    return HashedBigram(tensors["table"], tensors.get("bigram"), tensors.get("norm"), params["eps"],
                        params.get("buckets", 0), params.get("mul_prev", 0), params.get("mul_cur", 0),
                        params.get("copies", 1))
