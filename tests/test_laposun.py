"""The Laposun decoder against its plain implementation (``plain_laposun``): every mechanism
alone, the whole model replayed four ways in 32-bit and in bfloat16 on poisoned pools, keys at
the edges of windows and pages made loud, portions down to two tokens, long decoding, generation
through the entry points. The configurations are made for the tests: one, two and three streams,
one to five taps, no bigram table, partial rotation, one expert per token, every expert per
token, no shared expert, a layer without a feed-forward, sizes no 16-byte kernel takes."""

from __future__ import annotations

import json
import math
import subprocess
import sys
import types
from pathlib import Path

import pytest
import torch

import plain_laposun as plain
import trace_util

ROOT = Path(__file__).resolve().parents[1]


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, dims=None, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": dims or rot_dim}}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


# A: three streams, three taps, partial rotation, value size unlike key size, a layer without a
#    feed-forward, windows that no page size divides
LP_A = {"architecture": "Laposun", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "streams": 3,
        "canon": {"taps": 3}, "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
        "layers": [dict(latent(4, 16, 8, 24, 40, 32, 9), mlp=dense(96)),
                   dict(latent(3, 8, 12, 8, 24, 24, 13, dims=4, base=500.0), mlp=moe(6, 2, 32, 2.0, shared=48)),
                   dict(latent(2, 24, 4, 16, 16, 40, 40), mlp=None)]}
# B: one stream with connection weights, two taps, one expert per token without a shared expert,
#    every expert per token, a window of one position and one longer than any request
LP_B = {"architecture": "Laposun", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "streams": 1,
        "canon": {"taps": 2}, "embedding": {"bigram": {"buckets": 50, "mul_prev": 3, "mul_cur": 1000003}},
        "layers": [dict(latent(4, 12, 8, 12, 32, 16, 16), mlp=moe(5, 1, 40, 1.0)),
                   dict(latent(1, 8, 8, 8, 8, 8, 1), mlp=moe(4, 4, 24, 0.5, shared=16)),
                   dict(latent(6, 8, 2, 20, 48, 24, 500, scale=0.4), mlp=dense(80))]}
# C: no streams entry, no convolution, no bigram table; no window; one layer, one head
LP_C = {"architecture": "Laposun", "vocab": 128, "width": 32, "norm": {"eps": 1e-5},
        "layers": [dict(latent(1, 16, 16, 16, 16, 16, None), mlp=dense(32))]}
# D: sizes no 16-byte kernel takes; five taps (more than the shortest portions), two streams
LP_D = {"architecture": "Laposun", "vocab": 50, "width": 36, "norm": {"eps": 1e-5}, "streams": 2,
        "canon": {"taps": 5}, "embedding": {"bigram": {"buckets": 11, "mul_prev": 5, "mul_cur": 2}},
        "layers": [dict(latent(3, 10, 6, 6, 14, 20, 7, dims=2), mlp=moe(3, 2, 21, 1.5, shared=9)),
                   dict(latent(2, 6, 10, 10, 10, 12, 5), mlp=dense(30))]}
# E: sizes the tensor-core kernels take in bfloat16, windows over several pages, more experts
LP_E = {"architecture": "Laposun", "vocab": 400, "width": 128, "norm": {"eps": 1e-5}, "streams": 4,
        "canon": {"taps": 4}, "embedding": {"bigram": {"buckets": 509, "mul_prev": 211, "mul_cur": 13}},
        "layers": [dict(latent(8, 32, 32, 32, 64, 64, 40), mlp=moe(12, 3, 64, 1.0, shared=64)),
                   dict(latent(16, 16, 16, 16, 48, 128, 70), mlp=dense(160)),
                   dict(latent(4, 64, 32, 64, 64, 32, 24, dims=16), mlp=moe(8, 2, 128, 2.5))]}

CASES = {
    "A": dict(config=LP_A, seed=21, page=4, lengths=[1, 2, 7, 30, 61, 45]),
    "B": dict(config=LP_B, seed=22, page=8, lengths=[3, 19, 21, 50, 90, 33]),
    "C": dict(config=LP_C, seed=23, page=16, lengths=[1, 5, 64, 65, 140]),
    "D": dict(config=LP_D, seed=24, page=4, lengths=[1, 6, 23, 40]),
    "E": dict(config=LP_E, seed=25, page=16, lengths=[2, 31, 150, 65, 200, 90]),
}
# Bounds relative to a request's largest |logit|. The 32-bit model computes what the plain
# implementation computes, in another order; bfloat16 rounds every product's inputs and outputs.
TOL_F32 = {"A": 2e-5, "B": 2e-5, "C": 1e-5, "D": 2e-5, "E": 4e-5}
TOL_F32_SAME = {"A": 1e-5, "B": 1e-5, "C": 5e-6, "D": 1e-5, "E": 2e-5}
TOL_BF16 = {"A": 0.1, "B": 0.1, "C": 0.08, "D": 0.1, "E": 0.15}
CLOSE_CALLS = 0.06        # of a request's positions, in bfloat16 only (see ``compare``)


def make_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16: loud queries and keys (a key more or less behind a
    window's edge moves the logits far beyond rounding), connection weights around the plain
    residual stream, norm weights far from one, taps of the size of the signal."""
    from tokenomos_b200 import models
    from tokenomos_b200.weights.random_init import random_tensors

    arch = models.architecture_of(config)
    spec = arch.declare(arch.config_class.from_dict(config))
    tensors = random_tensors(spec.tensor_decls(), seed, std=1.0)
    S = config.get("streams") or 1
    out = {}
    noise = torch.Generator().manual_seed(seed + 1000)
    for name, t in tensors.items():
        if ".hc" in name or "norm" in name:          # (the random-weights mode draws these as ones)
            t = torch.randn(t.shape, generator=noise)
        if name.endswith((".hc1.in", ".hc2.in")):
            t = 1.0 / S + 0.3 * t
        elif name.endswith((".hc1.out", ".hc2.out")):
            t = 1.0 + 0.3 * t
        elif name.endswith((".hc1.mix", ".hc2.mix")):
            t = torch.eye(S) + 0.2 * t
        elif "norm" in name:
            t = 1.0 + 0.3 * t
        elif "canon" in name:
            t = 0.4 * t
        elif name.endswith((".mix.uq", ".mix.uk")):
            t = t * (2.0 / math.sqrt(t.shape[-1]))
        elif name.endswith(".router"):
            t = t * (3.0 / math.sqrt(t.shape[-1]))
        elif name in ("embed", "bigram"):
            t = t * 1.0
        else:
            t = t / math.sqrt(t.shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from safetensors.torch import save_file

    out = {}
    for name, case in CASES.items():
        folder = tmp_path_factory.mktemp(f"lp_{name}")
        tensors = make_tensors(case["config"], case["seed"])
        (folder / "config.json").write_text(json.dumps(case["config"]))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
        out[name] = (folder, {k: v.double() for k, v in tensors.items()})
    return out


def requests_for(name: str) -> dict[str, list[int]]:
    g = torch.Generator().manual_seed(177 + ord(name))
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist()
            for i, n in enumerate(CASES[name]["lengths"])}


def compare(got: dict, want: dict, tol: float, what: str, close_calls: float = 0.0):
    """``close_calls``: the share of a request's positions (at least one, if not zero) that may lie
    outside the bound. A 16-bit model's router sees inputs that differ from the plain
    implementation's by rounding; where two experts' scores are that close it takes the other
    one, and the position's logits move by a whole expert's output. The 32-bit model gets none."""
    for rid, ref in want.items():
        assert got[rid].shape == ref.shape, (what, rid, got[rid].shape, ref.shape)
        assert torch.isfinite(got[rid]).all(), (what, rid)
        err = (got[rid] - ref).abs().amax(dim=1)
        scale = ref.abs().max().item()
        bad = (err > tol * scale).nonzero()
        allowed = math.ceil(close_calls * len(err)) if close_calls else 0
        assert bad.numel() <= allowed, (f"{what}: request {rid}: first wrong position {int(bad[0])} of {len(err)}: "
                                  f"error {err[int(bad[0])].item():.3e}, allowed {tol * scale:.3e}")


# ---------------------------------------------------------------------------------------------
# without a GPU: configuration, declaration, the latent cache's pages, the oracle's own pieces
# ---------------------------------------------------------------------------------------------

def test_configuration_reads_every_size_and_lists_every_fault():
    from tokenomos_b200.config import ConfigError, LaposunConfig

    cfg = LaposunConfig.from_dict(LP_A)
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.taps) == (300, 64, 3, 3)
    assert (cfg.bigram.buckets, cfg.bigram.mul_prev, cfg.bigram.mul_cur) == (97, 31, 7)
    m = cfg.layers[1].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.window, m.rot_dims, m.rot_base) == (
        3, 8, 12, 8, 24, 24, 13, 4, 500.0)
    f = cfg.layers[1].mlp
    assert (f.kind, f.experts, f.top, f.ff, f.scale, f.shared_ff) == ("moe", 6, 2, 32, 2.0, 48)
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp.kind == "dense"
    plain_cfg = LaposunConfig.from_dict(LP_C)
    assert plain_cfg.streams is None and plain_cfg.taps is None and plain_cfg.bigram is None
    assert plain_cfg.layers[0].mixer.window is None
    bad = json.loads(json.dumps(LP_A))
    del bad["width"]
    bad["layers"][0]["mixer"]["rot"]["dims"] = 10          # above rot_dim
    bad["layers"][1]["mlp"]["router"]["top"] = 9           # of 6 experts
    bad["layers"][2]["type"] = "something"
    with pytest.raises(ConfigError) as err:
        LaposunConfig.from_dict(bad)
    text = str(err.value)
    assert "width" in text and "rot.dims" in text and "top = 9" in text and "something" in text


def test_declaration_lists_the_tensors_and_the_state():
    from tokenomos_b200 import models

    arch = models.architecture_of(LP_A)
    spec = arch.declare(arch.config_class.from_dict(LP_A))
    names = {d.name: d for d in spec.tensor_decls()}
    assert names["bigram"].shape == (98, 64) and names["l1.mlp.shared.sg"].shape == (1, 64)
    assert names["l0.hc1.mix"].shape == (3, 3) and names["l2.canon1"].shape == (64, 3)
    assert names["l1.mix.uq"].shape == (3 * 20, 24) and names["l1.mix.dkv"].shape == (24 + 12, 64)
    assert "l1.mlp.e5.down" in names and "l1.mlp.e6.up" not in names
    assert names["l2.norm2"].optional and "head" not in names
    bare = arch.declare(arch.config_class.from_dict(LP_C))
    assert not any(".hc" in d.name or "canon" in d.name or d.name == "bigram" for d in bare.tensor_decls())


def test_latent_cache_rows_and_window_pages_come_back():
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.parts.contract import EMBED_CALL, LatentKV, SlotState

    specs = {(0, "kv"): LatentKV(20, 9), (1, "kv"): LatentKV(12, None), (EMBED_CALL, "prev"): SlotState((1,), torch.int32)}
    cache = CacheManager(specs, 4, 12, 2, torch.float32, "cpu", max_len=40)
    assert tuple(cache.states[(0, "kv")].shape) == (12, 4, 20) and cache.states[(EMBED_CALL, "prev")].dtype == torch.int32
    cache.admit("a")
    cache.extend("a", 30)
    cache.commit("a", 30)
    cache.check()
    win, full = cache.block_table("a", ("window", 9)), cache.block_table("a", ("full",))
    assert sum(1 for p in full if p) == 8
    # positions 22.. are still visible to position 30: blocks 0..4 have gone back
    assert [bool(p) for p in win] == [False] * 5 + [True] * 3
    cache.release("a")
    cache.check()


def test_oracle_pieces():
    assert plain.bigram_rows([5, 9, 9], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7]
    h = torch.arange(8, dtype=torch.float64).view(4, 2)
    taps = torch.tensor([[1.0, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)
    out = plain.input_conv(h, taps)
    # channel 0: h + 1 * h(t-2) + 2 * h(t); channel 1: h + h(t-1)
    assert out[:, 0].tolist() == [0.0, 6.0, 12.0, 20.0] and out[:, 1].tolist() == [1.0, 4.0, 8.0, 12.0]
    idx, wgt = plain.route(torch.tensor([[0.0, 2.0, 1.0]], dtype=torch.float64), 2, 3.0)
    assert idx.tolist() == [[1, 2]] and abs(wgt.sum().item() - 3.0) < 1e-12
    x = torch.randn(3, 2, 6, dtype=torch.float64)
    r = plain.rotate_pairs(x, torch.tensor([0, 1, 7]), 100.0, 4)
    assert torch.equal(r[0], x[0]) and torch.equal(r[..., 4:], x[..., 4:])
    assert torch.allclose((r[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))
    assert plain.window_mask(5, 2).sum().item() == 9 and plain.window_mask(4, None).sum().item() == 10


# ---------------------------------------------------------------------------------------------
# each mechanism alone, on the GPU
# ---------------------------------------------------------------------------------------------

class Harness:
    """A cache manager over the given state specs and a step function's layouts, without a model."""

    def __init__(self, specs: dict, page: int, pages: int, dtype, vocab: int = 1000, slots: int = 3):
        from tokenomos_b200.cache.manager import CacheManager
        from tokenomos_b200.engine.step import StepFunction

        self.cache = CacheManager(specs, page, pages, slots, dtype, "cuda", max_len=(pages - 1) * page, poison=True)
        self.steps = StepFunction(types.SimpleNamespace(vocab=vocab), self.cache)

    def layout(self, entries: list[tuple[str, list[int]]]):
        from tokenomos_b200.engine.step import StepEntry

        for rid, _ in entries:
            if rid not in self.cache.requests:
                self.cache.admit(rid)
        ctx, ids, _ = self.steps.layout([StepEntry(rid, toks, []) for rid, toks in entries])
        return ctx, ids

    def commit(self, entries):
        for rid, toks in entries:
            self.cache.commit(rid, len(toks))


def cuts_of(n: int, sizes) -> list[tuple[int, int]]:
    out, a, k = [], 0, 0
    while a < n:
        b = min(n, a + sizes[k % len(sizes)])
        out.append((a, b))
        a, k = b, k + 1
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("copies, width, bigram", [(1, 40, True), (3, 33, True), (2, 64, False)])
def test_embedding_alone(dtype, copies, width, bigram):
    """Two requests fed in unequal portions side by side, one slot used again: the bigram row of a
    portion's first token comes from the request's state, the very first token takes the last row."""
    from tokenomos_b200.parts.contract import EMBED_CALL
    from tokenomos_b200.parts.embedding import HashedBigram

    g = torch.Generator().manual_seed(3)
    vocab, buckets = 90, 13
    table = torch.randn(vocab, width, generator=g).to(torch.bfloat16)
    big = torch.randn(buckets + 1, width, generator=g).to(torch.bfloat16)
    norm = 1.0 + 0.3 * torch.randn(width, generator=g).to(torch.bfloat16).float()
    config = {"norm": {"eps": 1e-5}, "embedding": {"bigram": {"buckets": buckets, "mul_prev": 1000003, "mul_cur": 17}}}
    if not bigram:
        del config["embedding"]
    w = {"embed": table.double(), "bigram": big.double(), "embed.norm": norm.double()}
    part = HashedBigram(table.to(dtype).cuda(), big.to(dtype).cuda() if bigram else None, norm.cuda(), 1e-5,
                        buckets, 1000003, 17, copies)
    specs = {(EMBED_CALL, k): v for k, v in part.state_specs().items()}
    hs = Harness(specs, 4, 40, dtype, vocab, slots=2)
    seqs = {"a": torch.randint(0, vocab, (23,), generator=g).tolist(),
            "b": torch.randint(0, vocab, (9,), generator=g).tolist(),
            "c": torch.randint(0, vocab, (5,), generator=g).tolist()}
    plan = {"a": cuts_of(23, (1, 1, 5, 2, 7, 1, 6)), "b": cuts_of(9, (4, 1, 1, 3)), "c": cuts_of(5, (2, 3))}
    got = {rid: [] for rid in seqs}
    live = ["a", "b"]
    while live:
        entries = [(rid, seqs[rid][slice(*plan[rid].pop(0))]) for rid in live]
        ctx, ids = hs.layout(entries)
        out = part.forward(ids, ctx)
        hs.commit(entries)
        o = 0
        for rid, toks in entries:
            got[rid].append(out[o:o + len(toks)].double().cpu())
            o += len(toks)
        for rid in list(live):
            if not plan[rid]:
                hs.cache.release(rid)
                live.remove(rid)
                if rid == "b":
                    live.append("c")           # takes the slot b left
    for rid, toks in seqs.items():
        want = plain.embedding(config, w, toks)
        have = torch.cat(got[rid])
        assert have.shape == (len(toks), copies * width)
        for c in range(copies):
            assert (have[:, c * width:(c + 1) * width] - want).abs().max() < 1e-5, (rid, c)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S, width", [(1, 36), (2, 64), (3, 50), (8, 128)])
def test_connections_alone(dtype, S, width):
    from tokenomos_b200 import ops

    g = torch.Generator().manual_seed(S)
    T = 11
    x = torch.randn(T, S, width, generator=g)
    y = torch.randn(T, width, generator=g).to(dtype)
    mix, out_w, in_w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    norm = 1.0 + 0.3 * torch.randn(width, generator=g)
    xs = [x[:, s].double() for s in range(S)]
    new = plain.hyper_write(xs, y.double(), mix.double(), out_w.double())
    want = plain.rms_norm(plain.hyper_read(new, in_w.double()), norm.double(), 1e-5)
    streams = x.reshape(T, S * width).cuda().contiguous()
    for keep32 in (True, False):
        st = streams.clone()
        h = ops.hc_mix_norm(st, y.cuda(), mix.reshape(-1).cuda(), out_w.cuda(), in_w.cuda(), norm.cuda(), 1e-5, S,
                            dtype, keep32)
        assert h.dtype == (torch.float32 if keep32 else dtype)
        tol = 1e-5 if (keep32 or dtype == torch.float32) else 2e-2
        assert (h.double().cpu() - want).abs().max() < tol * want.abs().max()
        assert (st.view(T, S, width).double().cpu() - torch.stack(new, 1)).abs().max() < 1e-5 * x.abs().max()
    # the plain sum of the copies (a final norm), and a read without a write
    st = streams.clone()
    h = ops.hc_mix_norm(st, None, None, None, None, norm.cuda(), 1e-5, S, dtype, True)
    assert torch.equal(st, streams)
    assert (h.double().cpu() - plain.rms_norm(sum(xs), norm.double(), 1e-5)).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("width", [20, 256, 300])
def test_input_convolution_alone(taps, width):
    """Sequences cut into portions down to one token, shorter than the taps, two requests side by
    side, a state row used again after its request ended."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts.contract import SlotState

    g = torch.Generator().manual_seed(taps * 7 + width)
    w_taps = torch.randn(width, taps, generator=g)
    specs = {(0, "c"): SlotState((taps - 1, width), torch.float32)} if taps > 1 else {}
    hs = Harness(specs, 4, 60, torch.float32, slots=2)
    seqs = {"a": torch.randn(41, width, generator=g), "b": torch.randn(13, width, generator=g),
            "c": torch.randn(6, width, generator=g)}
    plan = {"a": cuts_of(41, (1, 2, 1, 1, 9, 2, 20, 3)), "b": cuts_of(13, (3, 1, 1, 2, 6)), "c": cuts_of(6, (1, 5))}
    got = {rid: [] for rid in seqs}
    live = ["a", "b"]
    tile = max(4, taps - 1)
    while live:
        spans = {rid: plan[rid].pop(0) for rid in live}
        entries = [(rid, [0] * (spans[rid][1] - spans[rid][0])) for rid in live]
        ctx, _ = hs.layout(entries)
        h = torch.cat([seqs[rid][slice(*spans[rid])] for rid in live]).cuda()
        if ctx.host.decode_only:
            # a step of single tokens: the convolution inside the kernel that reads the streams (one
            # stream, unit weights, a norm that leaves rows of unit mean square as they are)
            unit = h / h.pow(2).mean(-1, keepdim=True).sqrt()
            out = ops.hc_mix_norm(unit.clone(), None, None, None, None, torch.ones(width, device="cuda"), 0.0, 1,
                                  torch.float32, False,
                                  conv=(w_taps.cuda(), hs.cache.states.get((0, "c")), ctx.seq_ctx, ctx.seq_slot))
            # the plain implementation below gets the unit rows too
            for k, rid in enumerate(live):
                a, b = spans[rid]
                seqs[rid] = seqs[rid].clone()
                seqs[rid][a:b] = unit[k:k + 1].cpu()
        else:
            out = ops.canon_conv(h, w_taps.cuda(), hs.cache.states.get((0, "c")), ctx.cu_seqlens, ctx.seq_ctx,
                                 ctx.seq_slot, ctx.tiles(tile), torch.float32)
        hs.commit(entries)
        o = 0
        for rid, toks in entries:
            got[rid].append(out[o:o + len(toks)].double().cpu())
            o += len(toks)
        for rid in list(live):
            if not plan[rid]:
                hs.cache.release(rid)
                live.remove(rid)
                if rid == "b":
                    live.append("c")
    for rid, h in seqs.items():
        want = plain.input_conv(h.double(), w_taps.double())
        assert (torch.cat(got[rid]) - want).abs().max() < 1e-5 * want.abs().max(), rid


class LatentSequence:
    """One request's latent attention through a poisoned latent cache with shuffled pages."""

    def __init__(self, H, D, Dr, R, rot, page, length, dtype, base=100.0):
        from tokenomos_b200.parts.contract import LatentKV
        from tokenomos_b200.parts.rope import Rotary

        self.H, self.D, self.Dr, self.R, self.rot, self.page, self.dtype = H, D, Dr, R, rot, page, dtype
        self.window = None
        self.hs = Harness({(0, "kv"): LatentKV(R + Dr, None)}, page, length // page + 8, dtype, slots=2)
        # hold and return a few pages so that the request's pages are neither first nor in order
        self.hs.cache.admit("junk")
        self.hs.cache.extend("junk", 3 * page)
        self.hs.cache.admit("x")
        self.hs.cache.extend("x", page)
        self.hs.cache.release("junk")
        freqs, _ = Rotary.table(rot, base, None)
        self.freq = torch.tensor(freqs, dtype=torch.float64).float().cuda()
        self.base = base

    def feed(self, proj, q, a, b, window, scale):
        """Positions [a, b): ``proj`` [T, R + Dr] the kv latent and key part before norm and rotation,
        ``q`` [T, H, D + Dr] before rotation, with the keys' up-projection ``uk`` applied by the caller
        (q_lat given). Returns the attended latents [b - a, H, R]."""
        from tokenomos_b200 import ops

        ctx, _ = self.hs.layout([("x", [0] * (b - a))])
        cache = self.hs.cache.states[(0, "kv")]
        table = ctx.block_tables[("full",)]
        ones = torch.ones(self.R, device="cuda")
        rows = torch.cat((torch.zeros(b - a, 8, dtype=proj.dtype), proj[a:b]), dim=1).to(self.dtype).cuda()
        ops.latent_prepare(rows, torch.ones(8, device="cuda"), ones, 1e-6, self.freq, ctx.positions, ctx.tok_seq,
                           table, cache, 8, self.R, self.Dr)
        qq = q[a:b].reshape(b - a, -1).to(self.dtype).cuda().contiguous()
        ops.latent_rotate_q(qq, self.freq, ctx.positions, self.H, self.D, self.Dr)
        q_lat = q[a:b, :, :self.R].transpose(0, 1).to(self.dtype).cuda().contiguous()       # D >= R in these tests
        per_tile = ops.attention_latent_tokens(self.H, self.D, self.R, self.Dr, self.dtype)
        if b - a == 1:
            per_tile = 1          # a single token: the 16-row form where the tensor-core kernel runs
        _, tok0, _, ntok = ctx.tiles(per_tile)
        # (a single token's keys shared out over three CTAs where the tensor-core form runs)
        out = ops.attention_latent(q_lat, qq, cache, ctx.positions, ctx.tok_seq, table, tok0, ntok, per_tile,
                                   self.H, self.D, self.Dr, window, scale, nsplit=3 if b - a == 1 else 1,
                                   rows16=b - a == 1 and per_tile == 1)
        self.hs.commit([("x", [0] * (b - a))])
        return out.transpose(0, 1).double().cpu()


def plain_latent_scores(proj, q, R, Dr, rot, base, window, scale, eps=1e-6):
    """The attended latents [T, H, R] of the plain equations, with q's first R columns as the
    query in the latent's space."""
    T = proj.shape[0]
    pos = torch.arange(T)
    c = plain.rms_norm(proj[:, :R], torch.ones(R, dtype=torch.float64), eps)
    k_rot = plain.rotate_pairs(proj[:, R:], pos, base, rot)
    D = q.shape[2] - Dr
    q_rot = plain.rotate_pairs(q[..., D:], pos, base, rot)
    vis = plain.window_mask(T, window)
    out = torch.zeros(T, q.shape[1], R, dtype=torch.float64)
    for h in range(q.shape[1]):
        s = (q[:, h, :R] @ c.T + q_rot[:, h] @ k_rot.T) * scale
        out[:, h] = torch.softmax(s.masked_fill(~vis, -math.inf), -1) @ c
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("case", [dict(H=3, D=20, Dr=6, R=20, rot=4, page=4, window=9),
                                  dict(H=16, D=64, Dr=32, R=64, rot=32, page=16, window=33),
                                  dict(H=6, D=96, Dr=16, R=96, rot=16, page=8, window=70),
                                  dict(H=40, D=32, Dr=16, R=32, rot=8, page=4, window=20),
                                  dict(H=5, D=40, Dr=8, R=40, rot=8, page=8, window=None),
                                  dict(H=2, D=24, Dr=2, R=24, rot=2, page=4, window=1)])
def test_latent_cache_and_attention_with_one_loud_key(case, dtype, how):
    """Random keys among which one is loud: at the first position, just inside and just outside the
    window of the last query, at a page border, far back. A window one position off moves the
    result by far more than the bound."""
    H, D, Dr, R, rot, page, window = (case[k] for k in ("H", "D", "Dr", "R", "rot", "page", "window"))
    T = 75
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for loud in sorted({0, 1, page - 1, page, T - (window or 40), T - (window or 40) - 1, T - 2, T - 1}):
        if not 0 <= loud < T:
            continue
        g = torch.Generator().manual_seed(loud)
        proj = torch.randn(T, R + Dr, generator=g).to(torch.bfloat16).double()
        q = (0.3 * torch.randn(T, H, D + Dr, generator=g)).to(torch.bfloat16).double()
        # every query leans towards the loud key's latent: its score stands ~R/4 above the others
        q[:, :, :R] += 0.5 * proj[loud, :R] / proj[loud, :R].norm() * math.sqrt(R)
        want = plain_latent_scores(proj, q, R, Dr, rot, 100.0, window, 0.5)
        seq = LatentSequence(H, D, Dr, R, rot, page, T + 8, dtype)
        if how == "whole":
            spans = [(0, T)]
        elif how == "decoded":
            spans = [(0, T - 30)] + [(i, i + 1) for i in range(T - 30, T)]
        else:
            spans = cuts_of(T, (5, 2, 17, 3, 2, 29, 1))
        got = torch.cat([seq.feed(proj, q, a, b, window, 0.5) for a, b in spans])
        assert torch.isfinite(got).all()
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err < tol, (case, loud, how, err)
        if window is not None and window > 1 and loud == T - window - 1:
            # the negative control: the same keys under a window one longer see the loud key
            off = plain_latent_scores(proj, q, R, Dr, rot, 100.0, window + 1, 0.5)
            # (ten times the 16-bit bound, 15,000 times the 32-bit one)
            assert (off[-1] - want[-1]).abs().max() > 0.3 * want.abs().max()


@pytest.mark.gpu
def test_batched_and_grouped_products():
    from tokenomos_b200 import ops

    g = torch.Generator().manual_seed(0)
    a = torch.randn(5, 70, 24, generator=g).cuda()
    w = torch.randn(5, 33, 24, generator=g).cuda()
    got = ops.gemm_batched(a, w)
    assert (got - torch.einsum("gmk,gnk->gmn", a.double(), w.double()).float()).abs().max() < 1e-4
    strided = torch.randn(70, 5, 40, generator=g).cuda()[:, :, :24].transpose(0, 1)      # [5, 70, 24], rows 200 apart
    got = ops.gemm_batched(strided, w)
    assert (got - torch.einsum("gmk,gnk->gmn", strided.double(), w.double()).float()).abs().max() < 1e-4
    # bfloat16 in whole 16-byte chunks: the tensor-core form; rows, columns and K that fill no tile
    for G, M, N, K in ((3, 70, 136, 72), (2, 1, 8, 8), (1, 200, 264, 40)):
        a16 = torch.randn(G, M, K, generator=g).to(torch.bfloat16).cuda()
        w16 = torch.randn(G, N, K, generator=g).to(torch.bfloat16).cuda()
        want = torch.einsum("gmk,gnk->gmn", a16.double(), w16.double())
        got = ops.gemm_batched(a16, w16).double()
        assert (got - want).abs().max() < 1e-2 * want.abs().max()
    # the same writing [M, G, N] through a view, every row times the sigmoid of its gate
    a16 = torch.randn(3, 70, 72, generator=g).to(torch.bfloat16).cuda()
    w16 = torch.randn(3, 40, 72, generator=g).to(torch.bfloat16).cuda()
    gate = torch.randn(70, 11, generator=g).to(torch.bfloat16).cuda()[:, 4:7]
    out = torch.empty(70, 3, 40, dtype=torch.bfloat16, device="cuda")
    ops.gemm_batched(a16, w16, out=out.transpose(0, 1), gate=gate)
    want = torch.einsum("gmk,gnk->mgn", a16.double(), w16.double()) * torch.sigmoid(gate.double())[:, :, None]
    assert (out.double() - want).abs().max() < 1e-2 * want.abs().max()
    # grouped, with gathered rows, zero rows and unused tiles
    for dtype, tile in ((torch.float32, 64), (torch.bfloat16, 64), (torch.bfloat16, 128)):
        x = torch.randn(50, 64, generator=g).to(torch.bfloat16).to(dtype).cuda()
        w3 = torch.randn(3, 72, 64, generator=g).to(torch.bfloat16).to(dtype).cuda()
        rows = 4 * tile
        row_index = torch.full((rows,), -1, dtype=torch.int32)
        row_index[:5] = torch.tensor([7, 7, 0, 49, 3])
        row_index[tile:tile + 2] = torch.tensor([1, 2])
        row_index[3 * tile:3 * tile + tile] = torch.arange(tile) % 50
        groups = torch.tensor([2, 0, -1, 1], dtype=torch.int32)
        got = ops.gemm_grouped(x, w3, groups.cuda(), row_index.cuda(), rows, act=True, tile=tile).double().cpu()
        for t, grp in enumerate(groups.tolist()):
            if grp < 0:
                continue
            idx = row_index[t * tile:(t + 1) * tile]
            src = torch.where(idx[:, None] >= 0, x.double().cpu()[idx.clamp(min=0).long()], torch.zeros(1, dtype=torch.float64))
            want = torch.relu(src @ w3[grp].double().cpu().T) ** 2
            assert (got[t * tile:(t + 1) * tile] - want).abs().max() < (1e-4 if dtype == torch.float32 else 2e-2) * want.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E, top, shared, T", [(6, 2, 48, 37), (5, 1, 0, 9), (4, 4, 16, 70), (40, 7, 8, 3),
                                               (3, 2, 0, 1), (9, 2, 16, 600)])      # the last: the library's grouped product
def test_routed_experts_alone(dtype, E, top, shared, T):
    from tokenomos_b200.parts.registry import Runtime, builder_of

    width, ff = 40, 24
    g = torch.Generator().manual_seed(E * 10 + top)
    bf = lambda t: t.to(torch.bfloat16)
    tensors = {"router": bf(torch.randn(E, width, generator=g) * 0.5)}
    for e in range(E):
        tensors[f"e{e}.up"] = bf(torch.randn(ff, width, generator=g) / math.sqrt(width))
        tensors[f"e{e}.down"] = bf(torch.randn(width, ff, generator=g) / math.sqrt(ff))
    if shared:
        tensors["shared_up"] = bf(torch.randn(shared, width, generator=g) / math.sqrt(width))
        tensors["shared_down"] = bf(torch.randn(width, shared, generator=g) / math.sqrt(shared))
        tensors["shared_gate"] = bf(torch.randn(1, width, generator=g) * 0.3)
    x = bf(torch.randn(T, width, generator=g))
    w = {"p." + k.replace("shared_gate", "shared.sg").replace("shared_up", "shared.up").replace(
        "shared_down", "shared.down"): v.double() for k, v in tensors.items()}
    f = {"router": {"experts": E, "top": top, "scale": 1.7}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_experts(x.double(), w, "p.", f)
    rt = Runtime(dtype, torch.device("cuda"))
    held = {k: (v.float() if k in ("router", "shared_gate") else v.to(dtype)).cuda() for k, v in tensors.items()}
    part = builder_of("feed_forward", "relu2_moe")({"experts": E, "top": top, "scale": 1.7}, held, rt)
    got = part.forward(x.to(dtype).cuda()).double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got - want).abs().max() < tol * want.abs().max()


@pytest.mark.gpu
def test_router_takes_the_lowest_index_of_equal_scores_and_stays_in_range():
    from tokenomos_b200 import ops

    z = torch.tensor([[1.0, 3.0, 3.0, 0.0, 3.0], [float("nan")] * 5, [-float("inf")] * 5], device="cuda")
    idx, w, gate = ops.moe_route(z, 4, 2, 2.0, True)
    assert idx[0].tolist() == [1, 2] and abs(w[0].sum().item() - 2.0) < 1e-6
    assert abs(gate[0].item() - 1 / (1 + math.exp(-3.0))) < 1e-6
    assert ((idx >= 0) & (idx < 4)).all()


# ---------------------------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------------------------

_oracle: dict = {}


def oracle(name, folders, reqs):
    if name not in _oracle:
        _, w = folders[name]
        _oracle[name] = {rid: plain.forward(CASES[name]["config"], w, ids)[0] for rid, ids in reqs.items()}
    return _oracle[name]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_way_of_cutting(name, dtype, folders):
    folder, _ = folders[name]
    page = CASES[name]["page"]
    reqs = requests_for(name)
    want = oracle(name, folders, reqs)
    results = {}
    for mode, steps in (("whole", trace_util.whole(reqs)),
                        ("tail", trace_util.tail_decoded(reqs, 48)),
                        ("portions", trace_util.portions(reqs)),
                        ("mixed", trace_util.mixed(reqs, live=4, seed=ord(name)))):
        # exactly the pages the trace's live requests need at its worst moment, all others and
        # every page and state row given back full of NaN
        max_tokens = trace_util.max_live_tokens(steps, page)
        per_step = trace_util.run_in_process(folder, dtype, steps, max_tokens, page, max_requests=4)
        got = trace_util.collect(steps, per_step)
        compare(got, want, (TOL_F32 if dtype == "float32" else TOL_BF16)[name], f"{name} {dtype} {mode}",
                close_calls=0.0 if dtype == "float32" else CLOSE_CALLS)
        results[mode] = got
    if dtype == "float32":
        for mode in ("tail", "portions", "mixed"):
            compare(results[mode], results["whole"], TOL_F32_SAME[name], f"{name} {dtype} {mode} vs whole")


def random_config(seed: int) -> tuple[dict, int]:
    """A configuration drawn from everything the design lets vary, and a page size."""
    import random

    rng = random.Random(seed)
    width = rng.choice([32, 40, 64, 96])
    layers = []
    for _ in range(rng.randint(1, 4)):
        rot_dim = rng.choice([2, 4, 8, 12, 16])
        layer = latent(rng.choice([1, 2, 3, 4, 6, 8]), rng.choice([4, 8, 12, 16, 24]), rot_dim,
                       rng.choice([4, 8, 12, 20]), rng.choice([8, 16, 24, 40]), rng.choice([8, 12, 16, 32, 64]),
                       rng.choice([None, 1, 2, 5, 16, 33, 100]), dims=rng.choice([rot_dim, rot_dim, 2]),
                       base=rng.choice([100.0, 10000.0, 500000.0]), scale=rng.choice([None, 0.05, 0.3]))
        kind = rng.random()
        if kind < 0.15:
            layer["mlp"] = None
        elif kind < 0.5:
            layer["mlp"] = dense(rng.choice([16, 24, 30, 64]))
        else:
            experts = rng.choice([2, 3, 5, 8, 17])
            layer["mlp"] = moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 20, 32]),
                               rng.choice([0.5, 1.0, 2.5]), shared=rng.choice([None, 8, 24]))
        layers.append(layer)
    config = {"architecture": "Laposun", "vocab": rng.randint(40, 300), "width": width,
              "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.85:
        config["streams"] = rng.choice([1, 2, 2, 3, 4])
    if rng.random() < 0.85:
        config["canon"] = {"taps": rng.choice([1, 2, 3, 4, 4, 6])}
    if rng.random() < 0.85:
        config["embedding"] = {"bigram": {"buckets": rng.choice([7, 101, 1000]), "mul_prev": rng.randint(1, 10 ** 6),
                                          "mul_cur": rng.randint(1, 10 ** 6)}}
    return config, rng.choice([4, 8, 16])


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(16))
def test_random_configurations(seed, tmp_path):
    """Configurations nobody chose: whatever the draw gives, the 32-bit model meets the plain
    implementation however the requests are cut, and the 16-bit one stays close to it."""
    from safetensors.torch import save_file

    config, page = random_config(seed)
    tensors = make_tensors(config, 200 + seed)
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    w = {k: v.double() for k, v in tensors.items()}
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([1, 2, 17, 45, 80, 130])}
    want = {rid: plain.forward(config, w, ids)[0] for rid, ids in reqs.items()}
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 0.25)):
        for steps in (trace_util.portions(reqs), trace_util.mixed(reqs, live=4, seed=seed)):
            per_step = trace_util.run_in_process(tmp_path, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                                 max_requests=4)
            # (a draw may have one expert per token out of many, and layers without a window that
            # carry a close call's other expert on to every later position: in bfloat16 half of a
            # request's positions must still lie within the bound, and all be finite)
            compare(trace_util.collect(steps, per_step), want, tol, f"random configuration {seed} {dtype}: {config}",
                    close_calls=0.0 if dtype == "float32" else 0.5)


def stream_sums(model, seen):
    """Wrap every block so that the sum of the streams after it (its last write applied) is kept."""
    for block in model.blocks:
        def wrapped(h, residual, pending, ctx, call, inner=block.forward):
            y, streams, writer = inner(h, residual, pending, ctx, call)
            S = writer.streams
            x = streams.view(streams.shape[0], S, -1).double()
            if writer.hc_mix is None:
                new = x + y.double()[:, None, :]
            else:
                new = (torch.einsum("st,nsw->ntw", writer.hc_mix.view(S, S).double(), x)
                       + writer.hc_out.double()[None, :, None] * y.double()[:, None, :])
            seen.append(new.sum(1).cpu())
            return y, streams, writer
        block.forward = wrapped


@pytest.mark.gpu
def test_layers_one_by_one(folders):
    """The sum of the streams after every layer, in 32-bit: a fault shows at the layer that has it."""
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    for name in ("A", "B", "C", "E"):
        folder, w = folders[name]
        ids = requests_for(name)["r3"]
        _, want = plain.forward(CASES[name]["config"], w, ids)
        conf = models.configure(folder, work="float32")
        model = models.load(folder, "cuda", conf)
        cache = CacheManager(model.state_specs(), 8, 40, 2, conf.work, "cuda", max_len=256, poison=True)
        seen = []
        stream_sums(model, seen)
        cache.admit("x")
        StepFunction(model, cache).run([StepEntry("x", ids, [0])])
        assert len(seen) == want.shape[0]
        for layer, (got, ref) in enumerate(zip(seen, want)):
            assert (got - ref).abs().max() <= 2e-5 * ref.abs().max(), (name, layer)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype, folders):
    """One and two token prompts, and 260 tokens decoded one by one: across many pages, far past
    every window."""
    for name in ("A", "E"):
        folder, w = folders[name]
        g = torch.Generator().manual_seed(99)
        vocab = CASES[name]["config"]["vocab"]
        reqs = {"one": torch.randint(0, vocab, (1,), generator=g).tolist(),
                "two": torch.randint(0, vocab, (2,), generator=g).tolist(),
                "long": torch.randint(0, vocab, (263,), generator=g).tolist()}
        want = {rid: plain.forward(CASES[name]["config"], w, ids)[0] for rid, ids in reqs.items()}
        steps = trace_util.tail_decoded(reqs, tail=260)
        page = CASES[name]["page"]
        per_step = trace_util.run_in_process(folder, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                             max_requests=4)
        compare(trace_util.collect(steps, per_step), want, (TOL_F32 if dtype == "float32" else TOL_BF16)[name],
                f"long decoding {name} {dtype}", close_calls=0.0 if dtype == "float32" else CLOSE_CALLS)


@pytest.mark.gpu
def test_a_wrong_window_a_lost_state_and_a_wrong_hash_show(folders, monkeypatch):
    """Negative controls: the same replay with a window one longer, without the convolution's
    state, without the previous token, or with the connection matrix read [to, from], is far
    outside the bound that the real model meets."""
    from tokenomos_b200 import ops
    from tokenomos_b200.parts import hyper as hyper_mod
    from tokenomos_b200.parts import latent as latent_mod

    name = "A"
    folder, _ = folders[name]
    reqs = {k: v for k, v in requests_for(name).items() if k in ("r3", "r4")}
    want = {rid: oracle(name, folders, requests_for(name))[rid] for rid in reqs}
    steps = trace_util.portions(reqs)
    page = CASES[name]["page"]

    def run():
        per_step = trace_util.run_in_process(folder, "float32", steps, trace_util.max_live_tokens(steps, page), page,
                                             poison=False)
        return trace_util.collect(steps, per_step)

    def worst(got):
        return max(((got[rid] - want[rid]).abs().max() / want[rid].abs().max()).item() for rid in reqs)

    compare(run(), want, TOL_F32[name], "control: the real model")
    real_init = latent_mod.LatentAttention.__init__

    def longer_window(self, *a, **kw):
        real_init(self, *a, **kw)
        if self.window == 9:
            self.window += 1
    monkeypatch.setattr(latent_mod.LatentAttention, "__init__", longer_window)
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(latent_mod.LatentAttention, "__init__", real_init)

    real_conv = ops.canon_conv

    def stateless(h, taps, state, cu, seq_ctx, *rest):
        return real_conv(h, taps, state, cu, torch.zeros_like(seq_ctx), *rest)
    monkeypatch.setattr(ops, "canon_conv", stateless)
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(ops, "canon_conv", real_conv)

    real_embed = ops.embed_bigram_norm

    def forgetful(table, bigram, norm_w, eps, ids, select, tok_seq, cu, seq_ctx, *rest):
        return real_embed(table, bigram, norm_w, eps, ids, select, tok_seq, cu, torch.zeros_like(seq_ctx), *rest)
    monkeypatch.setattr(ops, "embed_bigram_norm", forgetful)
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(ops, "embed_bigram_norm", real_embed)

    real_reader = hyper_mod.StreamReader.__init__

    def transposed(self, *a, **kw):
        real_reader(self, *a, **kw)
        if self.hc_mix is not None:
            self.hc_mix = self.hc_mix.view(self.streams, self.streams).t().contiguous().view(-1)
    monkeypatch.setattr(hyper_mod.StreamReader, "__init__", transposed)
    assert worst(run()) > 100 * TOL_F32[name]


# ---------------------------------------------------------------------------------------------
# the entry points: LLM.generate through the scheduler, the command line, the trace program
# ---------------------------------------------------------------------------------------------

def teacher_forced_ok(config, w, prompt, reply, margin, close_calls: int = 0):
    """Every token of ``reply`` is the plain implementation's best, or within ``margin`` of it, but
    for ``close_calls`` tokens (16-bit runs only: a router's close call)."""
    logits, _ = plain.forward(config, w, prompt + reply)
    missed = 0
    for i, tok in enumerate(reply):
        row = logits[len(prompt) + i - 1]
        if int(row.argmax()) != tok and row.max().item() - row[tok].item() > margin:
            missed += 1
    assert missed <= close_calls, (missed, close_calls)


@pytest.mark.gpu
@pytest.mark.parametrize("name, work, graphs", [("A", "fp32", False), ("B", "fp32", True), ("E", "bf16", True),
                                                ("D", "fp32", True), ("E", "fp32", False)])
def test_greedy_generation_through_llm(name, work, graphs, folders):
    from tokenomos_b200 import LLM, SamplingParams

    folder, w = folders[name]
    config = CASES[name]["config"]
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in (1, 9, 40, 64, 23)]
    steps = 40
    with LLM(str(folder), work=work, page=CASES[name]["page"], max_len=256, slots=4, pages=120,
             prefill_budget=48, poison=True, graphs=graphs) as llm:
        outs = llm.generate(prompts, SamplingParams(max_tokens=steps))
    for prompt, out in zip(prompts, outs):
        assert out.prompt_tokens == len(prompt) and len(out.token_ids) == steps
        teacher_forced_ok(config, w, prompt, out.token_ids, 1e-3 if work == "fp32" else 0.3,
                          close_calls=0 if work == "fp32" else 6)


@pytest.mark.gpu
def test_trace_program_and_command_line(folders, tmp_path):
    name = "A"
    folder, _ = folders[name]
    reqs = requests_for(name)
    want = oracle(name, folders, reqs)
    steps = trace_util.mixed(reqs, live=4, seed=3)
    per_step = trace_util.run_program(folder, "float32", steps, trace_util.max_live_tokens(steps, 64), tmp_path,
                                      CASES[name]["config"]["vocab"])
    compare(trace_util.collect(steps, per_step), want, TOL_F32[name], "trace program")
    cmd = [sys.executable, "-m", "tokenomos_b200.generate", "--model", str(folder), "--prompt-ids", "1,2,3,4",
           "--max-tokens", "5", "--arch-kw", '{"work": "fp32"}',
           "--engine-kw", '{"page": 4, "max_len": 64, "slots": 2, "pages": 40}']
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1 and len(lines[0]["token_ids"]) == 5
    teacher_forced_ok(CASES[name]["config"], folders[name][1], [1, 2, 3, 4], lines[0]["token_ids"], 1e-3)
