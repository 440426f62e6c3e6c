"""The Laposun decoder as a declaration: configuration -> ``ModelSpec``.

A pre-norm decoder whose residual stream is carried in ``streams`` copies joined by
hyper-connections, in 32-bit:

- embedding: ``norm(embed[token] + bigram[(previous * mul_prev + token * mul_cur) mod buckets])``
  (the bigram table's last row for a sequence's first token), copied into every stream;
- every sublayer reads ``u = sum_s in[s] x_s``, norms it, adds a short causal convolution over
  time (``h + conv(h)``, ``canon.taps`` taps per channel), and writes ``x_t <- sum_s mix[s, t] x_s +
  out[t] y``;
- mixer ``latent_attention``: queries through a normed latent, keys and values from one normed
  latent per position plus a rotated key part shared by the heads, interleaved rotary pairs, a
  sliding window, a per-head sigmoid output gate;
- feed-forward: SwiGLU, or a mixture of experts (softmax router, ``top`` experts with
  renormalised scores times ``router.scale``, experts ``down(relu(up h)^2)``, a shared expert
  behind a sigmoid gate), or none;
- output: the norm of the streams' sum, logits with the embedding table.

Tensor names: ``embed``, ``bigram``, ``embed.norm``, ``final.norm``, and per layer ``l<i>.``:
``norm1|norm2``, ``hc1|hc2.in|out|mix``, ``canon1|canon2``, ``mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``,
``mlp.gate|up|down`` or ``mlp.router``, ``mlp.e<k>.up|down``, ``mlp.shared.up|down|sg``.
"""

from __future__ import annotations

from tokenomos_b200.config.laposun import LaposunConfig
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_IDENTITY, ROLE_NORM, ROLE_VECTOR, BlockSpec, LayerCall,
                                       ModelSpec, PartSpec, TensorDecl)


class Laposun:
    names = ("Laposun",)
    config_class = LaposunConfig

    def declare(self, cfg: LaposunConfig, tensor_names=()) -> ModelSpec:
        d = cfg.width
        S = cfg.streams or 1

        def reader(p: str, q: int) -> PartSpec:
            tensors = {"weight": TensorDecl(f"{p}norm{q}", (d,), ROLE_NORM)}
            if cfg.streams is not None:
                # (roles: what the random-weights mode draws is the plain residual stream, not zeros)
                tensors["in"] = TensorDecl(f"{p}hc{q}.in", (S,), ROLE_NORM)
                tensors["out"] = TensorDecl(f"{p}hc{q}.out", (S,), ROLE_NORM)
                tensors["mix"] = TensorDecl(f"{p}hc{q}.mix", (S, S), ROLE_IDENTITY)
            if cfg.taps is not None:
                tensors["taps"] = TensorDecl(f"{p}canon{q}", (d, cfg.taps), ROLE_VECTOR)
            return PartSpec("hyper_norm", {"eps": cfg.norm_eps, "streams": S}, tensors)

        blocks = []
        for i, layer in enumerate(cfg.layers):
            m, p = layer.mixer, f"l{i}."
            a = p + "mix."
            mixer = PartSpec("latent_attention", {
                "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim, "q_rank": m.q_rank,
                "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window, "eps": cfg.norm_eps,
                "rot": {"base": m.rot_base, "dims": m.rot_dims},
            }, {
                "dq": TensorDecl(a + "dq", (m.q_rank, d)),
                "dq_norm": TensorDecl(a + "dq.norm", (m.q_rank,), ROLE_NORM),
                "uq": TensorDecl(a + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                "dkv": TensorDecl(a + "dkv", (m.kv_rank + m.rot_dim, d)),
                "dkv_norm": TensorDecl(a + "dkv.norm", (m.kv_rank,), ROLE_NORM),
                "uk": TensorDecl(a + "uk", (m.heads * m.dim, m.kv_rank)),
                "uv": TensorDecl(a + "uv", (m.heads * m.vdim, m.kv_rank)),
                "gate": TensorDecl(a + "g", (m.heads, d)),
                "o": TensorDecl(a + "o", (d, m.heads * m.vdim)),
            })
            ffn = None
            f = layer.mlp
            if f is not None and f.kind == "dense":
                ffn = PartSpec("swiglu", {}, {
                    "gate": TensorDecl(p + "mlp.gate", (f.ff, d)),
                    "up": TensorDecl(p + "mlp.up", (f.ff, d)),
                    "down": TensorDecl(p + "mlp.down", (d, f.ff)),
                })
            elif f is not None:
                tensors = {"router": TensorDecl(p + "mlp.router", (f.experts, d), ROLE_VECTOR)}
                for k in range(f.experts):
                    tensors[f"e{k}.up"] = TensorDecl(f"{p}mlp.e{k}.up", (f.ff, d))
                    tensors[f"e{k}.down"] = TensorDecl(f"{p}mlp.e{k}.down", (d, f.ff))
                if f.shared_ff:
                    tensors["shared_up"] = TensorDecl(p + "mlp.shared.up", (f.shared_ff, d))
                    tensors["shared_down"] = TensorDecl(p + "mlp.shared.down", (d, f.shared_ff))
                    tensors["shared_gate"] = TensorDecl(p + "mlp.shared.sg", (1, d), ROLE_VECTOR)
                ffn = PartSpec("relu2_moe", {"experts": f.experts, "top": f.top, "scale": f.scale}, tensors)
            blocks.append(BlockSpec("hyper", {
                "mixer": mixer,
                "ffn": ffn,
                "pre_mixer_norm": reader(p, 1),
                "pre_ffn_norm": reader(p, 2) if ffn is not None else None,
            }))

        # a folder may store the second reader of a layer without a feed-forward: nothing reads it
        unused = []
        for i, layer in enumerate(cfg.layers):
            if layer.mlp is None:
                for role, decl in reader(f"l{i}.", 2).tensors.items():
                    unused.append((f"unused.l{i}.{role}", TensorDecl(decl.name, decl.shape, decl.role, optional=True)))
        table = TensorDecl("embed", (cfg.vocab, d), ROLE_EMBEDDING)
        embed_tensors = {"table": table, "norm": TensorDecl("embed.norm", (d,), ROLE_NORM)}
        params = {"eps": cfg.norm_eps, "copies": S}
        if cfg.bigram is not None:
            b = cfg.bigram
            embed_tensors["bigram"] = TensorDecl("bigram", (b.buckets + 1, d), ROLE_EMBEDDING)
            params.update(buckets=b.buckets, mul_prev=b.mul_prev, mul_cur=b.mul_cur)
        return ModelSpec(
            width=d,
            vocab=cfg.vocab,
            embedding=table,
            blocks=tuple(blocks),
            order=tuple(LayerCall(i) for i in range(len(blocks))),
            final_norm=PartSpec("hyper_norm", {"eps": cfg.norm_eps, "streams": S},
                                {"weight": TensorDecl("final.norm", (d,), ROLE_NORM)}),
            head=None,
            extras=tuple(unused),
            embedder=PartSpec("bigram_hash", params, embed_tensors),
        )
