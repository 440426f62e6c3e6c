"""The Darizen decoder as a declaration: configuration -> ``ModelSpec``.

A pre-norm decoder whose residual stream, norms, rotations and softmax are 32-bit whatever the
storage type. Every layer is ``x += mixer(norm1(x)); x += ff(norm2(x))`` with RMS norms whose
weights are stored around zero (``1 + w``), one of two attention mixers and a feed-forward (or
none):

- ``attention``: grouped-query attention whose values are its keys as projected (no value
  projection, no biases), interleaved rotary pairs with YaRN-scaled frequencies, a sliding
  window, a softmax with one added to its denominator, an element-wise sigmoid output gate;
- ``attention_2``: the same with a value projection of its own (``vdim``), biases on q, k and v,
  rotate-half pairs with linearly scaled frequencies, and a window that keeps the first
  ``keep_first`` positions of a sequence;
- feed-forward: ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit, limit)``,
  ``down(g * sigmoid(1.702 g) * (u + 1))``, all three projections with biases.

The layers ``loop.start .. loop.stop-1`` run ``loop.times`` times in a row with the same
weights, each pass with a cache of its own: the layer list names their blocks once per pass.
Pass ``t`` first adds the embedding output (``t > 0`` only) and row ``t`` of ``loop.step`` to
the stream. Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|g|o``
(biases ``.b``), ``l<i>.mlp.gate|up|down`` (biases ``.b``), ``final.norm``, ``head``.
"""

from __future__ import annotations

from tokenomos_b200.config.darizen import DarizenConfig
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_MATRIX, ROLE_VECTOR, BlockSpec, LayerCall,
                                       ModelSpec, PartSpec, StreamAdd, TensorDecl)

# constants the design fixes
GLU_ALPHA = 1.702        # the sigmoid's slope in the feed-forward's activation
GLU_SHIFT = 1.0          # added to the clamped up branch
NORM_OFFSET = 1.0        # norm weights are stored around zero


class Darizen:
    names = ("Darizen",)
    config_class = DarizenConfig

    def declare(self, cfg: DarizenConfig, tensor_names=()) -> ModelSpec:
        d = cfg.width

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm32", {"eps": cfg.norm_eps, "offset": NORM_OFFSET},
                            {"weight": TensorDecl(name, (d,), ROLE_VECTOR)})

        blocks = []
        for i, layer in enumerate(cfg.layers):
            m, p = layer.mixer, f"l{i}."
            second = m.kind == "attention_2"
            a = p + "mix."
            tensors = {
                "q": TensorDecl(a + "q", (m.heads * m.dim, d)),
                "k": TensorDecl(a + "k", (m.kv_heads * m.dim, d)),
                "gate": TensorDecl(a + "g", (m.heads * m.vdim, d)),
                "o": TensorDecl(a + "o", (d, m.heads * m.vdim)),
            }
            if second:
                tensors["v"] = TensorDecl(a + "v", (m.kv_heads * m.vdim, d))
                tensors["q_bias"] = TensorDecl(a + "q.b", (m.heads * m.dim,), ROLE_VECTOR)
                tensors["k_bias"] = TensorDecl(a + "k.b", (m.kv_heads * m.dim,), ROLE_VECTOR)
                tensors["v_bias"] = TensorDecl(a + "v.b", (m.kv_heads * m.vdim,), ROLE_VECTOR)
            mixer = PartSpec("attention", {
                "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
                "v_is_k": not second, "scale": m.scale, "window": m.window, "keep_first": m.keep_first,
                "sink": True, "gate_kind": "element", "exact": True,
                "position": {"kind": "rotary", "params": {
                    "head_dim": m.dim, "dims": m.rot.dims, "base": m.rot.base,
                    "layout": "half" if second else "interleaved", "scaling": m.rot.scaling}},
            }, tensors)
            ffn = None
            if layer.mlp is not None:
                f, ff = p + "mlp.", layer.mlp.ff
                ffn = PartSpec("glu_clamped", {"limit": layer.mlp.limit, "alpha": GLU_ALPHA, "shift": GLU_SHIFT}, {
                    "gate": TensorDecl(f + "gate", (ff, d)),
                    "gate_bias": TensorDecl(f + "gate.b", (ff,), ROLE_VECTOR),
                    "up": TensorDecl(f + "up", (ff, d)),
                    "up_bias": TensorDecl(f + "up.b", (ff,), ROLE_VECTOR),
                    "down": TensorDecl(f + "down", (d, ff)),
                    "down_bias": TensorDecl(f + "down.b", (d,), ROLE_VECTOR),
                })
            blocks.append(BlockSpec("prenorm", {
                "mixer": mixer,
                "ffn": ffn,
                "pre_mixer_norm": norm(p + "norm1"),
                "pre_ffn_norm": norm(p + "norm2") if ffn is not None else None,
            }))

        n = len(blocks)
        # a folder may store the second norm of a layer that has no feed-forward: nothing reads it
        unused = tuple((f"unused.l{i}.norm2", TensorDecl(f"l{i}.norm2", (d,), ROLE_VECTOR, optional=True))
                       for i, layer in enumerate(cfg.layers) if layer.mlp is None)
        order, extras = [], ()
        if cfg.loop is None:
            order = [LayerCall(i) for i in range(n)]
        else:
            lp = cfg.loop
            extras = (("loop_step", TensorDecl("loop.step", (lp.times, d), ROLE_VECTOR)),)
            order = [LayerCall(i) for i in range(lp.start)]
            for t in range(lp.times):
                for i in range(lp.start, lp.stop):
                    opens = StreamAdd(embedding=t > 0, tensor="loop_step", row=t) if i == lp.start else None
                    order.append(LayerCall(i, add=opens))
            order += [LayerCall(i) for i in range(lp.stop, n)]
        return ModelSpec(
            width=d,
            vocab=cfg.vocab,
            embedding=TensorDecl("embed", (cfg.vocab, d), ROLE_EMBEDDING),
            blocks=tuple(blocks),
            order=tuple(order),
            final_norm=norm("final.norm"),
            head=TensorDecl("head", (cfg.vocab, d), ROLE_MATRIX),
            extras=extras + unused,
        )
