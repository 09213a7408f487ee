"""The Zikupel decoder put together from parts.

Layer i: the mixer reads the residual stream itself; its output passes through an RMS norm whose stored weight lies
around zero (the norm multiplies by 1 + w) and is added; then, unless the layer has no feed-forward, the same with
the feed-forward:  x += N1(mixer(x)),  x += N2(ff(x)).  That is the package's ``SandwichBlock`` with no norm on the
way in (``PassNorm``).  Mixers: softmax attention with normed queries and keys, values that are the keys, partial
rotary positions with stretched frequencies, capped scores and an output gate (``QKNormAttention``), or linear
attention with a decay per head and a state per request (``DecayLinearAttention``).  Feed-forwards: the dense gated
one, or routed experts without a gate (relu squared, sigmoid scores that multiply the experts' inputs, a shared
expert).  Embedding, a last norm of the same kind, an untied head.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.<q|q.b|k|k.b|q.norm|k.norm|g|o>`` or
``l<i>.mix.<q|k|v|g|o|norm>``, ``l<i>.mlp.<gate|up|down>`` or ``l<i>.mlp.<router|e<k>.up|e<k>.down|shared.up|shared.down>``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zikupel import ZikupelConfig
from ..parts import (DecayLinearAttention, GatedMLP, OutputHead, PassNorm, QKNormAttention, RMSNorm, RoutedExperts,
                     SandwichBlock, TokenEmbedding, YarnRotary)
from .decoder import Binding, DecoderModel, LayerCall


def build_zikupel(cfg: ZikupelConfig) -> DecoderModel:
    D, eps = cfg.width, cfg.norm_eps
    embed = TokenEmbedding(cfg.vocab, D)
    bindings = [Binding(embed, {"weight": "embed"})]
    blocks, order = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "attention":
            s = m.rot.scaling
            position = YarnRotary(m.dim, m.rot.base, m.rot.dims, factor=None if s is None else s.factor,
                                  original=0 if s is None else s.original, fast=1.0 if s is None else s.fast,
                                  slow=1.0 if s is None else s.slow)
            mixer = QKNormAttention(D, m.heads, m.kv_heads, m.dim, position, eps, scale=m.scale, softcap=m.softcap,
                                    qk_norm=True, qk_bias=True, values_from_keys=True, gate=True)
            names = {"q.weight": p + "mix.q", "q.bias": p + "mix.q.b", "k.weight": p + "mix.k", "k.bias": p + "mix.k.b",
                     "q.norm": p + "mix.q.norm", "k.norm": p + "mix.k.norm", "g.weight": p + "mix.g", "o.weight": p + "mix.o"}
        else:
            mixer = DecayLinearAttention(D, m.heads, m.dim, m.vdim, m.decay, eps, act="silu", gate=True)
            names = {"q.weight": p + "mix.q", "k.weight": p + "mix.k", "v.weight": p + "mix.v", "g.weight": p + "mix.g",
                     "norm": p + "mix.norm", "o.weight": p + "mix.o"}
        norm1 = RMSNorm(D, eps, one_plus=True)
        bindings += [Binding(mixer, names), Binding(norm1, {"weight": p + "norm1"})]
        pass2 = ff = norm2 = None
        if layer.mlp is not None:
            pass2, norm2 = PassNorm(D), RMSNorm(D, eps, one_plus=True)
            if layer.mlp.kind == "dense":
                ff = GatedMLP(D, layer.mlp.ff, "silu")
                ff_names = {f"{n}.weight": f"{p}mlp.{n}" for n in ("gate", "up", "down")}
            else:
                f = layer.mlp
                ff = RoutedExperts(D, f.ff, f.experts, f.top, act="relu2", router_bias=False, gated=False,
                                   scoring="sigmoid", weight_on="input", shared_inner=f.shared_ff)
                ff_names = {"router.weight": p + "mlp.router"}
                for e in range(f.experts):
                    ff_names.update({f"e{e}.{n}.weight": f"{p}mlp.e{e}.{n}" for n in ("up", "down")})
                if f.shared_ff:
                    ff_names.update({f"shared.{n}.weight": f"{p}mlp.shared.{n}" for n in ("up", "down")})
            bindings += [Binding(ff, ff_names), Binding(norm2, {"weight": p + "norm2"})]
        blocks.append(SandwichBlock(PassNorm(D), mixer, norm1, pass2, ff, norm2))
        order.append(LayerCall(block=i, cache=i))
    final_norm = RMSNorm(D, eps, one_plus=True)
    head = OutputHead(cfg.vocab, D)
    bindings += [Binding(final_norm, {"weight": "final.norm"}), Binding(head, {"weight": "head"})]
    return DecoderModel(cfg, embed, blocks, order, final_norm, head, bindings)
