"""The Zapipel decoder put together from parts.

Layer i: centred norm -> latent attention (with an output gate per head, no position encoding) -> centred norm
of the mixer's output -> add; then, unless the layer has no feed-forward, centred norm -> dense gated
feed-forward or routed experts -> centred norm -> add.  A layer with ``kv_from`` reads the cache entry of the
layer it names.  Embedding, last centred norm, an untied head whose logits are scaled and soft-capped.
Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.<dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o>``,
``l<i>.mlp.<gate|up|down>`` or ``l<i>.mlp.<router|router.b|e<k>.gate|e<k>.up|e<k>.down>``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zapipel import ZapipelConfig
from ..parts import (CentredNorm, GatedMLP, LatentAttention, OutputHead, RoutedExperts, SandwichBlock, TokenEmbedding)
from .decoder import Binding, DecoderModel, LayerCall


def build_zapipel(cfg: ZapipelConfig) -> DecoderModel:
    D, eps = cfg.width, cfg.norm_eps
    embed = TokenEmbedding(cfg.vocab, D)
    bindings = [Binding(embed, {"weight": "embed"})]
    blocks, order = [], []
    entry_of = {}                      # layer that keeps latents -> its cache entry
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        own = m.kv_from is None
        mixer = LatentAttention(D, m.heads, m.dim, m.vdim, m.q_rank, m.kv_rank, m.scale, eps, own_latent=own)
        names = {"dq.weight": p + "mix.dq", "dq.norm": p + "mix.dq.norm", "uq.weight": p + "mix.uq",
                 "uk.weight": p + "mix.uk", "uv.weight": p + "mix.uv", "g.weight": p + "mix.g", "o.weight": p + "mix.o"}
        if own:
            names.update({"dkv.weight": p + "mix.dkv", "dkv.norm": p + "mix.dkv.norm"})
            entry_of[i] = len(entry_of)
        norm1, norm1b = CentredNorm(D, eps), CentredNorm(D, eps)
        bindings += [Binding(norm1, {"weight": p + "norm1"}), Binding(mixer, names), Binding(norm1b, {"weight": p + "norm1b"})]
        norm2 = ff = norm2b = None
        if layer.mlp is not None:
            norm2, norm2b = CentredNorm(D, eps), CentredNorm(D, eps)
            if layer.mlp.kind == "dense":
                ff = GatedMLP(D, layer.mlp.ff, "silu")
                ff_names = {f"{n}.weight": f"{p}mlp.{n}" for n in ("gate", "up", "down")}
            else:
                ff = RoutedExperts(D, layer.mlp.ff, layer.mlp.experts, layer.mlp.top)
                ff_names = {"router.weight": p + "mlp.router", "router.bias": p + "mlp.router.b"}
                for e in range(layer.mlp.experts):
                    ff_names.update({f"e{e}.{n}.weight": f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")})
            bindings += [Binding(norm2, {"weight": p + "norm2"}), Binding(ff, ff_names),
                         Binding(norm2b, {"weight": p + "norm2b"})]
        blocks.append(SandwichBlock(norm1, mixer, norm1b, norm2, ff, norm2b))
        order.append(LayerCall(block=i, cache=entry_of[i if own else m.kv_from], store=own))
    final_norm = CentredNorm(D, eps)
    head = OutputHead(cfg.vocab, D, logit_scale=cfg.logit_scale, softcap=cfg.logit_softcap)
    bindings += [Binding(final_norm, {"weight": "final.norm"}), Binding(head, {"weight": "head"})]
    return DecoderModel(cfg, embed, blocks, order, final_norm, head, bindings)
