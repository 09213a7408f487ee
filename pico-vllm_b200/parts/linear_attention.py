"""Linear attention with one decay per head: a mixer whose memory is a matrix of fixed size per request.

For a token with mixer input h, H heads, key size d and value size d_v:

    q = act(W_q h), k = act(W_k h), v = act(W_v h)            (act = silu; heads side by side)
    per head a:  S_a <- decay_a * S_a + k_a v_a^T ,   o_a = S_a^T q_a          (S_a: [d, d_v], zero at a request's start)
    out = W_o ( rms(concat_a o_a) * w_norm * sigmoid(W_g h) )

The state lives in float32 in a fixed-size slot of the cache manager (``FixedState``; zeroed when a request is admitted)
and is carried from step to step: a prompt portion continues where the portion before stopped, a decoded token is a
portion of one.  Nothing depends on how a request is cut or on what else is in the batch.  The recurrence, its inputs'
activation, the norm and the gate are float32.

Launches: one product for q, k, v and the gate logits -> the recurrence (one kernel over all segments) -> norm and gate
(one kernel) -> output product.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from ..errors import ConfigError
from .attention import _linear
from .base import CacheView, FixedState, Param, Part, Piece
from .registry import register

_ACTS = {"none": 0, "silu": 1}


@register("mixer", "decay_linear_attention")
class DecayLinearAttention(Part):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float, act: str = "silu",
                 gate: bool = True):
        if len(decay) != heads:
            raise ConfigError(f"decay_linear_attention: {len(decay)} decays for {heads} heads")
        if act not in _ACTS:
            raise ConfigError(f"decay_linear_attention: activation {act!r} is not built (have {sorted(_ACTS)})")
        if dim > 256:
            raise ConfigError(f"decay_linear_attention: key size {dim} above 256 is not built")
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.decay_values, self.eps, self.act, self.has_gate = [float(a) for a in decay], float(eps), _ACTS[act], gate
        self.proj_weight = self.out_norm = self.o_weight = self.decay = None

    def params(self) -> List[Param]:
        qk, v = self.heads * self.dim, self.heads * self.vdim
        proj = [Piece("q.weight", (qk, self.width)), Piece("k.weight", (qk, self.width)), Piece("v.weight", (v, self.width))]
        if self.has_gate:
            proj.append(Piece("g.weight", (v, self.width)))
        return [Param("proj_weight", tuple(proj)),
                Param("out_norm", (Piece("norm", (v,)),), kind="vector", init="one_plus_normal"),
                Param("o_weight", (Piece("o.weight", (self.width, v)),))]

    def cache_spec(self):
        return FixedState((self.heads, self.vdim, self.dim), "float32")      # S transposed: a column of S is contiguous

    def materialize(self, device, dtype):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def forward(self, h: torch.Tensor, batch, cache: CacheView) -> torch.Tensor:
        H, d, dv = self.heads, self.dim, self.vdim
        proj = _linear(h, self.proj_weight)                      # [T, q | k | v | (gate logits)]
        o = ops.decay_linear_attention(proj, 0, H * d, 2 * H * d, self.decay, cache.state, batch.seg_slots, batch.cu_q,
                                       batch.positions, H, d, dv, self.act, max_q_len=max(batch.q_lens, default=1))
        g0 = 2 * H * d + H * dv
        y = ops.gated_rms_norm(o, self.out_norm, proj[:, g0:g0 + H * dv] if self.has_gate else None, self.eps, h.dtype)
        return _linear(y, self.o_weight)
