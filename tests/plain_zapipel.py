"""A plain, slow restatement of the Zapipel decoder in torch on the CPU: one function per mechanism,
written from the equations and sharing nothing with the package.  Everything runs in the dtype of the
tensors it is given (float64 in the tests).

Notation: x [T, D] residual stream; a layer is  x += N1b(mixer(N1(x))),  x += N2b(ff(N2(x)))  with
N(u) = (u - mean u) / sqrt(var u + eps) * w.  The mixer keeps one latent c_t [R] per token; keys and
values of head a are U_k[a] c_t and U_v[a] c_t.
"""
import torch


def layer_norm(u, w, eps):
    m = u.mean(-1, keepdim=True)
    d = u - m
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms_norm(u, w, eps):
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def latent_of(h, w_dkv, w_norm, eps):
    """The latent c [T, R] a layer caches for its tokens."""
    return rms_norm(h @ w_dkv.T, w_norm, eps)


def latent_attention(h, latents, start, p, heads, dim, vdim, scale, eps):
    """h [T, D]: the mixer's input for positions start .. start+T-1 of one sequence; latents [start+T, R]:
    the latents of positions 0 .. start+T-1 (this layer's own or another layer's).  p: the mixer's tensors
    by their short names.  Returns [T, D]."""
    T = h.shape[0]
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).view(T, heads, dim)
    k = (latents @ p["uk"].T).view(-1, heads, dim)
    v = (latents @ p["uv"].T).view(-1, heads, vdim)
    gate = torch.sigmoid(h @ p["g"].T)                       # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        n = start + t + 1                                    # keys 0 .. start+t are visible
        for a in range(heads):
            s = (k[:n, a] @ q[t, a]) * scale
            w = torch.softmax(s, dim=0)
            out[t, a] = (w[:, None] * v[:n, a]).sum(0) * gate[t, a]
    return out.reshape(T, heads * vdim) @ p["o"].T


def dense_ff(h, p):
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def route(h, w_router, b_router, top):
    """Chosen experts [T, top] and their weights [T, top]: softmax over the chosen logits only."""
    z = h @ w_router.T + b_router
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def route_margin(h, w_router, b_router, top):
    """How far each token is from another choice of experts: (smallest chosen logit - largest logit not chosen)
    over the largest |logit|; infinite when every expert is chosen."""
    z = h @ w_router.T + b_router
    val, _ = torch.sort(z, dim=-1, descending=True)
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], float("inf"), dtype=z.dtype)
    return (val[:, top - 1] - val[:, top]) / z.abs().amax(-1)


def moe_ff(h, p, experts, top):
    idx, wgt = route(h, p["router"], p["router.b"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            pe = {n: p[f"e{e}.{n}"] for n in ("gate", "up", "down")}
            out[t] += wgt[t, j] * dense_ff(h[t:t + 1], pe)[0]
    return out


def head_logits(x, w_norm, w_head, eps, logit_scale, softcap):
    y = layer_norm(x, w_norm, eps) @ w_head.T * logit_scale
    return y if softcap is None else softcap * torch.tanh(y / softcap)


def _sub(tensors, prefix):
    return {n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)}


class PlainZapipel:
    """The whole model over explicit per-sequence lists of latents (no pages, no batches)."""

    def __init__(self, config: dict, tensors: dict, dtype=torch.float64):
        self.cfg = config
        self.t = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.dtype = dtype

    def new_state(self):
        return {"len": 0, "latents": {}, "margin": []}        # latents: layer index -> [len, R]; margin: per position

    def forward(self, state, tokens, keep_layers=False):
        """Feeds the next tokens of one sequence; returns logits [T, vocab] (and, on request, the residual
        stream after every layer)."""
        cfg, t, eps = self.cfg, self.t, self.eps
        x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        start = state["len"]
        after = []
        margin = torch.full((len(tokens),), float("inf"), dtype=self.dtype)
        for i, layer in enumerate(cfg["layers"]):
            assert layer["type"] == "latent_attention"
            m = layer["mixer"]
            pre = f"l{i}."
            h = layer_norm(x, t[pre + "norm1"], eps)
            p = _sub(t, pre + "mix.")
            src = m.get("kv_from")
            if src is None:
                c = latent_of(h, p["dkv"], p["dkv.norm"], eps)
                old = state["latents"].get(i)
                state["latents"][i] = c if old is None else torch.cat([old, c], 0)
                src = i
            y = latent_attention(h, state["latents"][src], start, p, m["heads"], m["dim"], m["vdim"],
                                 float(m["scale"]), eps)
            x = x + layer_norm(y, t[pre + "norm1b"], eps)
            ff = layer.get("mlp")
            if ff is not None:
                h = layer_norm(x, t[pre + "norm2"], eps)
                pf = _sub(t, pre + "mlp.")
                if ff["kind"] == "dense":
                    y = dense_ff(h, pf)
                else:
                    y = moe_ff(h, pf, ff["router"]["experts"], ff["router"]["top"])
                    margin = torch.minimum(margin, route_margin(h, pf["router"], pf["router.b"], ff["router"]["top"]))
                x = x + layer_norm(y, t[pre + "norm2b"], eps)
            after.append(x.clone())
        state["len"] = start + len(tokens)
        state["margin"] += margin.tolist()
        logits = head_logits(x, t["final.norm"], t["head"], eps, float(cfg.get("logit_scale", 1.0)), cfg.get("logit_softcap"))
        return (logits, after) if keep_layers else logits

    def greedy(self, prompt, n_new):
        state = self.new_state()
        out = []
        logits = self.forward(state, list(prompt))
        for _ in range(n_new):
            tok = int(torch.argmax(logits[-1]))
            out.append(tok)
            logits = self.forward(state, [tok])
        return out

