"""A plain, slow restatement of the Zikupel decoder in torch on the CPU: one function per mechanism,
written from the equations and sharing nothing with the package.  Everything runs in the dtype of the
tensors it is given (float64 in the tests).

Notation: x [T, D] residual stream.  A layer is  x += N1(mixer(x)),  x += N2(ff(x))  with
N(u) = u / sqrt(mean u^2 + eps) * (1 + w): the sublayers read x itself and only their outputs are normed.
Two mixers: softmax attention over grouped heads whose values are the un-normed, un-rotated keys, and a linear
attention with one decay per head whose state S [dim, vdim] is carried from token to token.
A sequence's memory is a plain dictionary per layer: lists of keys and values, or the state.
"""
import math

import torch


def rms(u, eps):
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def norm_one_plus(u, w, eps):
    return rms(u, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def relu2(z):
    return torch.relu(z) ** 2


# ----------------------------------------------------------------------------------------------------- rotary
def yarn_frequencies(dims, base, scaling, dtype=torch.float64):
    """Frequencies [dims/2] and the factor on cos and sin.  ``scaling``: None, or a dictionary with factor,
    original, fast, slow: dimensions that turn more than ``fast`` times within ``original`` positions keep their
    frequency, those that turn fewer than ``slow`` times get it divided by ``factor``, with a linear ramp between."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if scaling is None:
        return f, 1.0

    def dim_of(turns):
        return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    f = f / scaling["factor"] * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(scaling["factor"]) + 1.0


def rotate(u, positions, freqs, mult, dims):
    """u [T, heads, dim]: the first ``dims`` dimensions of every head turn, dimension i with i + dims/2."""
    ang = positions.to(u.dtype)[:, None] * freqs[None, :]           # [T, dims/2]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    a, b = u[..., :dims // 2], u[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, u[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------------------------------- mixers
def softmax_attention(h, mem, start, p, m, eps):
    """h [T, D]: positions start .. start+T-1 of one sequence.  mem: {"k": list of [G, dim], "v": the same} for the
    positions before ``start``; the new tokens' keys and values are appended.  p: the mixer's tensors by short name;
    m: its sizes and constants (heads, kv_heads, dim, vdim, scale, softcap, rot{base, dims, scaling})."""
    T, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    k_raw = (h @ p["k"].T + p["k.b"]).view(T, G, d)
    q = rms(q, eps) * p["q.norm"]
    k = rms(k_raw, eps) * p["k.norm"]
    rot = m["rot"]
    freqs, mult = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
    pos = torch.arange(start, start + T)
    q, k = rotate(q, pos, freqs, mult, rot["dims"]), rotate(k, pos, freqs, mult, rot["dims"])
    for t in range(T):
        mem["k"].append(k[t])
        mem["v"].append(k_raw[t])            # the values are the keys as projected
    K, V = torch.stack(mem["k"]), torch.stack(mem["v"])            # [n, G, d]
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        n = start + t + 1
        for a in range(H):
            g = a // (H // G)
            s = (K[:n, g] @ q[t, a]) * m["scale"]
            if m.get("softcap"):
                s = m["softcap"] * torch.tanh(s / m["softcap"])
            w = torch.softmax(s, dim=0)
            out[t, a] = (w[:, None] * V[:n, g]).sum(0)
    gate = torch.sigmoid(h @ p["g"].T)
    return (out.reshape(T, H * d) * gate) @ p["o"].T


def linear_attention(h, mem, p, m, eps):
    """mem: {"S": [heads, dim, vdim]} the state after the tokens before (zeros at the start), updated in place."""
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].T).view(T, H, d)
    k = silu(h @ p["k"].T).view(T, H, d)
    v = silu(h @ p["v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = mem["S"]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    mem["S"] = S
    o = rms(out.reshape(T, H * dv), eps) * p["norm"]
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


# ----------------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, p):
    return (silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def expert(h, up, down):
    return relu2(h @ up.T) @ down.T


def router_scores(h, w_router):
    return torch.sigmoid(h @ w_router.T)


def route_margin(h, w_router, top):
    """(smallest chosen score's logit - largest logit not chosen) / largest |logit| per token; inf when all are chosen."""
    z = h @ w_router.T
    val, _ = torch.sort(z, dim=-1, descending=True)
    if top >= z.shape[-1]:
        return torch.full(z.shape[:-1], float("inf"), dtype=z.dtype)
    return (val[:, top - 1] - val[:, top]) / z.abs().amax(-1)


def moe_ff(h, p, f):
    """f: {"router": {experts, top}, "expert": {ff}, "shared": {ff} or absent}.  The chosen experts' scores multiply
    the experts' inputs and are not renormalised."""
    s = router_scores(h, p["router"])
    val, idx = torch.topk(s, f["router"]["top"], dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += expert(val[t, j] * h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if f.get("shared"):
        out = out + expert(h, p["shared.up"], p["shared.down"])
    return out


# ----------------------------------------------------------------------------------------------------- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def new_memory(raw, dtype=torch.float64):
    """Empty memory of one sequence: per layer keys and values, or a zero state."""
    mem = []
    for layer in raw["layers"]:
        m = layer["mixer"]
        if layer["type"] == "attention":
            mem.append({"k": [], "v": []})
        else:
            mem.append({"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dtype)})
    return mem


def forward(raw, tensors, ids, mem, start, layers_out=None):
    """Runs the tokens ``ids`` (positions start ..) of one sequence from its memory; returns logits [T, vocab].
    ``layers_out``: a list that gets the residual stream after every layer."""
    eps = raw["norm"]["eps"]
    x = tensors["embed"][torch.as_tensor(ids, dtype=torch.long)]
    for i, layer in enumerate(raw["layers"]):
        p = sub(tensors, f"l{i}.mix.")
        if layer["type"] == "attention":
            y = softmax_attention(x, mem[i], start, p, layer["mixer"], eps)
        elif layer["type"] == "lightning":
            y = linear_attention(x, mem[i], p, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, tensors[f"l{i}.norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            pf = sub(tensors, f"l{i}.mlp.")
            y = dense_ff(x, pf) if f["kind"] == "dense" else moe_ff(x, pf, f)
            x = x + norm_one_plus(y, tensors[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, tensors["final.norm"], eps) @ tensors["head"].T


class PlainZikupel:
    """The whole model over explicit per-sequence memory; ``forward`` may be called again with further tokens."""

    def __init__(self, raw, tensors, dtype=torch.float64):
        self.raw = raw
        self.t = {k: v.to(dtype) for k, v in tensors.items()}
        self.dtype = dtype

    def new_state(self):
        return {"mem": new_memory(self.raw, self.dtype), "n": 0, "margin": [], "top": []}

    def forward(self, state, ids):
        """Logits [len(ids), vocab]; the smallest router margin of every token is appended to state["margin"]."""
        raw, eps = self.raw, self.raw["norm"]["eps"]
        x = self.t["embed"][torch.as_tensor(ids, dtype=torch.long)]
        margin = torch.full((len(ids),), float("inf"), dtype=self.dtype)
        for i, layer in enumerate(raw["layers"]):
            p = sub(self.t, f"l{i}.mix.")
            if layer["type"] == "attention":
                y = softmax_attention(x, state["mem"][i], state["n"], p, layer["mixer"], eps)
            else:
                y = linear_attention(x, state["mem"][i], p, layer["mixer"], eps)
            x = x + norm_one_plus(y, self.t[f"l{i}.norm1"], eps)
            f = layer.get("mlp")
            if f is not None:
                pf = sub(self.t, f"l{i}.mlp.")
                if f["kind"] == "dense":
                    y = dense_ff(x, pf)
                else:
                    margin = torch.minimum(margin, route_margin(x, pf["router"], f["router"]["top"]))
                    y = moe_ff(x, pf, f)
                x = x + norm_one_plus(y, self.t[f"l{i}.norm2"], eps)
        state["n"] += len(ids)
        state["margin"] += margin.tolist()
        return norm_one_plus(x, self.t["final.norm"], eps) @ self.t["head"].T

    def greedy(self, prompt, n):
        st = self.new_state()
        logits = self.forward(st, prompt)
        out = []
        for _ in range(n):
            tok = int(logits[-1].argmax())
            out.append(tok)
            logits = self.forward(st, [tok])
        return out
