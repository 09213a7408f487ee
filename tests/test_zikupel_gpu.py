"""The Zikupel design in the engine against the plain implementation of tests/plain_zikupel.py: every new kernel alone,
whole models of several small shapes in every cutting of requests into steps, batches against each request alone, a key
that stands out far back and at page borders, a state that must survive from step to step, long decoding through pages
and slots that are used again, and greedy generation through the entry points.

Routers: the float32 runs route by the data.  In bfloat16 the router's input differs from the float64 oracle's by the
rounding of the layers before it, enough to send some tokens to other experts than the oracle does, and a token that
took another expert changes every later token through attention; so the bfloat16 runs of whole models choose all of a
layer's experts (the scores, which weigh the experts' inputs, still differ from token to token), and data-dependent
routing in bfloat16 is covered by the kernels' own tests, which are given the choices.
"""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fake_ops
import helpers
import plain_zikupel as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# max |difference| / max |logit| over a step; float32 is the sharp test.  Every sublayer's output is normed to unit size
# before it is added, however small it was, so bfloat16 rounding shows more than in a pre-norm decoder.
REL = {"float32": 5e-5, "bfloat16": 6e-2}


def _att(heads, kv_heads, dim, scale, rot_dims, base=10000.0, softcap=None, scaling=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, rot=dict(base=base, dims=rot_dims))
    if softcap is not None:
        m["softcap"] = softcap
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(type="attention", mixer=m)


def _lin(heads, dim, vdim, decay):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay)))


def _moe(ff, experts, top, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


SHAPES = {
    # starts with the linear mixer; key and value sizes differ; 2 of 5 experts with a shared expert of another size;
    # a head of 32 turned in its first 16 dims with stretched frequencies and a cap; a layer without feed-forward whose
    # heads turn whole, without stretching or cap, one query head per kv head; all 3 of 3 experts, no shared one
    "a": dict(architecture="Zikupel", vocab=211, width=96, norm=dict(eps=1e-5),
              layers=[_layer(_lin(3, 16, 24, (0.5, 0.9, 0.995)), _moe(40, 5, 2, shared=24)),
                      _layer(_att(4, 2, 32, 0.3, 16, 5000.0, softcap=6.0, scaling=(8.0, 32, 8.0, 2.0)), dict(kind="dense", ff=72)),
                      _layer(_att(2, 2, 64, 0.2, 64), None),
                      _layer(_lin(2, 48, 16, (0.97, 0.8)), _moe(24, 3, 3))]),
    # the head sizes the tensor-core kernels take (64 and 128): 8 query heads on one kv head, 3 on 3; a linear mixer with
    # keys of 128; 1 of 4 experts
    "b": dict(architecture="Zikupel", vocab=300, width=128, norm=dict(eps=1e-6),
              layers=[_layer(_att(8, 1, 64, 0.25, 32, 30000.0, softcap=15.0, scaling=(3.0, 64, 16.0, 1.5)), _moe(64, 4, 1, shared=64)),
                      _layer(_lin(2, 128, 64, (0.999, 0.7)), dict(kind="dense", ff=160)),
                      _layer(_att(3, 3, 128, 0.15, 128, 1000.0), _moe(32, 6, 3))]),
    # awkward sizes: a width that is a multiple of 4 only, an odd vocabulary, heads of 24 and 40 (padded to 32 and 48 in
    # the cache), a rotation of 6 dims, inner sizes that are no multiples of 8, a linear mixer with keys of 20 and values
    # of 12, a single head
    "c": dict(architecture="Zikupel", vocab=203, width=100, norm=dict(eps=1e-4),
              layers=[_layer(_att(5, 5, 24, 0.4, 6, 300.0, softcap=10.0), _moe(28, 7, 3, shared=20)),
                      _layer(_lin(1, 20, 12, (0.9,)), dict(kind="dense", ff=52)),
                      _layer(_att(6, 2, 40, 0.3, 40, 777.0, scaling=(2.0, 16, 4.0, 0.5)), None)]),
    # sizes that are multiples of 2 at most: width 90, heads of 16 with 4 dims turned, a linear mixer with keys of 8 and values
    # of 4, inner sizes 14, 10 and 6, one of two experts
    "d": dict(architecture="Zikupel", vocab=101, width=90, norm=dict(eps=1e-5),
              layers=[_layer(_lin(2, 8, 4, (0.9, 0.6)), _moe(10, 2, 1, shared=6)),
                      _layer(_att(3, 1, 16, 0.5, 4, 50.0, softcap=8.0), dict(kind="dense", ff=14))]),
}
SEEDS = {"a": 11, "b": 22, "c": 35, "d": 44}     # c: a seed without a token whose tiny sublayer output the post-norm blows up in bfloat16
STD = 0.12      # weights large enough that attention and routers are far from uniform


def _raw(name, dtype):
    """The shape as tested in ``dtype``: in bfloat16 every routed layer chooses all of its experts."""
    raw = copy.deepcopy(SHAPES[name])
    if dtype == "bfloat16":
        for layer in raw["layers"]:
            if layer["mlp"] and layer["mlp"]["kind"] == "moe":
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def _tensors(raw, seed):
    from pico_vllm_b200.registry import config_from_dict
    from pico_vllm_b200.weights import random_tensors
    t = random_tensors(config_from_dict(raw), seed, std=STD, dtype=torch.bfloat16)
    for n in t:         # weights of the query and key norms: around one, some well away from it
        if n.endswith(".q.norm") or n.endswith(".k.norm") or n.endswith("mix.norm"):
            t[n] = (1.0 + 4.0 * (t[n].float() - 1.0)).to(torch.bfloat16)
    return t


def _runner(raw, tensors, dtype, max_tokens, graph=False, page_size=16, max_num_seqs=4):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    from pico_vllm_b200.registry import config_from_dict
    ecfg = EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_num_seqs=max_num_seqs,
                        use_cuda_graph=graph, device=DEV)
    model = model_from_tensors(config_from_dict(raw), tensors, ecfg)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


def _oracle(raw, tensors, reqs):
    model = plain.PlainZikupel(raw, tensors, torch.float64)
    return {rid: model.forward(model.new_state(), ids) for rid, ids in reqs.items()}


def _compare(steps, reqs, got, logits, dtype, what):
    want = helpers.expected_logits(steps, reqs, logits)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None), f"{what} step {i}"
        if w is not None:
            assert g.shape == w.shape and torch.isfinite(g).all(), f"{what} step {i}: shape or a value that is not finite"
            helpers.assert_close_logits(g, w.float(), REL[dtype], f"{what} step {i}")


_CUTS = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 32),
         "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, max_live=4, seed=3)}
LENGTHS = {"a": [1, 9, 33, 70, 150, 230], "b": [2, 17, 48, 97, 200], "c": [3, 40, 129, 75], "d": [5, 60, 300]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("cut,graph", [("whole", False), ("tail", False), ("tail", True), ("portions", False),
                                       ("mixed", False), ("mixed", True)])
def test_every_cutting_matches_plain(dtype, name, cut, graph):
    raw = _raw(name, dtype)
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 500 + i) for i, n in enumerate(LENGTHS[name])}
    steps = _CUTS[cut](reqs)
    tensors = _tensors(raw, SEEDS[name])
    runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), graph=graph)
    logits = _oracle(raw, tensors, reqs)
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{name}/{cut}/{dtype}")
    if graph:
        assert runner.graph_replays > 0
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)      # every page came back
    from pico_vllm_b200 import ops
    ops.check_kernel_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [4, 16, 64])
def test_other_page_sizes_and_batches_against_each_alone(dtype, page_size):
    """Unequal requests in one batch give what each gives alone (the same engine, one request per step), and both agree
    with the plain implementation."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 900 + i) for i, n in enumerate([6, 50, 17, 120])}
    together = [dict(entries=[dict(id=r, tokens=ids[:-4], want=list(range(len(ids) - 4))) for r, ids in reqs.items()], end=[])]
    for k in range(4, 0, -1):
        together.append(dict(entries=[dict(id=r, tokens=[ids[-k]], want=[0]) for r, ids in reqs.items()],
                             end=list(reqs) if k == 1 else []))
    alone = helpers.trace_tail_decode(reqs, 4)
    logits = _oracle(raw, tensors, reqs)
    outs = {}
    for what, steps in (("together", together), ("alone", alone)):
        runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), page_size=page_size)
        got = helpers.replay(runner, steps)
        _compare(steps, reqs, got, logits, dtype, f"{what}/page {page_size}/{dtype}")
        at, rows = {r: 0 for r in reqs}, {}
        for st, g in zip(steps, got):
            i = 0
            for e in st["entries"]:
                for w in e["want"]:
                    rows[(e["id"], at[e["id"]] + w)] = g[i]
                    i += 1
                at[e["id"]] += len(e["tokens"])
        outs[what] = rows
    assert outs["together"].keys() == outs["alone"].keys()
    scale = max(float(v.abs().max()) for v in outs["alone"].values())
    worst = max(float((outs["together"][k] - outs["alone"][k]).abs().max()) for k in outs["alone"])
    assert worst <= (2e-5 if dtype == "float32" else 4e-2) * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_key_that_stands_out_at_page_borders_first_tokens_and_far_back(dtype):
    """One attention layer whose scores are made sharp (a large factor on q.k, a cap of 30): most queries then give
    nearly all their weight to one key, wherever it lies.  The oracle says which key each query prefers; the test needs
    preferred keys at the first positions, on both sides of page borders and hundreds of tokens back - read from a whole
    prompt, from single tokens and from portions cut at page borders - and losing one of them would move the output by
    about the size of a value."""
    raw = dict(architecture="Zikupel", vocab=97, width=64, norm=dict(eps=1e-5),
               layers=[_layer(_att(4, 2, 32, 3.0, 8, 100.0, softcap=30.0), None)])
    tensors = _tensors(raw, 77)
    ids = helpers.random_ids(600, raw["vocab"], 5)
    model = plain.PlainZikupel(raw, tensors, torch.float64)
    st = model.new_state()
    logits = {"r": model.forward(st, ids)}
    # which key every query prefers, from the oracle's own keys (recomputed here from its memory)
    K = torch.stack(st["mem"][0]["k"])                                   # [n, G, d]
    p = plain.sub(model.t, "l0.mix.")
    x = model.t["embed"][torch.tensor(ids)]
    m = raw["layers"][0]["mixer"]
    q = plain.rms((x @ p["q"].T + p["q.b"]).view(len(ids), 4, 32), 1e-5) * p["q.norm"]
    f, mult = plain.yarn_frequencies(8, 100.0, None)
    q = plain.rotate(q, torch.arange(len(ids)), f, mult, 8)
    seen = set()
    for t in range(len(ids)):
        for a in range(4):
            s = m["softcap"] * torch.tanh((K[:t + 1, a // 2] @ q[t, a]) * m["scale"] / m["softcap"])
            w = torch.softmax(s, 0)
            j = int(w.argmax())
            if float(w[j]) > 0.6:
                seen.add((t, j))
    far = [(t, j) for t, j in seen if t - j >= 300]
    first = [(t, j) for t, j in seen if j <= 1 and t - j >= 16]
    border = [(t, j) for t, j in seen if j % 16 in (15, 0) and t - j >= 32]
    assert len(far) >= 5 and len(first) >= 1 and len(border) >= 10, (len(far), len(first), len(border))
    reqs = {"r": ids}
    cuts = {"whole": helpers.trace_whole(reqs), "single": helpers.trace_tail_decode(reqs, 280),
            "pages": helpers.trace_portions(reqs, sizes=(16, 32, 15, 1, 48, 17, 31))}
    for what, steps in cuts.items():
        runner = _runner(raw, tensors, dtype, 640)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_that_remembers_the_first_tokens(dtype):
    """One linear-attention layer with a head that forgets almost nothing (decay 0.9999) beside one that forgets fast:
    the output at the end of 500 tokens still holds the first ones, so a state that is lost, zeroed or handed to
    another request between steps shows.  Two requests take turns, in portions down to two tokens and single tokens,
    in slots that were used before."""
    raw = dict(architecture="Zikupel", vocab=120, width=64, norm=dict(eps=1e-5),
               layers=[_layer(_lin(2, 32, 16, (0.9999, 0.5)), None)])
    tensors = _tensors(raw, 8)
    reqs = {"w": helpers.random_ids(40, raw["vocab"], 1), "x": helpers.random_ids(500, raw["vocab"], 2),
            "y": helpers.random_ids(300, raw["vocab"], 3)}
    model = plain.PlainZikupel(raw, tensors, torch.float64)
    logits = {r: model.forward(model.new_state(), ids) for r, ids in reqs.items()}
    # the first tokens matter at the end: the oracle without them gives other logits
    late = model.forward(model.new_state(), reqs["x"][8:])
    assert float((late[-1] - logits["x"][-1]).abs().max()) > 100 * REL["float32"] * float(logits["x"].abs().max())
    steps = helpers.trace_whole({"w": reqs["w"]})                         # uses a slot and gives it back
    steps += helpers.trace_mixed({"x": reqs["x"], "y": reqs["y"]}, max_live=2, seed=5, chunk_sizes=(2, 7, 64, 3, 2, 33))
    runner = _runner(raw, tensors, dtype, 1024, max_num_seqs=2)
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"state/{dtype}")
    # whole prompts of 500 and 300 tokens: the chunks of a long portion run side by side with a scan between them
    steps = helpers.trace_whole({"x": reqs["x"], "y": reqs["y"]}) + helpers.trace_portions({"x": reqs["x"]}, sizes=(300, 2, 198))
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"long portions/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_reused_slots(dtype):
    """300 single-token steps after a short prompt, twice, through a pool that holds one request."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    reqs = {"x": helpers.random_ids(330, raw["vocab"], 41), "y": helpers.random_ids(330, raw["vocab"], 42)}
    steps = helpers.trace_tail_decode(reqs, 300)
    runner = _runner(raw, tensors, dtype, 384, graph=True, max_num_seqs=1)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"long/{dtype}")
    assert runner.graph_replays > 500


# ------------------------------------------------------------------ the kernels alone, against their torch doubles
def _close(got, want, dtype, what):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = float((got.double().cpu() - want.double().cpu()).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: {err}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,norm_dim,rot,own_v", [(4, 2, 32, 32, 16, False), (5, 5, 32, 24, 6, False), (8, 1, 128, 128, 128, False),
                                                     (3, 1, 64, 64, 0, True), (2, 2, 48, 40, 40, True), (16, 4, 256, 256, 64, False)])
def test_norm_rotation_and_store_kernel(dtype, H, G, hd, norm_dim, rot, own_v):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + hd)
    T, ps, pages = 37, 8, 12
    cols = (H + G * (2 if own_v else 1)) * hd + 24              # the row is wider than its parts
    qkv = torch.randn(T, cols, generator=g)
    mask = (torch.arange(hd) < norm_dim).float()
    qkv[:, :(H + G) * hd] *= mask.repeat(H + G)                 # padded dims are zero, as zero weight rows make them
    qkv = qkv.to(dtype)
    bias = torch.randn((H + G * (2 if own_v else 1)) * hd, generator=g) * mask.repeat(H + G * (2 if own_v else 1))
    qw, kw = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5
    pos = torch.randint(0, 3000, (T,), generator=g).to(torch.int32)
    pos[5] = -1
    slots = torch.randperm(ps * pages, generator=g)[:T].to(torch.int32)
    slots[9] = -1
    inv = (1.0 / 50.0 ** (torch.arange(rot // 2).float() / max(rot // 2, 1))).float()
    res = []
    for dev, fn in (("cpu", fake_ops.qk_norm_rope_store), (DEV, ops.qk_norm_rope_store)):
        a = qkv.clone().to(dev)
        kp = torch.zeros(pages, G, ps, hd, dtype=dtype, device=dev)
        vp = torch.zeros_like(kp)
        fn(a, bias.to(dev), pos.to(dev), inv.to(dev), 1.3, qw.to(dev), kw.to(dev), 1e-5, slots.to(dev), kp, vp, H, G, hd, ps,
           not own_v, norm_dim=norm_dim)
        res.append((a.cpu(), kp.cpu(), vp.cpu()))
    live = pos >= 0
    _close(res[1][0][live, :H * hd], res[0][0][live, :H * hd], dtype, "q")
    assert torch.equal(res[1][0][:, H * hd:], qkv[:, H * hd:])            # nothing but q is written back
    _close(res[1][1], res[0][1], dtype, "k pages")
    _close(res[1][2], res[0][2], dtype, "v pages")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(3, 16, 24), (2, 128, 64), (1, 20, 12), (4, 32, 32), (2, 200, 40), (5, 64, 130)])
@pytest.mark.parametrize("chunk", [0, 16, 3])
@pytest.mark.parametrize("off", [4, 8])
def test_linear_attention_kernel(dtype, H, d, dv, chunk, off):
    """Segments of 1, 2, 8, 9 and 70 tokens and a padding segment, from states that are not zero, into slots in any order;
    walked token by token (chunk 0) or as chunks of 16 or 3 tokens side by side with a scan between them."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(d * 7 + dv)
    lens = [1, 70, 2, 9, 8, 1]
    T = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)
    pos[cu[5]:] = -1                                             # the last segment is padding
    seg_slots = torch.tensor([4, 0, 6, 2, 5, 0], dtype=torch.int32)
    width = H * (2 * d + dv) + 16
    proj = (torch.randn(T, width, generator=g) * 0.7).to(dtype)
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    state = torch.randn(7, H, dv, d, generator=g) * 0.3
    want_state = state.clone()
    want = fake_ops.decay_linear_attention(proj, off, off + H * d, off + 2 * H * d, decay, want_state, seg_slots, cu, pos, H, d, dv, 1)
    st = state.clone().to(DEV)
    got = ops.decay_linear_attention(proj.to(DEV), off, off + H * d, off + 2 * H * d, decay.to(DEV), st, seg_slots.to(DEV),
                                     cu.to(DEV), pos.to(DEV), H, d, dv, 1, max_q_len=70, chunk=chunk)
    n = int(cu[5])
    _close(got[:n], want[:n], torch.float32, "outputs")
    _close(st, want_state, torch.float32, "states")
    assert torch.equal(st[1].cpu(), state[1]) and torch.equal(st[3].cpu(), state[3])      # slots of no segment are untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dv", [(3, 16, 24), (2, 128, 64), (1, 20, 12), (2, 200, 40), (5, 64, 130), (2, 30, 8)])
def test_linear_attention_of_single_tokens(dtype, H, d, dv):
    """A step in which every segment brings one token (a decode step: a stream of states): slots in any order, a padding
    row, states that are not zero."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(d * 3 + dv)
    S = 9
    cu = torch.arange(S + 1, dtype=torch.int32)
    pos = torch.randint(0, 500, (S,), generator=g).to(torch.int32)
    pos[6] = -1
    seg_slots = torch.tensor([4, 0, 6, 2, 5, 9, 0, 1, 8], dtype=torch.int32)
    proj = (torch.randn(S, H * (2 * d + dv) + 8, generator=g) * 0.7).to(dtype)
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    state = torch.randn(10, H, dv, d, generator=g) * 0.3
    want_state = state.clone()
    want = fake_ops.decay_linear_attention(proj, 0, H * d, 2 * H * d, decay, want_state, seg_slots, cu, pos, H, d, dv, 1)
    st = state.clone().to(DEV)
    got = ops.decay_linear_attention(proj.to(DEV), 0, H * d, 2 * H * d, decay.to(DEV), st, seg_slots.to(DEV), cu.to(DEV),
                                     pos.to(DEV), H, d, dv, 1, max_q_len=1)
    live = pos >= 0
    _close(got[live], want[live], torch.float32, "outputs")
    _close(st, want_state, torch.float32, "states")
    assert torch.equal(st[3].cpu(), state[3]) and torch.equal(st[7].cpu(), state[7])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [48, 130, 1024, 4100])
def test_gated_norm_and_gate_kernels(dtype, N):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(N)
    x = torch.randn(19, N, generator=g) * 3
    w = torch.rand(N, generator=g) + 0.5
    wide = torch.randn(19, N + 40, generator=g).to(dtype)
    want = fake_ops.gated_rms_norm(x, w, wide[:, 16:16 + N], 1e-5, dtype)
    got = ops.gated_rms_norm(x.to(DEV), w.to(DEV), wide.to(DEV)[:, 16:16 + N], 1e-5, dtype)
    _close(got, want, dtype, "gated norm")
    _close(ops.gated_rms_norm(x.to(DEV), None, None, 1e-5, dtype), fake_ops.gated_rms_norm(x, None, None, 1e-5, dtype), dtype, "plain")
    o = torch.randn(19, N, generator=g).to(dtype)
    _close(ops.sigmoid_gate(o.clone().to(DEV), wide.to(DEV)[:, 16:16 + N]), fake_ops.sigmoid_gate(o.clone(), wide[:, 16:16 + N]),
           dtype, "gate")


@pytest.mark.parametrize("experts,top", [(5, 1), (12, 3), (3, 3)])
def test_router_with_sigmoid_scores(experts, top):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(experts)
    for T, D in ((50, 72), (701, 72), (9, 70)):
        h = torch.randn(T, D, generator=g)
        wr = torch.randn(experts, D, generator=g)
        idx, wgt = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, ops.MOE_SCORE_SIGMOID)
        widx, wwgt = fake_ops.moe_route(h, wr, None, top, 1)
        assert torch.equal(idx.cpu().sort(-1).values, widx.sort(-1).values)
        _close(wgt.cpu().sort(-1).values, wwgt.sort(-1).values, torch.float32, "scores")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,ff,experts,top", [(1, 64, 32, 4, 2), (150, 96, 40, 6, 2), (300, 72, 24, 3, 1), (9, 100, 28, 7, 3),
                                                (1200, 64, 48, 5, 2)])
@pytest.mark.parametrize("on_input", [True, False])
def test_ungated_experts_kernels(dtype, T, D, ff, experts, top, on_input):
    """Experts without a gate, relu squared, the weight on the input or on the output, a shared expert's output added:
    lists longer than a tile, an expert without tokens, widths that are no multiple of 8, enough rows for the library."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(T + D)
    h = torch.randn(T, D, generator=g).to(dtype)
    up = (torch.randn(experts, ff, D, generator=g) * 0.2).to(dtype)
    down = (torch.randn(experts, D, ff, generator=g) * 0.2).to(dtype)
    base = torch.randn(T, D, generator=g).to(dtype)
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if experts > 2:
        idx[idx == experts - 1] = 0 if top == 1 else idx[idx == experts - 1]        # top 1: the last expert gets no token
    wgt = torch.rand(T, top, generator=g) * 0.8 + 0.1
    want = fake_ops.moe_experts(h, idx, wgt, up, down, gated=False, act=1, weight_on_input=on_input, base=base)
    got = ops.moe_experts(h.to(DEV), idx.to(DEV), wgt.to(DEV), up.to(DEV), down.to(DEV), gated=False, act=ops.MOE_ACT_RELU2,
                          weight_on_input=on_input, base=base.to(DEV))
    _close(got, want, dtype, "experts")
    u = torch.randn(33, 50, generator=g).to(dtype)
    _close(ops.activation(u.clone().to(DEV), ops.MOE_ACT_RELU2), fake_ops.activation(u.clone(), 1), dtype, "relu squared")


@pytest.mark.parametrize("hd,H,G,ps", [(64, 8, 1, 16), (128, 10, 2, 16), (32, 4, 2, 8), (128, 3, 3, 64), (48, 6, 3, 4)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_attention_kernels_with_capped_scores(dtype, hd, H, G, ps):
    """Prompt portions and single tokens in one batch through the kernels the mixer uses (tensor cores in bfloat16 - with
    the tensor maps the cache manager makes for heads of 64 and 128 -, the float32 kernel otherwise), a cap of 5 on
    scores that reach well beyond it, against the double."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(hd + H)
    lens, starts = [150, 1, 33, 1, 2], [40, 333, 0, 64, 127]
    n_pages = sum(-(-(s + n) // ps) for s, n in zip(starts, lens)) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    kp = torch.randn(n_pages, G, ps, hd, generator=g).to(dtype)
    vp = torch.randn(n_pages, G, ps, hd, generator=g).to(dtype)
    width = max(-(-(s + n) // ps) for s, n in zip(starts, lens))
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    at = 0
    for i, (s, n) in enumerate(zip(starts, lens)):
        k = -(-(s + n) // ps)
        table[i, :k] = torch.tensor(order[at:at + k], dtype=torch.int32)
        at += k
    T = sum(lens)
    q = (torch.randn(T, H * hd + 16, generator=g) * 1.5).to(dtype)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    want = torch.zeros(T, H * hd, dtype=dtype)
    fake_ops.paged_attention(q, kp, vp, want, seg, pos, table, H, G, hd, ps, None, 0.3, softcap=5.0)
    d = lambda t: t.to(DEV)
    kpd, vpd = d(kp), d(vp)
    out = torch.zeros(T, H * hd, dtype=dtype, device=DEV)
    if dtype == torch.bfloat16:
        pf = torch.tensor([0, 2, 4], dtype=torch.int32)
        dec = torch.tensor([int(cu[1]), int(cu[3])], dtype=torch.int32)
        splits = 2
        scratch = torch.empty(ops.attention_scratch_floats(T, H, hd, splits), dtype=torch.float32, device=DEV)
        ops.paged_attention_mma(d(q), kpd, vpd, out, d(seg), d(pos), d(table), d(cu), d(pf), 3, 150, d(dec), 2, H, G, hd, ps,
                                None, 0.3, splits, scratch, ops.make_kv_tensor_map(kpd), ops.make_kv_tensor_map(vpd),
                                ops.make_kv_tensor_map_2d(kpd), ops.make_kv_tensor_map_2d(vpd, values=True), 0, softcap=5.0)
    else:
        ops.paged_attention(d(q), kpd, vpd, out, d(seg), d(pos), d(table), H, G, hd, ps, None, 0.3, softcap=5.0)
    _close(out, want, dtype, "attention")
    ops.check_kernel_status()


# ------------------------------------------------------------------ through the entry points
def test_greedy_generation_through_the_entry_point(tmp_path):
    from pico_vllm_b200 import LLM, SamplingParams
    from pico_vllm_b200.registry import config_from_dict
    from safetensors.torch import save_file
    raw = SHAPES["a"]
    tensors = _tensors(raw, SEEDS["a"])
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config_from_dict(raw).to_dict()))
    save_file(tensors, str(folder / "model.safetensors"))
    llm = LLM(str(folder), dtype="float32", max_cache_tokens=1024, device=DEV)
    prompts = [helpers.random_ids(n, raw["vocab"], 70 + n) for n in (4, 23, 61)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    model = plain.PlainZikupel(raw, tensors, torch.float64)
    for p, o in zip(prompts, outs):
        assert list(o.token_ids) == model.greedy(p, 12)


def test_command_line_writes_a_model_folder_and_generates(tmp_path, capsys):
    from pico_vllm_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(SHAPES["c"]))
    folder = str(tmp_path / "model")
    assert main(["random-model", "--config", str(tmp_path / "config.json"), "--seed", "9", "--out", folder, "--std", str(STD)]) == 0
    capsys.readouterr()
    prompts = [[5, 17, 3], [9, 9]]
    rc = main(["run", "--model", folder, "--dtype", "float32", "--prompt-ids", "5,17,3", "--prompt-ids", "9,9",
               "--max-new-tokens", "5", "--temperature", "0", "--num-gpu-blocks", "32", "--ignore-eos"])
    assert rc == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[")]
    printed = {int(l[1:l.index("]")]): [int(t) for t in l.split("] ")[1].split()] for l in lines}
    from safetensors.torch import load_file
    model = plain.PlainZikupel(SHAPES["c"], load_file(os.path.join(folder, "model.safetensors")), torch.float64)
    for rid, p in enumerate(prompts):       # prompt and generated tokens are printed together
        assert printed[rid] == p + model.greedy(p, 5)


def test_trace_replay_of_a_model_folder(tmp_path):
    from pico_vllm_b200.registry import config_from_dict
    from safetensors.torch import save_file
    raw = SHAPES["b"]
    tensors = _tensors(raw, SEEDS["b"])
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config_from_dict(raw).to_dict()))
    save_file(tensors, str(folder / "model.safetensors"))
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 300 + i) for i, n in enumerate([40, 7, 95, 33, 64])}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=1)
    lines = "".join(json.dumps(dict(step=i, **st)) + "\n" for i, st in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(helpers.live_token_peak(steps))],
                       input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    logits = _oracle(raw, tensors, reqs)
    for i, w in enumerate(helpers.expected_logits(steps, reqs, logits)):
        if w is not None:
            got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, raw["vocab"]))
            helpers.assert_close_logits(got, w.float(), REL["float32"], f"step {i}")
