"""The Zapipel design through the step function, the cache and the batch building on the CPU, with the kernels
replaced by torch doubles (tests/fake_ops.py): cache entries shared between layers, groups of different row sizes,
positions, cache rows, page reuse and wanted rows, in every way of cutting requests into steps."""
import pytest
import torch

import fake_ops
import helpers
import plain_zapipel as plain
from test_zapipel_gpu import SHAPES, SEEDS, STD


def _runner(raw, tensors, max_tokens, page_size):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    from pico_vllm_b200.registry import config_from_dict
    ecfg = EngineConfig(dtype="float32", page_size=page_size, max_cache_tokens=max_tokens, max_num_seqs=4,
                        use_cuda_graph=False, device="cpu")
    model = model_from_tensors(config_from_dict(raw), tensors, ecfg)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


@pytest.mark.parametrize("name,page_size", [("p", 8), ("r", 16)])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_cutting_matches_plain(monkeypatch, name, page_size, cut):
    fake_ops.install(monkeypatch)
    from pico_vllm_b200.registry import config_from_dict
    from pico_vllm_b200.weights import random_tensors
    raw = SHAPES[name]
    tensors = random_tensors(config_from_dict(raw), SEEDS[name], std=STD, dtype=torch.bfloat16)
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 40 + i) for i, n in enumerate([1, 7, 30, 45, 18])}
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 12),
             "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, max_live=3, seed=2)}[cut](reqs)
    runner = _runner(raw, tensors, helpers.live_token_peak(steps), page_size)
    model = plain.PlainZapipel(raw, tensors, torch.float64)
    logits = {rid: model.forward(model.new_state(), ids) for rid, ids in reqs.items()}
    want = helpers.expected_logits(steps, reqs, logits)
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None)
        if w is not None:
            helpers.assert_close_logits(g, w.float(), 5e-5, f"{name}/{cut} step {i}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)
