"""Speculative one-layer-ahead prefetch: predictor kernels against the oracle, admission through the unchanged LRU,
slot bytes after the side-stream gather, and the route trace file."""
import numpy as np
import pytest
import torch

import oracle
from qwen36_moe_16gb_b200 import synth
from qwen36_moe_16gb_b200.kernel import B200Nvfp4MoEKernel, MoEConfig
from qwen36_moe_16gb_b200.pregate import DecodePregate, RouteTrace
from qwen36_moe_16gb_b200.slot_cache import SlotCache

pytestmark = pytest.mark.gpu
DEV = "cuda"
SHAPE = synth.Shape(hidden=512, intermediate=512, num_experts=16, top_k=4, shared_intermediate=128)


def _cache(layers=3, slots=24):
    layout = B200Nvfp4MoEKernel().layout(MoEConfig(SHAPE.num_experts, SHAPE.hidden, SHAPE.intermediate, SHAPE.top_k))
    g = torch.Generator().manual_seed(9)
    sources = {r: [] for r in synth.ROLES}
    for _ in range(layers):
        b = synth.make_banks(g, SHAPE)
        for r in synth.ROLES:
            sources[r].append(b[r].pin_memory())
    cache = SlotCache(layers, SHAPE.num_experts, slots, DEV, layout=layout)
    cache.collect_stats = True
    cache.set_bank_sources(sources)
    return cache, sources


def test_predictor_matches_oracle_and_admits_through_the_lru():
    cache, sources = _cache()
    for c in cache.bank_caches.values():
        c.view(torch.uint8).fill_(0xA5)
    g = torch.Generator().manual_seed(4)
    residual = (torch.randn(1, SHAPE.hidden, generator=g) * 2).to(torch.bfloat16)
    norm_w = (torch.randn(SHAPE.hidden, generator=g) * 0.1 + 1).to(torch.bfloat16)
    gate_w = (torch.randn(SHAPE.num_experts, SHAPE.hidden, generator=g) * 0.05).to(torch.bfloat16)
    pre = DecodePregate(cache, DEV, linear_cap=3)
    assert pre.predictor_ok(residual.to(DEV), norm_w.to(DEV), gate_w.to(DEV), SHAPE.num_experts)
    # make two of the would-be predictions resident first, so the selection has hits to skip
    want_logits = oracle.pregate_logits(residual, norm_w, gate_w, 1e-6)
    order = torch.sort(-want_logits, stable=True).indices[:SHAPE.top_k].tolist()
    warm = torch.tensor([order[0], order[2]], dtype=torch.int32, device=DEV)
    cache.ensure_experts(1, warm)
    cache.copy_missing()
    torch.cuda.synchronize()
    o = oracle.SlotCacheOracle(3, SHAPE.num_experts, 24)
    o.ensure(1, np.array([order[0], order[2]]))
    want_query = oracle.pregate_select(want_logits, o.slot_for_id[SHAPE.num_experts:2 * SHAPE.num_experts], 3, SHAPE.top_k, pre.width)
    pre.launch(1, residual.to(DEV), norm_w.to(DEV), 1e-6, gate_w.to(DEV), pre.cap(attention=False), SHAPE.top_k)
    pre.release_input()
    pre.join()
    torch.cuda.synchronize()
    got_logits = pre.logits.cpu()
    assert torch.allclose(got_logits, want_logits, rtol=1e-4, atol=1e-4)
    o.ensure(1, np.array(want_query))
    assert np.array_equal(cache.slot_for_id.view(-1).cpu().numpy(), o.slot_for_id)
    assert np.array_equal(cache.id_of_slot.cpu().numpy(), o.id_of_slot)
    assert int(pre.rows[1]) == len(o.src_indices) == 2              # two of the four predictions missed
    assert int(cache.lru_stats[1, 1]) == 2                            # only the warm-up misses are the cache's misses
    ios = cache.id_of_slot.cpu()
    for slot in torch.nonzero(ios >= 0).reshape(-1).tolist():
        l, e = divmod(int(ios[slot]), SHAPE.num_experts)
        for r in synth.ROLES:
            assert torch.equal(cache.bank_caches[r][slot].cpu().view(torch.uint8), sources[r][l][e].view(torch.uint8))


def test_select_ties_nan_and_no_miss_padding():
    """Crafted logits (a residual with one non-zero element makes logit e = gate_w[e, 0] * const): a three-way tie is
    taken in ascending id, a NaN logit ranks last, resident predictions are skipped, and when nothing misses the
    query is the top-1 prediction repeated."""
    cache, _ = _cache(layers=1, slots=32)
    pre = DecodePregate(cache, DEV, linear_cap=2)
    e = SHAPE.num_experts
    col = torch.zeros(e)
    col[[3, 7, 9]] = 5.0
    col[12] = 4.0
    col[1] = float("nan")
    gate_w = torch.zeros(e, SHAPE.hidden)
    gate_w[:, 0] = col
    residual = torch.zeros(1, SHAPE.hidden)
    residual[0, 0] = 2.0
    norm_w = torch.ones(SHAPE.hidden)
    args = [t.to(torch.bfloat16).to(DEV) for t in (residual, norm_w, gate_w)]
    cache.ensure_experts(0, torch.tensor([3], dtype=torch.int32, device=DEV))     # the top prediction is resident
    pre.launch(0, args[0], args[1], 1e-6, args[2], 2, SHAPE.top_k)
    pre.join()
    torch.cuda.synchronize()
    logits = pre.logits.cpu()
    assert torch.isnan(logits[1]) and logits[3] == logits[7] == logits[9] > logits[12] > 0
    # the query was rewritten to slot ids by the ensure: look the admitted experts up in the tables instead
    ios = cache.id_of_slot.cpu().tolist()
    assert sorted(i for i in ios if i >= 0) == [3, 7, 9]             # 3 (warm) + the two first misses in id order
    # nothing misses: everything the predictor could pick is made resident first
    cache.ensure_experts(0, torch.tensor([12, 0, 2, 4], dtype=torch.int32, device=DEV))
    before = cache.id_of_slot.clone()
    pre.launch(0, args[0], args[1], 1e-6, args[2], 2, SHAPE.top_k)
    pre.join()
    torch.cuda.synchronize()
    assert torch.equal(before, cache.id_of_slot)                     # top-1 repeated: a hit, nothing admitted
    want = oracle.pregate_select(logits, cache.slot_for_id[0].cpu(), 2, SHAPE.top_k, pre.width)
    assert want == [3, 3]


def test_route_trace_writes_replayable_file(tmp_path):
    cache, _ = _cache()
    trace = RouteTrace(cache, tmp_path)
    ids = torch.tensor([[1, 5, 9, 2]], dtype=torch.int32, device=DEV)
    for step in range(2):
        for layer in range(3):
            trace.predict(layer, torch.tensor([1, 5, 0, 3]))
            trace.observe(layer, ids)
            work = ids.clone()
            cache.ensure_experts(layer, work)
    path = trace.flush()
    z = np.load(path)
    assert z["actual"].shape == (2, 3, 4) and z["missed"][0].all() and not z["missed"][1].any()
    assert (z["predicted"][0, 0] == [1, 5, 0, 3]).all() and int(z["cache_size"]) == 24
    assert (z["slot_for_id"] == -1).all() and int(z["step"]) == 0
