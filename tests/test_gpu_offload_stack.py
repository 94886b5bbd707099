"""Slot-cache decode stack: tables and miss sequence bit-exact against the oracle policy, outputs identical
to computing straight from the layer's full bank."""
import numpy as np
import pytest
import torch

import oracle
from qwen36_moe_16gb_b200 import ops, synth
from qwen36_moe_16gb_b200.offload_runner import OffloadDecodeStack

pytestmark = pytest.mark.gpu


def test_offload_stack_matches_policy_oracle_and_direct_compute():
    shape = synth.Shape(hidden=1024, intermediate=512, num_experts=16, top_k=4, shared_intermediate=256)
    L, S, steps = 5, 40, 30
    stack = OffloadDecodeStack(shape, L, S, seed=3)
    for c in stack.cache.bank_caches.values():
        c.view(torch.uint8).fill_(0xA5)
    routing = synth.cache_routing(seed=11, steps=steps, layers=L, num_experts=shape.num_experts, top_k=shape.top_k)
    res = stack.run(routing, keep_outputs=True)
    o = oracle.SlotCacheOracle(L, shape.num_experts, S)
    c = 0
    for s in range(steps):
        for layer in range(L):
            o.ensure(layer, routing[s, layer].numpy())
            src, dst = stack.miss_log[c]
            assert src == o.src_indices.tolist() and dst == o.evict_slots.tolist(), (s, layer)
            c += 1
    assert np.array_equal(stack.cache.slot_for_id.view(-1).numpy(), o.slot_for_id)
    assert np.array_equal(stack.cache.id_of_slot.numpy(), o.id_of_slot)
    assert np.array_equal(stack.cache.usage.numpy(), o.usage) and int(stack.cache.step) == o.step
    assert res["h2d_bytes"] == int(o.stats[:, 1].sum()) * shape.expert_bytes
    assert 0.0 < res["miss_rate"] < 1.0
    # every mapped slot holds its host bytes
    ios = stack.cache.id_of_slot
    for slot in torch.nonzero(ios >= 0).reshape(-1).tolist():
        l, e = divmod(int(ios[slot]), shape.num_experts)
        for role in synth.ROLES:
            assert torch.equal(stack.cache.bank_caches[role][slot].cpu().view(torch.uint8),
                               stack.sources[role][l][e].view(torch.uint8)), (role, slot)
    # last step's outputs == decode straight from the full layer bank with expert ids
    w = torch.full((1, shape.top_k), 1.0 / shape.top_k, device="cuda")
    for layer in range(L):
        full = {r: stack.sources[r][layer].cuda() for r in synth.ROLES}
        handle = ops.make_banks(full)
        stack.block.decode_route(stack.x, handle)
        want = stack.block.decode_experts(stack.x, handle, w, routing[steps - 1, layer].view(1, -1).cuda())
        assert torch.equal(res["out"][layer].view(torch.int16), want.view(torch.int16)), layer


def test_native_runner_policy_at_full_geometry():
    """The native step runner's recency-list form of the policy at the benchmark's geometry (40 layers, 256 experts,
    4603 slots): ordered miss plans of every call and the final tables against the oracle.  Small expert shape, so
    the host banks stay small; the policy does not depend on it."""
    shape = synth.Shape(hidden=512, intermediate=512, num_experts=256, top_k=8, shared_intermediate=128)
    L, S, steps = 40, 4603, 48
    stack = OffloadDecodeStack(shape, L, S, seed=5)
    routing = synth.cache_routing(seed=0, steps=steps, layers=L)
    stack.run(routing)
    o = oracle.SlotCacheOracle(L, shape.num_experts, S)
    c = 0
    for s in range(steps):
        for layer in range(L):
            o.ensure(layer, routing[s, layer].numpy())
            src, dst = stack.miss_log[c]
            assert src == o.src_indices.tolist() and dst == o.evict_slots.tolist(), (s, layer)
            c += 1
    assert np.array_equal(stack.cache.slot_for_id.view(-1).numpy(), o.slot_for_id)
    assert np.array_equal(stack.cache.id_of_slot.numpy(), o.id_of_slot)
    assert np.array_equal(stack.cache.usage.numpy(), o.usage) and int(stack.cache.step) == o.step
    stack.close()


def test_device_routed_stack_in_one_graph():
    """Router -> device LRU -> miss gather on a side stream while the shared expert's rows run -> expert GEMVs, for
    a stack of layers captured in ONE CUDA graph: ordered miss plans and final tables bit-exact against the oracle,
    every mapped slot holds its host bytes, outputs equal decoding straight from the full layer bank, and a second
    replay of the same step leaves the plan empty (everything resident) and the outputs unchanged."""
    from qwen36_moe_16gb_b200.decode_overlap import DeviceRoutedDecodeStack

    shape = synth.Shape(hidden=1024, intermediate=512, num_experts=16, top_k=4, shared_intermediate=256)
    L, S, steps = 5, 40, 12
    host = OffloadDecodeStack(shape, L, S, seed=3)          # only for its pinned host banks
    stack = DeviceRoutedDecodeStack(shape, L, S, host.records, seed=3, log_plans=True)
    routing = synth.cache_routing(seed=11, steps=steps, layers=L, num_experts=shape.num_experts, top_k=shape.top_k)
    x = host.x
    ids_buf = torch.zeros((L, 1, shape.top_k), dtype=torch.int32, device="cuda")
    stack.capture(x, ids_buf, keep_outputs=True)
    for c in stack.cache.bank_caches.values():
        c.view(torch.uint8).fill_(0xA5)
    res = stack.run(routing, ids_buf, collect_plans=True)
    o = oracle.SlotCacheOracle(L, shape.num_experts, S)
    c = 0
    for s in range(steps):
        for layer in range(L):
            o.ensure(layer, routing[s, layer].numpy())
            src, dst = res["plans"][c]
            assert src == o.src_indices.tolist() and dst == o.evict_slots.tolist(), (s, layer)
            c += 1
    cache = stack.cache
    assert np.array_equal(cache.slot_for_id.view(-1).cpu().numpy(), o.slot_for_id)
    assert np.array_equal(cache.id_of_slot.cpu().numpy(), o.id_of_slot)
    assert np.array_equal(cache.usage.cpu().numpy(), o.usage) and int(cache.step) == o.step
    assert res["h2d_bytes"] == int(o.stats[:, 1].sum()) * shape.expert_bytes
    ios = cache.id_of_slot.cpu()
    for slot in torch.nonzero(ios >= 0).reshape(-1).tolist():
        l, e = divmod(int(ios[slot]), shape.num_experts)
        for role in synth.ROLES:
            assert torch.equal(cache.bank_caches[role][slot].cpu().view(torch.uint8),
                               cache.bank_sources[role][l][e].view(torch.uint8)), (role, slot)
    # outputs of the last step == decode straight from the full layer bank with expert ids and the same weights
    w = torch.full((1, shape.top_k), 1.0 / shape.top_k, device="cuda")
    first = [t.clone() for t in stack.outs]
    for layer in range(L):
        blk = stack.blocks[layer]
        full = {r: cache.bank_sources[r][layer].cuda() for r in synth.ROLES}
        handle = ops.make_banks(full)
        blk.decode_route(x, handle)
        want = blk.decode_experts(x, handle, w, routing[steps - 1, layer].view(1, -1).cuda())
        assert torch.equal(first[layer].view(torch.int16), want.view(torch.int16)), layer
    # the same step again: no misses, identical outputs
    again = stack.run(routing[steps - 1:], ids_buf, collect_plans=True)
    assert all(src == [] for src, _ in again["plans"])
    for layer in range(L):
        assert torch.equal(stack.outs[layer].view(torch.int16), first[layer].view(torch.int16))
    host.close()
