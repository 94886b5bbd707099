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
