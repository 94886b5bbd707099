"""Host twin of the LRU policy (b200moe_slot_ensure_host) against the oracle and the reference's vectors."""
import numpy as np
import pytest
import torch

import oracle
from qwen36_moe_16gb_b200 import build, synth
from qwen36_moe_16gb_b200.slot_cache import SlotCache


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()


def _host_cache(L, E, S):
    c = SlotCache.__new__(SlotCache)
    # construct without touching CUDA: host tables only
    SlotCache.__init__(c, L, E, S, device="cpu", host_tables=True)
    return c


def test_known_answer_vector():
    # harness/test-transport-cpu.py:293-305 of the reference (3 slots < 4 experts: below the cache class's
    # floor, so the policy entry point is called on raw tables)
    import ctypes as C

    from qwen36_moe_16gb_b200 import _lib

    slot_for_id = torch.tensor([[-1, 0, -1, -1], [-1, -1, 2, -1]], dtype=torch.int32)
    id_of_slot = torch.tensor([1, -1, 6], dtype=torch.int32)
    usage, step = torch.tensor([5, 0, 1]), torch.tensor([9])
    src, dst, num = torch.zeros(4, dtype=torch.int32), torch.zeros(4, dtype=torch.int32), torch.zeros(1, dtype=torch.int64)
    t = _lib.SlotTables(slot_for_id.data_ptr(), id_of_slot.data_ptr(), usage.data_ptr(), step.data_ptr(),
                        src.data_ptr(), dst.data_ptr(), num.data_ptr(), None, 2, 4, 3)
    ids = torch.tensor([3, 1, 0, 3], dtype=torch.int32)
    assert _lib.lib().b200moe_slot_ensure_host(C.byref(t), 0, ids.data_ptr(), 4, ids.data_ptr()) == 0
    assert int(num) == 2 and src[:2].tolist() == [0, 3] and dst[:2].tolist() == [1, 2]
    assert slot_for_id.view(-1)[[0, 1, 3, 6]].tolist() == [1, 0, 2, -1]
    assert usage.tolist() == [10, 10, 10] and ids.tolist() == [2, 0, 1, 2]
    ids = torch.tensor([2], dtype=torch.int32)
    assert _lib.lib().b200moe_slot_ensure_host(C.byref(t), 1, ids.data_ptr(), 1, ids.data_ptr()) == 0
    assert int(slot_for_id.view(-1)[6]) == 0


@pytest.mark.parametrize("geom", [(6, 32, 48, 40, 4), (40, 256, 4603, 24, 8), (3, 16, 16, 30, 8)])
def test_host_lru_matches_oracle(geom):
    L, E, S, steps, k = geom
    routing = synth.cache_routing(seed=7, steps=steps, layers=L, num_experts=E, top_k=k)
    c = _host_cache(L, E, S)
    c.collect_stats = True
    o = oracle.SlotCacheOracle(L, E, S)
    for s in range(steps):
        for layer in range(L):
            ids = routing[s, layer].clone()
            n = c.ensure_experts_host(layer, ids)
            want = o.ensure(layer, routing[s, layer].numpy())
            assert ids.tolist() == want.tolist()
            assert c.src_indices[:n].tolist() == o.src_indices.tolist()
            assert c.evict_slots[:n].tolist() == o.evict_slots.tolist()
        assert np.array_equal(c.slot_for_id.view(-1).numpy(), o.slot_for_id)
        assert np.array_equal(c.id_of_slot.numpy(), o.id_of_slot)
        assert np.array_equal(c.usage.numpy(), o.usage) and int(c.step) == o.step
    assert np.array_equal(c.lru_stats.numpy(), o.stats)


def test_more_misses_than_slots_and_negative_ids():
    c = _host_cache(1, 8, 8)
    o = oracle.SlotCacheOracle(1, 8, 8)
    ids = torch.tensor([5, -1, 2, 5], dtype=torch.int32)
    want = o.ensure(0, ids.numpy())
    c.ensure_experts_host(0, ids)
    assert ids.tolist() == want.tolist() and ids[1] == -1
    with pytest.raises(ValueError):
        SlotCache(1, 8, 4, device="cpu", host_tables=True)  # cache_size < num_experts


def test_host_bank_is_lazy_page_aligned_and_views_exactly():
    """HostBank: page-aligned anonymous mapping, zero until written, a torch view of exactly the asked shape;
    pageable until pinned (pinning itself needs a GPU and is covered by the offload-stack tests)."""
    from qwen36_moe_16gb_b200.host_banks import HostBank, HostResidency

    bank = HostBank((3, 1000), torch.uint8)
    assert bank.addr % 4096 == 0 and bank.nbytes == 3000
    assert bank.tensor.shape == (3, 1000) and bank.tensor.dtype == torch.uint8
    assert int(bank.tensor.sum()) == 0
    bank.tensor[1].fill_(7)
    assert bank.tensor.data_ptr() == bank.addr and int(bank.tensor.sum()) == 7000
    assert bank.residency is HostResidency.PAGEABLE
    f = HostBank((4, 8), torch.float32, huge_pages=False)
    f.tensor.copy_(torch.arange(32, dtype=torch.float32).view(4, 8))
    assert float(f.tensor[3, 7]) == 31.0
