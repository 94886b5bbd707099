"""Device slot cache: tables and miss sequences bit-exact against the oracle; fills move the right bytes."""
import numpy as np
import pytest
import torch

import oracle
from qwen36_moe_16gb_b200 import synth
from qwen36_moe_16gb_b200.slot_cache import SlotCache

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_tables(c: SlotCache, o: oracle.SlotCacheOracle):
    assert np.array_equal(c.slot_for_id.view(-1).cpu().numpy(), o.slot_for_id)
    assert np.array_equal(c.id_of_slot.cpu().numpy(), o.id_of_slot)
    assert np.array_equal(c.usage.cpu().numpy(), o.usage)
    assert int(c.step) == o.step


def test_reference_mirror_trace(golden_dir):
    z = np.load(golden_dir / "lru_mirror_trace.npz")
    L, E, S, steps = z["geometry"].tolist()
    routing = torch.from_numpy(z["routing"])
    c = SlotCache(L, E, S, DEV)
    row = 0
    for s in range(steps):
        for layer in range(L):
            ids = routing[s, layer].to(DEV)
            c.ensure_experts(layer, ids)
            n = int(c.num_indices)
            want = [m for m in z["misses"][row].tolist() if m >= 0]
            assert c.src_indices[:n].tolist() == want
            row += 1
        snap = np.concatenate([c.slot_for_id.view(-1).cpu().numpy(), c.id_of_slot.cpu().numpy(),
                               c.usage.cpu().numpy(), [int(c.step)]])
        assert np.array_equal(snap, z["snapshots"][s])


@pytest.mark.parametrize("geom", [(40, 256, 4603, 12, 8, 1), (4, 64, 80, 30, 8, 4), (2, 16, 16, 20, 4, 8)])
def test_tables_and_miss_sequence_match_oracle(geom):
    L, E, S, steps, k, m = geom
    routing = synth.cache_routing(seed=5, steps=steps * m, layers=L, num_experts=E, top_k=k)
    c = SlotCache(L, E, S, DEV)
    c.collect_stats = True
    o = oracle.SlotCacheOracle(L, E, S)
    for s in range(steps):
        for layer in range(L):
            raw = routing[s * m:(s + 1) * m, layer].contiguous()  # [m, k]: several tokens share one call
            ids = raw.to(DEV)
            c.ensure_experts(layer, ids)
            want = o.ensure(layer, raw.numpy())
            n = int(c.num_indices)
            assert ids.cpu().tolist() == want.tolist()
            assert c.src_indices[:n].tolist() == o.src_indices.tolist()
            assert c.evict_slots[:n].tolist() == o.evict_slots.tolist()
        _check_tables(c, o)
    assert np.array_equal(c.lru_stats.cpu().numpy(), o.stats)
    # maps stay mutual inverses
    ios = c.id_of_slot.cpu()
    sfi = c.slot_for_id.view(-1).cpu()
    for slot in torch.nonzero(ios >= 0).reshape(-1).tolist():
        assert int(sfi[int(ios[slot])]) == slot


def test_materialize_reset_and_negative_ids():
    c = SlotCache(2, 4, 6, DEV)
    o = oracle.SlotCacheOracle(2, 4, 6)
    ids = torch.tensor([[3, 0]], dtype=torch.int32, device=DEV)
    c.ensure_experts(1, ids)
    o.ensure(1, np.array([[3, 0]]))
    c.materialize_layer(0)
    o.materialize_layer(0)
    _check_tables(c, o)
    assert int(c.num_indices) == 4 and c.evict_slots[:4].tolist() == [0, 1, 2, 3]
    ids = torch.tensor([2, -1, 2], dtype=torch.int32, device=DEV)
    c.ensure_experts(1, ids)
    want = o.ensure(1, np.array([2, -1, 2]))
    assert ids.cpu().tolist() == want.tolist()
    c.reset()
    o.reset()
    _check_tables(c, o)


def _fingerprint_banks(L, E, shape):
    """Every row of expert e of layer l filled with a value derived from l*E+e."""
    layout = synth.bank_shapes(shape)
    src = {}
    for role, (shp, dt) in layout.items():
        per_layer = []
        for l in range(L):
            base = (torch.arange(E) + l * E).view(E, *([1] * len(shp)))
            t = (base % 251).expand(E, *shp).to(torch.uint8 if dt != torch.float32 else torch.float32)
            t = t.contiguous()
            if dt == synth.FP8:
                t = t.view(synth.FP8)
            per_layer.append(t.pin_memory())
        src[role] = per_layer
    return src


@pytest.mark.parametrize("host_plan", [False, True])
def test_fills_move_the_right_bytes(host_plan):
    L, E, S, k = 3, 16, 24, 4
    shape = synth.Shape(hidden=256, intermediate=128, num_experts=E, top_k=k)
    src = _fingerprint_banks(L, E, shape)
    c = SlotCache(L, E, S, DEV, host_tables=host_plan)
    c.set_bank_sources(src)
    for cache in c.bank_caches.values():
        cache.view(torch.uint8).fill_(0xA5)
    routing = synth.cache_routing(seed=9, steps=12, layers=L, num_experts=E, top_k=k)
    copy_stream = torch.cuda.Stream()
    for s in range(12):
        for layer in range(L):
            if host_plan:
                ids = routing[s, layer].clone()
                c.ensure_experts_host(layer, ids)
                c.fill_planned(layer, copy_stream)
            else:
                ids = routing[s, layer].to(DEV)
                c.ensure_experts(layer, ids)
                c.copy_missing()
    torch.cuda.synchronize()
    ios = c.id_of_slot.cpu()
    mapped = torch.nonzero(ios >= 0).reshape(-1).tolist()
    assert mapped
    for slot in mapped:
        fid = int(ios[slot])
        l, e = divmod(fid, E)
        for role in c.bank_schema:
            got = c.bank_caches[role][slot].cpu().view(torch.uint8)
            want = src[role][l][e].view(torch.uint8)
            assert torch.equal(got, want), (role, slot, fid)
    unmapped = torch.nonzero(ios < 0).reshape(-1).tolist()
    for slot in unmapped:
        assert bool((c.bank_caches["gate_up"][slot].view(torch.uint8) == 0xA5).all())


def test_slot_offsets_beyond_4gib():
    # gate_up rows are 1 MiB at the full shape: slot 4096 starts at 2^32 bytes
    L, E, S = 1, 256, 4200
    rows = 1 << 20
    src = {"gate_up": [torch.zeros((E, rows), dtype=torch.uint8).pin_memory()]}
    src["gate_up"][0][7].fill_(77)
    c = SlotCache(L, E, S, DEV, layout={"gate_up": __import__("qwen36_moe_16gb_b200").BankSpec((rows,), torch.uint8)})
    c.set_bank_sources(src)
    c.usage[:4150] = 5          # make slot 4150 the LRU victim
    c.step.fill_(5)
    ids = torch.tensor([7], dtype=torch.int32, device=DEV)
    c.ensure_experts(0, ids)
    c.copy_missing()
    torch.cuda.synchronize()
    assert ids.item() == 4150
    assert bool((c.bank_caches["gate_up"][4150] == 77).all())


def test_prefill_double_buffer_streams_whole_layers():
    """Slots [0, 2E) as two whole-layer buffers (copy stream + ready/release events): every layer's prefill reads
    its own banks, and residents of the borrowed slots are unmapped when the epoch opens."""
    from qwen36_moe_16gb_b200 import ops

    L, E, S, k = 4, 16, 48, 4
    shape = synth.Shape(hidden=256, intermediate=128, num_experts=E, top_k=k)
    src = _fingerprint_banks(L, E, shape)
    c = SlotCache(L, E, S, DEV, prefill_overlap=True)
    c.set_bank_sources(src)
    ids = torch.tensor([[1, 5, 9, 13]], dtype=torch.int32, device=DEV)
    c.ensure_experts(2, ids)            # decode residents land in slots 0..3, inside the future buffers
    c.copy_missing()
    assert int((c.id_of_slot[: 2 * E] >= 0).sum()) == 4
    c.begin_prefill()
    assert int((c.id_of_slot[: 2 * E] >= 0).sum()) == 0 and int((c.slot_for_id >= 0).sum()) == 0
    c.prefetch_prefill_layer(0)
    for layer in range(L):
        if layer + 1 < L:
            c.prefetch_prefill_layer(layer + 1)
        view = c.wait_prefill_layer(layer)
        got = {r: v.clone() for r, v in view.items()}    # the "expert GEMM" of this test: read the buffer
        c.release_prefill_layer(layer)
        torch.cuda.synchronize()
        for r in c.bank_schema:
            assert torch.equal(got[r].cpu().view(torch.uint8), src[r][layer].view(torch.uint8)), (layer, r)
    assert c.h2d_bytes == L * E * c.expert_bytes


def test_prefill_through_the_cache_feeds_the_grouped_gemm():
    """Four layers streamed through the two prefill buffers with the grouped GEMM as the consumer, in three forms:
    whole layers, whole layers with resident experts copied device-to-device, and only the selected experts of a
    short chunk.  Every layer's output equals the kernels run straight on the layer's full bank; buffer rows hold
    the host bytes; the hit/miss split counts match the residency."""
    from qwen36_moe_16gb_b200 import ops, synth
    from qwen36_moe_16gb_b200.kernel import B200Nvfp4MoEKernel, MoEConfig
    from qwen36_moe_16gb_b200.offload_layer import OffloadMoELayer
    from qwen36_moe_16gb_b200.slot_cache import SlotCache

    shape = synth.Shape(hidden=512, intermediate=256, num_experts=16, top_k=4, shared_intermediate=128)
    L, S, T = 4, 48, 300
    layout = B200Nvfp4MoEKernel().layout(MoEConfig(shape.num_experts, shape.hidden, shape.intermediate, shape.top_k))
    g = torch.Generator().manual_seed(21)
    sources = {r: [] for r in synth.ROLES}
    for _ in range(L):
        b = synth.make_banks(g, shape)
        for r in synth.ROLES:
            sources[r].append(b[r].pin_memory())
    x = torch.randn(T, shape.hidden, generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(shape.num_experts, generator=g)[:shape.top_k] for _ in range(T)]).to(torch.int32).cuda()
    w = torch.rand(T, shape.top_k, generator=g).cuda()
    want = [ops.prefill_experts(x, {r: sources[r][l].cuda() for r in synth.ROLES}, w, ids, check_status=True).clone()
            for l in range(L)]
    for hit_d2d in (False, True):
        cache = SlotCache(L, shape.num_experts, S, "cuda", prefill_overlap=True, prefill_hit_d2d=hit_d2d, layout=layout)
        cache.set_bank_sources(sources)
        for c in cache.bank_caches.values():
            c.view(torch.uint8).fill_(0xA5)
        if hit_d2d:
            # a previous decode left residents: the first 2E slots (the buffers' region) hold layers 3 and 2, then
            # three experts of layers 0 and 1 sit in slots outside the buffers
            for l in (3, 2):
                every = torch.arange(shape.num_experts, dtype=torch.int32, device="cuda")
                cache.ensure_experts(l, every)
                cache.copy_missing()
            for l in (0, 1):
                warm = torch.tensor([1, 5, 9], dtype=torch.int32, device="cuda")
                cache.ensure_experts(l, warm)
                cache.copy_missing()
            assert int((cache.slot_for_id >= 2 * shape.num_experts).sum()) == 6
        layers = [OffloadMoELayer(l, shape.num_experts, shape.top_k, cache) for l in range(L)]
        for l in range(L):
            got = layers[l].forward(x, w, ids.clone(), is_prefill=True)
            assert torch.equal(got.view(torch.int16), want[l].view(torch.int16)), (hit_d2d, l)
            if hit_d2d and l == 0:   # buffers 0 and 1 now hold layers 0 and 1: three residents each came device-to-device
                torch.cuda.synchronize()
                st = cache.prefill_transfer_stats()
                for b in (0, 1):
                    assert st[b]["d2d_rows"] == 3 and st[b]["h2d_rows"] == shape.num_experts - 3, st
        torch.cuda.synchronize()
    # short chunk: only the experts it routes to move
    cache = SlotCache(L, shape.num_experts, S, "cuda", prefill_overlap=True, layout=layout)
    cache.set_bank_sources(sources)
    cache.prefill_selected_max = 64
    for c in cache.bank_caches.values():
        c.view(torch.uint8).fill_(0xA5)
    xs, ws = x[:9].contiguous(), w[:9].contiguous()
    ids_s = ids[:9].contiguous()
    ids_s[:, :] = torch.tensor([2, 3, 7, 11], dtype=torch.int32)
    layers = [OffloadMoELayer(l, shape.num_experts, shape.top_k, cache) for l in range(L)]
    for l in range(L):
        ref = ops.prefill_experts(xs, {r: sources[r][l].cuda() for r in synth.ROLES}, ws, ids_s, check_status=True).clone()
        got = layers[l].forward(xs, ws, ids_s.clone(), is_prefill=True)
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), l
    torch.cuda.synchronize()
    assert cache.prefill_selected_chunks == 1
    st = cache.prefill_transfer_stats()
    assert st[1]["h2d_rows"] == 4 and st[1]["d2d_rows"] == 0
    e = shape.num_experts
    buf = cache.bank_caches["gate_up"][e:2 * e].cpu().view(torch.uint8)      # layer 3 went into buffer 1
    assert torch.equal(buf[7], sources["gate_up"][3][7].view(torch.uint8))
    assert bool((buf[0] == 0xA5).all())                                       # an expert nobody routed to stayed untouched


@pytest.mark.parametrize("per_layer", [True, False])
def test_banks_loaded_from_files_feed_the_cache_and_the_decode_kernels(per_layer, tmp_path):
    """Disk -> pinned record banks (`bank_files.load_records`) -> slot cache misses -> expert GEMVs: the result is
    the one the resident banks give."""
    from qwen36_moe_16gb_b200 import bank_files, ops
    from qwen36_moe_16gb_b200.kernel import B200Nvfp4MoEKernel, MoEConfig

    L, E, S, k = 3, 16, 20, 4
    shape = synth.Shape(hidden=1024, intermediate=512, num_experts=E, top_k=k, shared_intermediate=256)
    g = torch.Generator().manual_seed(3)
    layers = [synth.make_banks(g, shape) for _ in range(L)]
    bank_files.write_expert_banks(str(tmp_path), layers, per_layer=per_layer, shard_limit=1 << 20)
    layout = B200Nvfp4MoEKernel().layout(MoEConfig(E, shape.hidden, shape.intermediate, k))
    records, keep = bank_files.load_records(str(tmp_path), L, layout)
    assert all(b.residency.value == "pinned" for b in keep)
    cache = SlotCache(L, E, S, DEV, layout=layout)
    cache.set_record_sources(records)
    x = (torch.randn(2, shape.hidden, generator=g) * 0.5).bfloat16().to(DEV)
    w = torch.full((2, k), 1.0 / k, device=DEV)
    for layer in (0, 2, 1, 2):
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(2)]).to(torch.int32)
        want = ops.decode_experts(x, {r: t.to(DEV) for r, t in layers[layer].items()}, w, ids.to(DEV))
        slots = ids.to(DEV)
        cache.ensure_experts(layer, slots)
        cache.copy_missing()
        got = ops.decode_experts(x, cache.bank_dict(), w, slots)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    for b in keep:
        b.unpin()
