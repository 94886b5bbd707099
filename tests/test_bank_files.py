"""Expert banks on disk: this package's reader/writer/loaders against two directories written by the reference's own
writer (tests/golden/bank_files, generator script beside them), plus round trips and index validation."""
import filecmp
import importlib.util
import json
import pathlib

import pytest
import torch

from qwen36_moe_16gb_b200 import bank_files as bf
from qwen36_moe_16gb_b200.kernel import B200Nvfp4MoEKernel, MoEConfig
from qwen36_moe_16gb_b200.slot_cache import SlotCache

GOLDEN = pathlib.Path(__file__).parent / "golden"
spec = importlib.util.spec_from_file_location("make_bank_files", GOLDEN / "make_bank_files.py")
gen = importlib.util.module_from_spec(spec)
spec.loader.exec_module(gen)


@pytest.fixture(scope="module")
def layers():
    return gen.bank_layers()


@pytest.mark.parametrize("form", ["per_layer", "flat"])
def test_reader_returns_the_reference_writers_tensors(form, layers):
    path = str(GOLDEN / "bank_files" / form)
    assert bf.is_bank_directory(path)
    with bf.BankFileReader(path) as r:
        assert r.meta("quant_format") == "nvfp4" and r.meta(bf.NUM_LAYERS_KEY) == gen.LAYERS
        for name, want in gen.dense_extras().items():
            got = r.tensor(name)
            assert got.dtype == want.dtype and got.shape == want.shape and torch.equal(got, want)
        assert [e["name"] for e in r.entries("weight")] == list(gen.dense_extras())
        assert len(r.entries(bf.BANK_KIND)) == (6 * gen.LAYERS if form == "per_layer" else 6)
    loaded = bf.load_banks(path, gen.LAYERS, pin=False)
    assert loaded.quant_format == "nvfp4" and loaded.num_experts == gen.EXPERTS
    assert set(loaded.sources) == set(gen.ROLES)
    for role in gen.ROLES:
        for l in range(gen.LAYERS):
            got, want = loaded.sources[role][l], layers[l][role]
            assert got.dtype == want.dtype and got.shape == want.shape
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), (role, l)


@pytest.mark.parametrize("form", ["per_layer", "flat"])
def test_writer_produces_the_reference_writers_bytes(form, layers, tmp_path):
    """Same tensors in the same order -> the same index and the same shard files, byte for byte."""
    w = bf.BankFileWriter(str(tmp_path), gen.SHARD_LIMIT)
    for name, t in gen.dense_extras().items():
        w.add_tensor(name, t, "weight")
    for role, stored in zip(gen.ROLES, gen.STORED):
        if form == "per_layer":
            for l in range(gen.LAYERS):
                w.add_tensor(bf.layer_entry_name(stored, l), layers[l][role], bf.BANK_KIND)
        else:
            w.add_tensor(stored, torch.cat([b[role] for b in layers]), bf.BANK_KIND)
    w.finalize({"quant_format": "nvfp4", bf.NUM_LAYERS_KEY: gen.LAYERS})
    ref = GOLDEN / "bank_files" / form
    mine = json.loads((tmp_path / bf.INDEX_NAME).read_text())
    assert mine == json.loads((ref / bf.INDEX_NAME).read_text())
    for sh in mine["shards"]:
        assert filecmp.cmp(tmp_path / sh["file"], ref / sh["file"], shallow=False), sh["file"]


@pytest.mark.parametrize("per_layer", [True, False])
def test_record_loader_builds_the_slot_caches_host_banks(per_layer, layers, tmp_path):
    bf.write_expert_banks(str(tmp_path), layers, per_layer=per_layer, shard_limit=8192)
    layout = B200Nvfp4MoEKernel().layout(MoEConfig(gen.EXPERTS, gen.HIDDEN, gen.INTER, 2))
    records, keep = bf.load_records(str(tmp_path), gen.LAYERS, layout, pin=False)
    assert len(records) == gen.LAYERS and records[0].shape == (gen.EXPERTS, SlotCache.record_bytes(layout))
    for l, rec in enumerate(records):
        views = SlotCache.record_views(rec, layout)
        for role in layout:
            assert torch.equal(views[role].view(torch.uint8), layers[l][role].view(torch.uint8)), (l, role)
    assert all(b.residency.value == "pageable" for b in keep)


def test_tensors_larger_than_a_shard_span_shards_and_small_ones_never_split(tmp_path):
    g = torch.Generator().manual_seed(0)
    big = torch.randint(0, 256, (3 * 8192 + 100,), dtype=torch.uint8, generator=g)
    small = torch.randint(0, 256, (5000,), dtype=torch.uint8, generator=g)
    w = bf.BankFileWriter(str(tmp_path), 8192)
    w.add_tensor("a", small)
    w.add_tensor("b", small * 2)          # 5000 + 5000 > 8192: starts a new shard instead of splitting
    w.add_tensor("big", big)
    w.add_tensor("empty", torch.empty(0, 4))
    w.add_tensor("tail", small[:7])
    idx = w.finalize()
    offs = {t["name"]: t["global_off"] for t in idx["tensors"]}
    starts = [s["global_off"] for s in idx["shards"]]
    assert offs["b"] in starts and all(o % bf.ALIGN == 0 for o in offs.values())
    with bf.BankFileReader(str(tmp_path), workers=3) as r:
        r.CHUNK = 4096                     # several jobs per piece
        assert len(r.pieces(offs["big"], big.numel())) >= 3
        assert torch.equal(r.tensor("big"), big) and torch.equal(r.tensor("b"), small * 2)
        assert r.tensor("empty").shape == (0, 4) and torch.equal(r.tensor("tail"), small[:7])
        with pytest.raises(ValueError):
            r.pieces(idx["total_bytes"] - 10, 20)


def test_direct_reads_fall_back_where_the_file_system_refuses(tmp_path, layers):
    bf.write_expert_banks(str(tmp_path), layers)
    with bf.BankFileReader(str(tmp_path), direct=True) as r:      # O_DIRECT or page cache: same bytes either way
        buf, head = r.read_window(r.tensors["down_packed#L00001"]["global_off"] + 5, 1000)
        want = layers[1]["down"].reshape(-1)[5:1005]
        assert torch.equal(torch.frombuffer(buf, dtype=torch.uint8, count=1000, offset=head), want)


def _rewrite(path, fn):
    f = pathlib.Path(path) / bf.INDEX_NAME
    idx = json.loads(f.read_text())
    fn(idx)
    f.write_text(json.dumps(idx))


@pytest.mark.parametrize("damage,word", [
    (lambda i: i.update(version=2), "version"),
    (lambda i: i.update(align=512), "align"),
    (lambda i: i["shards"][1].update(global_off=i["shards"][1]["global_off"] + 4096), "gap"),
    (lambda i: i["shards"][0].update(file="other.ftw"), "file name"),
    (lambda i: i["tensors"].append(dict(i["tensors"][0])), "duplicate"),
    (lambda i: i["tensors"][2].update(nbytes=i["tensors"][2]["nbytes"] + 1), "nbytes"),
    (lambda i: i["tensors"][3].update(global_off=i["tensors"][2]["global_off"]), "overlaps"),
    (lambda i: i["tensors"][1].update(dtype="float7"), "dtype"),
    (lambda i: i.update(total_bytes=i["total_bytes"] + 4096), "cover"),
])
def test_damaged_indexes_are_refused_before_any_shard_is_read(damage, word, layers, tmp_path):
    bf.write_expert_banks(str(tmp_path), layers, shard_limit=16384)
    _rewrite(tmp_path, damage)
    with pytest.raises(bf.BankIndexError, match=word):
        bf.read_index(str(tmp_path))


def test_loader_refuses_mismatched_layer_counts_and_shapes(layers, tmp_path):
    bf.write_expert_banks(str(tmp_path), layers)
    with pytest.raises(RuntimeError):
        bf.load_banks(str(tmp_path), gen.LAYERS + 1, pin=False)
    layout = B200Nvfp4MoEKernel().layout(MoEConfig(gen.EXPERTS, gen.HIDDEN * 2, gen.INTER, 2))
    with pytest.raises(bf.BankIndexError):
        bf.load_records(str(tmp_path), gen.LAYERS, layout, pin=False)
    empty = tmp_path / "none"
    bf.BankFileWriter(str(empty)).finalize()
    assert bf.load_banks(str(empty), 1, pin=False) is None
