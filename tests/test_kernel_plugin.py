"""Host logic of the MoE-kernel plugin (layout / pack / selection rules) -- no GPU."""
import pytest
import torch

from qwen36_moe_16gb_b200 import B200Nvfp4MoEKernel, MoEConfig, synth
from qwen36_moe_16gb_b200.slot_cache import SlotCache


def test_layout_matches_native_rows():
    cfg = MoEConfig(num_experts=256, hidden=2048, intermediate=512, top_k=8)
    lay = B200Nvfp4MoEKernel().layout(cfg)
    assert list(lay) == list(synth.ROLES)
    want = synth.bank_shapes(synth.QWEN36)
    for role, spec in lay.items():
        assert (tuple(spec.shape), spec.dtype) == want[role] and not spec.resident
    assert SlotCache.record_bytes(lay) == synth.QWEN36.expert_bytes == 1_781_760


def test_pack_from_separate_and_fused_pieces():
    cfg = MoEConfig(num_experts=4, hidden=256, intermediate=128, top_k=2)
    k = B200Nvfp4MoEKernel()
    e, h, i = 3, cfg.hidden, cfg.intermediate
    g = torch.Generator().manual_seed(0)
    u8 = lambda *s: torch.randint(0, 256, s, dtype=torch.uint8, generator=g)
    f8 = lambda *s: (torch.rand(*s, generator=g) + 0.25).to(torch.float8_e4m3fn)
    pieces = {"gate": u8(e, i, h // 2), "up": u8(e, i, h // 2), "gate_scale": f8(e, i, h // 16), "up_scale": f8(e, i, h // 16),
              "gate_global": torch.tensor([[0.5], [0.25], [1.0]]), "up_global": torch.tensor([[2.0], [4.0], [8.0]]),
              "down": u8(e, h, i // 2), "down_scale": f8(e, h, i // 16), "down_global": torch.tensor([0.75, 1.5, 3.0]).view(e, 1)}
    out = {r: torch.zeros((e, *spec.shape), dtype=spec.dtype) for r, spec in k.layout(cfg).items()}
    assert k.pack(pieces, cfg, out) == {}
    assert torch.equal(out["gate_up"][:, :i], pieces["gate"]) and torch.equal(out["gate_up"][:, i:], pieces["up"])
    assert torch.equal(out["gate_up_scale"].view(torch.uint8)[:, i:], pieces["up_scale"].view(torch.uint8))
    assert out["gate_up_global"][1, :i].unique().tolist() == [0.25] and out["gate_up_global"][1, i:].unique().tolist() == [4.0]
    assert out["down_global"][2].unique().tolist() == [3.0]
    fused = {"gate_up": out["gate_up"].clone(), "gate_up_scale": out["gate_up_scale"].clone(),
             "gate_up_global": out["gate_up_global"].clone(), "down": pieces["down"], "down_scale": pieces["down_scale"],
             "down_global": out["down_global"].clone()}
    out2 = {r: torch.zeros_like(t) for r, t in out.items()}
    k.pack(fused, cfg, out2)
    for r in out:
        assert torch.equal(out[r].view(torch.uint8), out2[r].view(torch.uint8))


@pytest.mark.parametrize("kw,fragment", [
    (dict(strategy="resident"), "resident"), (dict(tp_size=2), "TP > 1"), (dict(decode_target="cpu"), "CPU executor"),
    (dict(has_bias=True), "bias"), (dict(activation="swigluoai", alpha=1.702, limit=7.0), "plain-silu"),
    (dict(apply_router_weight_on_input=True), "router weight"), (dict(hidden=2000), "do not tile")])
def test_unusable_reasons(kw, fragment):
    base = dict(num_experts=256, hidden=2048, intermediate=512, top_k=8)
    base.update(kw)
    reason = B200Nvfp4MoEKernel().unusable_reason(MoEConfig(**base))
    assert reason is not None and fragment in reason
    assert B200Nvfp4MoEKernel().unusable_reason(MoEConfig(256, 2048, 512, 8)) in (None, "needs an sm_100 device")


def test_slot_cache_geometry_errors():
    with pytest.raises(ValueError):
        SlotCache(2, 8, 4, "cpu", host_tables=True)
    with pytest.raises(ValueError):
        SlotCache(2, 8, 16, "cpu", host_tables=True, max_slots=12)
    with pytest.raises(AssertionError):
        SlotCache(2, 8, 12, "cpu", host_tables=True, prefill_overlap=True)  # needs 2 * num_experts slots
    c = SlotCache(2, 8, 16, "cpu", host_tables=True)
    with pytest.raises(ValueError):
        c.validate_rebuild(4)
    c.rebuild(24)
    assert c.cache_size == 24 and c.id_of_slot.numel() == 24 and int(c.step) == 0


def test_plugin_types_agree_with_the_reference_interface_when_it_is_present():
    """Field-for-field agreement of the mirrored plugin types with the reference's own, read from the reference's
    source text (its module needs packages that are not installed; skipped where the checkout is absent)."""
    import ast
    import dataclasses
    import pathlib

    src = pathlib.Path("/root/reference/freetoken/python/freetoken/layers/quantization/moe/base.py")
    if not src.exists():
        pytest.skip("reference checkout not present")
    tree = ast.parse(src.read_text())
    classes = {n.name: n for n in tree.body if isinstance(n, ast.ClassDef)}
    from qwen36_moe_16gb_b200 import kernel

    for name in ("MoEConfig", "BankSpec", "ExpertView"):
        theirs = [st.target.id for st in classes[name].body if isinstance(st, ast.AnnAssign) and isinstance(st.target, ast.Name)]
        ours = [f.name for f in dataclasses.fields(getattr(kernel, name))]
        assert ours == theirs, (name, ours, theirs)
    theirs = {st.name for st in classes["MoEKernel"].body if isinstance(st, ast.FunctionDef)}
    for method in ("unusable_reason", "worth_it", "slot_limit", "layout", "pack", "apply"):
        assert method in theirs and callable(getattr(kernel.B200Nvfp4MoEKernel, method)), method
