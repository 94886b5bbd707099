"""The dense bf16 linears of the block (router gate, shared expert gate_up + SwiGLU, shared down, gate logit) on
the tcgen05 dense GEMM against a plain fp32 PyTorch statement of the same op.

Tolerances: the kernel accumulates in fp32 and rounds once to bf16, so an output may differ from the fp32
reference rounded to bf16 by one bf16 step (2^-8 relative) where the two fp32 sums fall on either side of a rounding
boundary; the SwiGLU form rounds both halves to bf16 first, which can move its product by a few steps."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(t, n, k, seed, scale=0.05):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(t, k, generator=g, device="cuda")).bfloat16()
    w = (torch.randn(n, k, generator=g, device="cuda") * scale).bfloat16()
    return x, w


def _close(got, ref, steps=1.0):
    got, ref = got.float(), ref.float()
    tol = steps * (2.0 ** -8) * ref.abs() + 1e-3
    bad = (got - ref).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} outside tolerance, max err {(got - ref).abs().max().item()}"


@pytest.mark.parametrize("t,n,k", [(1, 8, 256), (77, 16, 512), (128, 256, 2048), (1000, 256, 2048), (300, 2048, 512),
                                   (513, 264, 128), (4096, 256, 2048)])
def test_dense_linear_matches_fp32(t, n, k):
    from qwen36_moe_16gb_b200 import ops

    x, w = _mk(t, n, k, 1)
    out = ops.dense_linear(x, w)
    torch.cuda.synchronize()
    assert int(ops.dense_status("cuda")) == 0
    _close(out, x.float() @ w.float().t())


def test_dense_linear_bias_is_added_before_the_rounding():
    from qwen36_moe_16gb_b200 import ops

    x, w = _mk(333, 256, 2048, 2)
    bias = torch.randn(256, device="cuda") * 3
    out = ops.dense_linear(x, w, bias)
    _close(out, x.float() @ w.float().t() + bias)


@pytest.mark.parametrize("t,si,k", [(5, 64, 256), (200, 128, 512), (1000, 512, 2048), (4096, 512, 2048), (129, 192, 1024)])
def test_gate_up_with_swiglu_matches_linear_then_activation(t, si, k):
    from qwen36_moe_16gb_b200 import ops

    x, w = _mk(t, 2 * si, k, 3, scale=0.03)
    out = ops.dense_linear(x, w, swiglu=True)
    torch.cuda.synchronize()
    assert int(ops.dense_status("cuda")) == 0
    hs = (x.float() @ w.float().t()).bfloat16().float()
    ref = torch.nn.functional.silu(hs[:, :si]) * hs[:, si:]
    got = out.float()
    # a half that lands on the other side of a bf16 boundary moves the product by about one step of that half
    tol = 3 * (2.0 ** -8) * (ref.abs() + hs[:, si:].abs() * (2.0 ** -8) + hs[:, :si].abs() * (2.0 ** -8)) + 2e-3
    assert ((got - ref).abs() <= tol).all(), (got - ref).abs().max().item()
    # the same activation kernel on the linear's own output is bit-identical where both halves rounded the same way
    same = ops.silu_and_mul(ops.dense_linear(x, w))
    assert (same == out).float().mean().item() == 1.0


def test_row_dot_matches_fp32():
    from qwen36_moe_16gb_b200 import ops

    x, w = _mk(1000, 1, 2048, 4)
    _close(ops.row_dot(x, w), x.float() @ w.float().t(), steps=2.0)


def test_dense_linear_rejects_bad_shapes():
    from qwen36_moe_16gb_b200 import ops

    x, w = _mk(16, 12, 256, 5)
    with pytest.raises(RuntimeError):
        ops.dense_linear(x, w)            # N % 8
    x, w = _mk(16, 16, 96, 5)
    with pytest.raises(RuntimeError):
        ops.dense_linear(x, w)            # K % 64
    assert ops.dense_linear(torch.empty((0, 256), dtype=torch.bfloat16, device="cuda"), _mk(1, 16, 256, 6)[1]).shape == (0, 16)


def test_block_prefill_path_launches_no_library_gemm():
    """The prefill block with the profiler on: every kernel in it is one of this library's."""
    from qwen36_moe_16gb_b200 import synth
    from qwen36_moe_16gb_b200.block import MoEBlock

    shape = synth.Shape(hidden=1024, intermediate=512, num_experts=16, top_k=4, shared_intermediate=256)
    layer = {k: v.cuda() for k, v in synth.make_layer(11, 256, shape).items()}
    blk = MoEBlock(layer["router_w"], layer["shared_gate_up"], layer["shared_down"], layer["shared_gate"], shape.top_k)
    banks = {r: layer[r] for r in synth.ROLES}
    blk.forward(layer["x"], banks, is_prefill=True)
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        blk.forward(layer["x"], banks, is_prefill=True)
        torch.cuda.synchronize()
    names = [e.key for e in prof.key_averages()]
    if not any("b200moe" in n for n in names):
        pytest.skip("the profiler recorded no kernel names on this machine")
    assert any("dense_gemm_kernel" in n for n in names), names
    foreign = [n for n in names if "b200moe" not in n and any(s in n.lower() for s in ("nvjet", "cutlass", "cublas", "gemm", "gemv"))]
    assert not foreign, foreign


def test_prefill_and_decode_router_logits_agree_to_one_rounding_step():
    """The prefill GEMM (tcgen05, k in 16-wide steps) and the decode GEMV (warp MMA, k split over lanes) add the same
    2048 products in different orders: both are within one bf16 step of the fp32 result, their top-8 sets agree
    wherever the 8th and 9th logits are further apart than that step, and most logits are bit-identical."""
    from qwen36_moe_16gb_b200 import ops, synth
    from qwen36_moe_16gb_b200.block import MoEBlock

    shape = synth.QWEN36
    layer = synth.make_layer(3, 8, shape, with_banks=False)
    d = {k: v.cuda() for k, v in layer.items()}
    blk = MoEBlock(d["router_w"], d["shared_gate_up"], d["shared_down"], d["shared_gate"], shape.top_k)
    x = d["x"]
    prefill = blk.router_logits(x).float()
    ws = ops.decode_block_workspace(8, shape.top_k, shape.hidden, shape.intermediate, shape.shared_intermediate, x.device)
    decode = ops.decode_dense_rows(x, blk.dense, 1, ws).float()
    exact = x.float() @ d["router_w"].float().t()
    step = 2.0 ** -8 * exact.abs() * 1.02 + 1e-6   # half a bf16 step of the value, plus the fp32 summation error
    assert ((prefill - exact).abs() <= step).all() and ((decode - exact).abs() <= step).all()
    same = (prefill == decode).float().mean().item()
    assert same > 0.9, same
    assert ((prefill - decode).abs() <= 2 * step).all()
    top_p, top_d = prefill.topk(9, dim=1), decode.topk(9, dim=1)
    for t in range(8):
        if (top_p.values[t, 7] - top_p.values[t, 8]) > 2 * step[t].max():
            assert set(top_p.indices[t, :8].tolist()) == set(top_d.indices[t, :8].tolist())
