"""Decoder-layer glue around the block: fused residual add + RMSNorm against the oracle, and the layer wrapper."""
import pytest
import torch

import oracle
from qwen36_moe_16gb_b200 import ops, synth
from qwen36_moe_16gb_b200.block import DecoderLayerMoE, MoEBlock

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close_bf16(got, want, ulps=1):
    g, w = got.float().cpu(), want.float()
    tol = w.abs() * 2.0 ** -8 * ulps + 1e-30
    return bool(((g - w).abs() <= tol + w.abs() * 2.0 ** -8).all())


@pytest.mark.parametrize("rows,h,plus_one", [(1, 2048, False), (37, 2048, False), (300, 1024, True), (5, 8, False)])
def test_fused_add_rmsnorm_matches_oracle(rows, h, plus_one):
    g = torch.Generator().manual_seed(rows * 7 + h)
    x = (torch.randn(rows, h, generator=g) * 3).to(torch.bfloat16)
    r = (torch.randn(rows, h, generator=g) * 5).to(torch.bfloat16)
    w = (torch.randn(h, generator=g) * 0.5 + (0.0 if plus_one else 1.0)).to(torch.bfloat16)
    want_y, want_r = oracle.fused_add_rmsnorm(x, r, w, 1e-6, plus_one)
    xd, rd = x.to(DEV), r.to(DEV)
    ops.fused_add_rmsnorm(xd, rd, w.to(DEV), 1e-6, plus_one)
    assert torch.equal(rd.cpu().view(torch.int16), want_r.view(torch.int16))      # the residual sum: one exact rounding
    assert _close_bf16(xd, want_y)                                                 # the norm: one bf16 ulp (sum order)
    got = ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, plus_one)
    assert _close_bf16(got, oracle.rmsnorm(x, w, 1e-6, plus_one))


def test_decoder_layer_wrapper_runs_block_on_normed_sum():
    shape = synth.QWEN36
    layer = synth.make_layer(0, 16)
    d = {k: v.to(DEV) for k, v in layer.items()}
    blk = MoEBlock(d["router_w"], d["shared_gate_up"], d["shared_down"], d["shared_gate"], shape.top_k)
    g = torch.Generator().manual_seed(5)
    norm_w = (torch.randn(shape.hidden, generator=g) * 0.1 + 1.0).to(torch.bfloat16)
    mixer = (torch.randn(16, shape.hidden, generator=g)).to(torch.bfloat16)
    resid = layer["x"].clone()
    want_h, want_r = oracle.fused_add_rmsnorm(mixer, resid, norm_w)
    glue = DecoderLayerMoE(blk, norm_w.to(DEV))
    md, rd = mixer.to(DEV), resid.to(DEV)
    banks = {r: d[r] for r in synth.ROLES}
    out, r_out = glue.forward(md, rd, banks, is_prefill=True)
    assert torch.equal(r_out.cpu().view(torch.int16), want_r.view(torch.int16))
    # the block sees the kernel's normed rows: compare with the block run on exactly those rows
    direct = blk.forward(md.clone(), banks, is_prefill=True)
    assert torch.equal(out.view(torch.int16), direct.view(torch.int16))
    assert _close_bf16(md, want_h)
