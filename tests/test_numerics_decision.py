"""Why the prefill GEMM multiplies exact 16-bit operands instead of block-scaled FP4 activations.

The parity gate (max-abs 2e-2, rel-L2 1e-3 against the reference's bf16 result) is set on the production-faithful
oracle.  This test reproduces, on CPU, the measurement behind the decision: quantising the ACTIVATIONS to NVFP4
(E2M1 codes, one E4M3 scale per 16 values) as `tcgen05.mma kind::mxf4nvf4` would need misses the gate even when
the quantisation residual is fed back through one, two or three extra MMA terms -- and with four terms the FP4 path
no longer has more throughput than the 16-bit path.  A small layer keeps it to seconds; the errors do not depend on
the layer size (they are per-element rounding errors of the activations).
"""
import torch

import oracle
from qwen36_moe_16gb_b200 import synth

E2M1_MAGS = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
SHAPE = synth.Shape(hidden=512, intermediate=256, num_experts=8, top_k=2, shared_intermediate=128)


def _quantise_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest E2M1 code under an E4M3 scale per 16 values (scale = block max / 6)."""
    blocks = x.reshape(-1, 16)
    scale = (blocks.abs().amax(1, keepdim=True) / 6).to(torch.float8_e4m3fn).float().clamp_min(2.0 ** -9)
    y = blocks / scale
    idx = (y.abs().unsqueeze(-1) - E2M1_MAGS).abs().argmin(-1)
    return (E2M1_MAGS[idx] * y.sign() * scale).reshape(x.shape)


def _residual_terms(x: torch.Tensor, n: int) -> torch.Tensor:
    rest, acc = x.clone(), torch.zeros_like(x)
    for _ in range(n):
        t = _quantise_nvfp4(rest)
        acc += t
        rest = rest - t
    return acc


def test_fp4_activations_miss_the_parity_gate_with_up_to_four_terms():
    layer = synth.make_layer(0, 64, SHAPE)
    w, ids = oracle.router_topk(synth.router_logits(layer["x"], layer["router_w"]), SHAPE.top_k)
    want = oracle.moe_experts_bf16(layer["x"], layer, w, ids)
    errs = []
    for n in (1, 2, 3, 4):
        xa = _residual_terms(layer["x"].float(), n)
        got = oracle.moe_experts_bf16(xa, layer, w, ids)
        errs.append(oracle.error_metrics(got, want)[1])
    assert errs[0] > errs[1] > errs[2] > errs[3]          # every term helps ...
    assert all(e > 1e-3 for e in errs), errs               # ... and none reaches the gate
    assert errs[0] > 5e-2 and errs[3] > 1.5e-3, errs


def test_exact_16bit_operands_meet_it():
    """The path that is shipped: weights dequantised exactly (E2M1 x E4M3 has at most 6 significant bits), activations
    unchanged (fp16 rows rescaled by a power of two hold every bf16 value exactly) -- the only difference left to
    the oracle is the accumulation order, modelled here by a float64 accumulation."""
    layer = synth.make_layer(1, 64, SHAPE)
    w, ids = oracle.router_topk(synth.router_logits(layer["x"], layer["router_w"]), SHAPE.top_k)
    want = oracle.moe_experts_bf16(layer["x"], layer, w, ids)
    x = layer["x"].float()
    scale = 2.0 ** (14 - torch.floor(torch.log2(x.abs().amax(1, keepdim=True))))
    assert torch.equal((x * scale).half().float() / scale, x)           # the rescaled fp16 row is exact
    gu = oracle.dequant_nvfp4(layer["gate_up"][0], layer["gate_up_scale"][0])
    assert torch.equal(gu.half().float(), gu)                            # the unpacked weights are exact in fp16
    max_abs, rel_l2 = oracle.error_metrics(oracle.moe_experts_bf16(layer["x"].double().float(), layer, w, ids), want)
    assert max_abs == 0.0 and rel_l2 == 0.0
