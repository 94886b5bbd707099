"""Tensor-level wrappers over the C ABI: one function per entry point, launched on torch's current stream."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import Banks, Dense, SlotTables, check, lib, ptr, stream_ptr

ROLES = ("gate_up", "gate_up_scale", "gate_up_global", "down", "down_scale", "down_global")


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise _lib.B200MoeError("b200moe kernels take CUDA tensors only (no CPU fallback)")


def fused_topk_softmax(gating_output: torch.Tensor, topk: int, renormalize: bool,
                       num_token_non_padded: torch.Tensor | None = None):
    """Same signature and results as the reference's ``fused_topk_softmax``
    (``freetoken/python/freetoken/kernel/triton/moe_router.py:109``)."""
    assert gating_output.ndim == 2, "gating_output must be 2D"
    _need_cuda(gating_output)
    if gating_output.dtype not in (torch.bfloat16, torch.float32):
        gating_output = gating_output.float()
    if gating_output.stride(1) != 1:
        gating_output = gating_output.contiguous()
    m, n = gating_output.shape
    weights = torch.empty((m, topk), dtype=torch.float32, device=gating_output.device)
    ids = torch.empty((m, topk), dtype=torch.int32, device=gating_output.device)
    lim = num_token_non_padded
    if lim is not None:
        assert lim.dtype in (torch.int32, torch.int64) and lim.is_cuda
    check(lib().b200moe_router_topk(ptr(gating_output), 0 if gating_output.dtype == torch.bfloat16 else 1,
                                    gating_output.stride(0), m, n, topk, int(renormalize), ptr(lim),
                                    int(lim is not None and lim.dtype == torch.int64), ptr(weights), ptr(ids),
                                    stream_ptr()), "b200moe_router_topk")
    return weights, ids


def fused_topk(hidden_states, gating_output, topk, renormalize, num_token_non_padded=None):
    """``freetoken/python/freetoken/moe/fused.py:33-44``."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    return fused_topk_softmax(gating_output, topk, renormalize, num_token_non_padded)


def align_sizes(numel: int, block: int, num_experts: int) -> tuple[int, int]:
    cap = numel * block if numel < num_experts + 1 else numel + (num_experts + 1) * (block - 1)
    return cap, (cap + block - 1) // block


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int, with_routes: bool = False):
    """``freetoken/python/freetoken/moe/fused.py:47`` -- same three buffers, deterministic in-expert order.
    ``with_routes`` also returns (sorted_routes [numel], expert_offsets [num_experts+2])."""
    assert topk_ids.dtype == torch.int32 and topk_ids.is_contiguous()
    _need_cuda(topk_ids)
    dev = topk_ids.device
    numel = topk_ids.numel()
    cap, nblocks = align_sizes(numel, block_size, num_experts)
    sorted_ids = torch.empty((cap,), dtype=torch.int32, device=dev)
    expert_ids = torch.empty((nblocks,), dtype=torch.int32, device=dev)
    post = torch.empty((1,), dtype=torch.int32, device=dev)
    routes = torch.empty((max(numel, 1),), dtype=torch.int32, device=dev)
    offsets = torch.empty((num_experts + 2,), dtype=torch.int32, device=dev)
    wbytes = lib().b200moe_permute_workspace_bytes(numel, num_experts)
    ws = torch.empty((wbytes,), dtype=torch.uint8, device=dev)
    check(lib().b200moe_permute(ptr(topk_ids), numel, num_experts, block_size, ptr(sorted_ids), cap, ptr(expert_ids),
                                nblocks, ptr(post), ptr(routes), ptr(offsets), ptr(ws), wbytes, stream_ptr()),
          "b200moe_permute")
    if with_routes:
        return sorted_ids, expert_ids, post, routes[:numel], offsets
    return sorted_ids, expert_ids, post


def make_banks(tensors: dict[str, torch.Tensor]) -> tuple[Banks, tuple]:
    """Bank descriptor from role -> ``[S, ...]`` tensors; returns (struct, keep-alive tuple)."""
    t = [tensors[r] for r in ROLES]
    _need_cuda(*t)
    gu, gus, gug, dn, dns, dng = t
    s, two_i, h2 = gu.shape
    h, i = h2 * 2, two_i // 2
    if gus.shape != (s, two_i, h // 16) or gug.shape != (s, two_i) or dn.shape != (s, h, i // 2) \
            or dns.shape != (s, h, i // 16) or dng.shape != (s, h):
        raise ValueError("NVFP4 bank shapes do not match the native layout")
    if gug.dtype != torch.float32 or dng.dtype != torch.float32:
        raise ValueError("global scales must be fp32 (one per output row)")
    strides = []
    for x in t:
        if not x[0].is_contiguous():
            raise ValueError("every slot of a bank must be contiguous")
        # dense [S, ...] banks, or slots strided through one contiguous per-slot record
        strides.append(0 if x.is_contiguous() else x.stride(0) * x.element_size())
    b = Banks(*(x.data_ptr() for x in t), s, h, i)
    for r, v in enumerate(strides):
        b.slot_stride[r] = v
    return b, tuple(t)


def make_dense(router_w, shared_gate_up, shared_down, shared_gate) -> tuple[Dense, tuple]:
    t = (router_w, shared_gate_up, shared_down, shared_gate)
    _need_cuda(*t)
    for x in t:
        assert x.dtype == torch.bfloat16 and x.is_contiguous()
    return Dense(*(x.data_ptr() for x in t), router_w.shape[0], shared_gate_up.shape[0] // 2), t


_ws_cache: dict[tuple, torch.Tensor] = {}


def _workspace(kind: str, nbytes: int, device: torch.device) -> torch.Tensor:
    """Per (kind, device, stream) scratch, grown on demand and reused (stream-ordered reuse is safe)."""
    key = (kind, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty((max(nbytes, 256),), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def decode_experts(x, banks: dict[str, torch.Tensor], topk_weights, topk_ids, out=None):
    """Routed experts for 1..8 tokens; ``topk_ids`` index bank rows (slot ids)."""
    _need_cuda(x, topk_weights, topk_ids)
    b, keep = make_banks(banks)
    m, h = x.shape
    k = topk_ids.shape[1]
    out = torch.empty_like(x) if out is None else out
    nbytes = lib().b200moe_decode_workspace_bytes(m, k, h, b.intermediate, 0, 0)
    ws = _workspace("decode", nbytes, x.device)
    check(lib().b200moe_decode_experts(ptr(x), C.byref(b), ptr(topk_weights), ptr(topk_ids), m, k, ptr(out), ptr(ws),
                                       ws.numel(), stream_ptr()), "b200moe_decode_experts")
    return out


def decode_block_route(x, dense: tuple[Dense, tuple], top_k: int, ws: torch.Tensor):
    d, _ = dense
    m, h = x.shape
    logits = torch.empty((m, d.num_experts), dtype=torch.bfloat16, device=x.device)
    w = torch.empty((m, top_k), dtype=torch.float32, device=x.device)
    ids = torch.empty((m, top_k), dtype=torch.int32, device=x.device)
    check(lib().b200moe_decode_block_route(ptr(x), C.byref(d), m, h, top_k, ptr(logits), ptr(w), ptr(ids), ptr(ws),
                                           ws.numel(), stream_ptr()), "b200moe_decode_block_route")
    return logits, w, ids


def decode_dense_rows(x, dense: tuple[Dense, tuple], segment_mask: int, ws: torch.Tensor, logits=None):
    """The dense rows of a decode layer by segment (1: router logits, returned; 2: shared gate_up and 4: shared gate
    logit, both left in ``ws`` for :func:`decode_block_experts`)."""
    d, _ = dense
    m, h = x.shape
    if logits is None and (segment_mask & 1):
        logits = torch.empty((m, d.num_experts), dtype=torch.bfloat16, device=x.device)
    check(lib().b200moe_decode_dense_rows(ptr(x), C.byref(d), m, h, segment_mask, ptr(logits), ptr(ws), ws.numel(),
                                          stream_ptr()), "b200moe_decode_dense_rows")
    return logits


def decode_block_experts(x, banks: tuple[Banks, tuple], dense: tuple[Dense, tuple], w, ids, ws, out=None):
    b, _ = banks
    d, _ = dense
    m, _ = x.shape
    out = torch.empty_like(x) if out is None else out
    check(lib().b200moe_decode_block_experts(ptr(x), C.byref(b), C.byref(d), ptr(w), ptr(ids), m, ids.shape[1], ptr(out),
                                             ptr(ws), ws.numel(), stream_ptr()), "b200moe_decode_block_experts")
    return out


def decode_block(x, banks: tuple[Banks, tuple], dense: tuple[Dense, tuple], top_k: int, ws, out=None):
    """Whole block for 1..8 tokens with every expert resident: three launches, routing fused into the first
    expert GEMM.  Returns (out, logits, topk_weights, topk_ids)."""
    b, _ = banks
    d, _ = dense
    m, _ = x.shape
    out = torch.empty_like(x) if out is None else out
    logits = torch.empty((m, d.num_experts), dtype=torch.bfloat16, device=x.device)
    w = torch.empty((m, top_k), dtype=torch.float32, device=x.device)
    ids = torch.empty((m, top_k), dtype=torch.int32, device=x.device)
    check(lib().b200moe_decode_block(ptr(x), C.byref(b), C.byref(d), m, top_k, ptr(logits), ptr(w), ptr(ids), ptr(out),
                                     ptr(ws), ws.numel(), stream_ptr()), "b200moe_decode_block")
    return out, logits, w, ids


def decode_block_workspace(m: int, top_k: int, hidden: int, intermediate: int, shared_intermediate: int, device):
    n = lib().b200moe_decode_workspace_bytes(m, top_k, hidden, intermediate, shared_intermediate, 0)
    return torch.empty((n,), dtype=torch.uint8, device=device)


class PrefillStatus(RuntimeError):
    pass


STAGE_PLAN, STAGE_GEMM1, STAGE_GEMM2, STAGE_COMBINE, STAGE_ALL, STAGE_ROUTE_ORDER = 1, 2, 4, 8, 15, 16


def prefill_experts(x, banks: dict[str, torch.Tensor], topk_weights, topk_ids, shared=None, shared_gate_logit=None,
                    out=None, check_status: bool = False, stages: int = STAGE_ALL):
    """Routed experts for any T through the tcgen05 grouped GEMM; ``topk_ids`` index bank rows."""
    _need_cuda(x, topk_weights, topk_ids)
    b, keep = make_banks(banks)
    t, h = x.shape
    k = topk_ids.shape[1]
    out = torch.empty_like(x) if out is None else out
    nbytes = lib().b200moe_prefill_workspace_bytes(t, k, h, b.intermediate, b.num_slots)
    ws = _workspace("prefill", nbytes + 64, x.device)
    status = ws[nbytes:nbytes + 16].view(torch.int32)
    check(lib().b200moe_prefill_stages(ptr(x), C.byref(b), ptr(topk_weights), ptr(topk_ids), t, k, ptr(shared),
                                       ptr(shared_gate_logit), ptr(out), ptr(ws), nbytes, ptr(status), stages,
                                       stream_ptr()), "b200moe_prefill_stages")
    if check_status:
        code = int(status[0].item())
        if code:
            raise PrefillStatus(f"grouped GEMM gave up on a bounded wait (status {code}); the output is invalid")
    return out


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    rows, d2 = x.reshape(-1, x.shape[-1]).shape
    out = torch.empty((*x.shape[:-1], d2 // 2), dtype=x.dtype, device=x.device)
    check(lib().b200moe_silu_and_mul(ptr(x), ptr(out), rows, d2 // 2, stream_ptr()), "b200moe_silu_and_mul")
    return out


def shared_epilogue(routed, shared, gate):
    """``routed + shared * sigmoid(gate)`` with torch's bf16 roundings, one launch."""
    _need_cuda(routed, shared, gate)
    t, h = routed.shape
    out = torch.empty_like(routed)
    check(lib().b200moe_shared_epilogue(ptr(routed), ptr(shared.contiguous()), ptr(gate.contiguous()), ptr(out), t, h,
                                        stream_ptr()), "b200moe_shared_epilogue")
    return out


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                      plus_one: bool = False) -> None:
    """In place: ``residual += x`` (rounded once to bf16), ``x = rmsnorm(residual_fp32) * (weight [+ 1])``."""
    _need_cuda(x, residual, weight)
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and residual.is_contiguous() and x.shape == residual.shape
    rows, h = x.reshape(-1, x.shape[-1]).shape
    check(lib().b200moe_fused_add_rmsnorm(ptr(x), ptr(residual), ptr(weight), float(eps), int(plus_one), rows, h,
                                          stream_ptr()), "b200moe_fused_add_rmsnorm")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, plus_one: bool = False, out=None) -> torch.Tensor:
    _need_cuda(x, weight)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    rows, h = x.reshape(-1, x.shape[-1]).shape
    out = torch.empty_like(x) if out is None else out
    check(lib().b200moe_rmsnorm(ptr(x), ptr(weight), ptr(out), float(eps), int(plus_one), rows, h, stream_ptr()),
          "b200moe_rmsnorm")
    return out


_dense_status: dict = {}


def dense_status(device) -> torch.Tensor:
    """The int32 word the dense GEMM sets when one of its bounded waits ran out (zero in a correct run)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _dense_status:
        _dense_status[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _dense_status[key]


def dense_linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, swiglu: bool = False, out=None) -> torch.Tensor:
    """``bf16(x @ w.T + bias)`` on the tensor cores; with ``swiglu`` the rows of ``w`` are gate rows then up rows and the
    result is ``silu(gate) * up`` (each half rounded to bf16 first, as the linear followed by the activation gives)."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    t, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n
    cols = n // 2 if swiglu else n
    out = torch.empty((t, cols), dtype=torch.bfloat16, device=x.device) if out is None else out
    assert out.is_contiguous() and out.shape == (t, cols)
    check(lib().b200moe_dense_linear(ptr(x), ptr(w), None if bias is None else ptr(bias), ptr(out), t, n, k, int(swiglu),
                                     ptr(dense_status(x.device)), stream_ptr()), "b200moe_dense_linear")
    return out


def row_dot(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``bf16(x @ w.T)`` for a single weight row: [T, K] x [1, K] -> [T, 1]."""
    _need_cuda(x, w)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    t, k = x.shape
    assert w.numel() == k
    out = torch.empty((t, 1), dtype=torch.bfloat16, device=x.device)
    check(lib().b200moe_row_dot(ptr(x), ptr(w), ptr(out), t, k, stream_ptr()), "b200moe_row_dot")
    return out


def sum_routes(ic3: torch.Tensor) -> torch.Tensor:
    _need_cuda(ic3)
    t, k, h = ic3.shape
    out = torch.empty((t, h), dtype=ic3.dtype, device=ic3.device)
    check(lib().b200moe_sum_routes(ptr(ic3.contiguous()), ptr(out), t, k, h, stream_ptr()), "b200moe_sum_routes")
    return out


def prefill_route_rows(x, banks: dict[str, torch.Tensor], topk_weights, topk_ids):
    """Per-route expert outputs ``ic3 [T, top_k, H]`` bf16 (already multiplied by the router weight), without the
    sum over routes.  Rows of routes with an id outside the banks are NOT written.  The result is a view into the
    stream's prefill workspace: consume it before the next prefill call on the same stream."""
    _need_cuda(x, topk_weights, topk_ids)
    b, keep = make_banks(banks)
    t, h = x.shape
    k = topk_ids.shape[1]
    nbytes = lib().b200moe_prefill_workspace_bytes(t, k, h, b.intermediate, b.num_slots)
    ws = _workspace("prefill", nbytes + 64, x.device)
    status = ws[nbytes:nbytes + 16].view(torch.int32)
    check(lib().b200moe_prefill_stages(ptr(x), C.byref(b), ptr(topk_weights), ptr(topk_ids), t, k, None, None, ptr(x),
                                       ptr(ws), nbytes, ptr(status), STAGE_PLAN | STAGE_GEMM1 | STAGE_GEMM2 | STAGE_ROUTE_ORDER,
                                       stream_ptr()), "b200moe_prefill_stages")
    off = lib().b200moe_prefill_ic3_offset(t, k, h, b.intermediate, b.num_slots)
    return ws[off:off + t * k * h * 2].view(torch.bfloat16).view(t, k, h)


def combine_routes(ic3, topk_ids=None, num_slots: int = 0, shared=None, shared_gate_logit=None, out=None):
    """``out[t] = bf16(sum_k ic3[t,k])`` skipping routes with ids outside [0, num_slots), then the optional merge."""
    _need_cuda(ic3)
    t, k, h = ic3.shape
    out = torch.empty((t, h), dtype=ic3.dtype, device=ic3.device) if out is None else out
    check(lib().b200moe_combine_routes(ptr(ic3), ptr(topk_ids), num_slots, t, k, h, ptr(shared), ptr(shared_gate_logit),
                                       ptr(out), stream_ptr()), "b200moe_combine_routes")
    return out


def prefill_ep_routes(x, local_banks: dict[str, torch.Tensor], weights, local_ids, first_token: int,
                      peer_ic3_ptrs: torch.Tensor, world: int, tokens_per_rank: int):
    """Owner-side half of expert-parallel prefill for a slice of the box's tokens (first row = global token
    ``first_token``): grouped GEMMs for the local experts; per-route rows are stored by the kernel into the home
    GPU's ``ic3`` buffer (``peer_ic3_ptrs``: int64 device tensor of ``world`` peer-mapped addresses)."""
    _need_cuda(x, weights, local_ids, peer_ic3_ptrs)
    b, keep = make_banks(local_banks)
    t, h = x.shape
    k = local_ids.shape[1]
    nbytes = lib().b200moe_prefill_workspace_bytes(t, k, h, b.intermediate, b.num_slots)
    ws = _workspace("prefill", nbytes + 64, x.device)
    status = ws[nbytes:nbytes + 16].view(torch.int32)
    check(lib().b200moe_prefill_ep_routes(ptr(x), C.byref(b), ptr(weights), ptr(local_ids), t, first_token, k,
                                          ptr(peer_ic3_ptrs), world, tokens_per_rank, ptr(ws), nbytes, ptr(status),
                                          stream_ptr()), "b200moe_prefill_ep_routes")
    return status
