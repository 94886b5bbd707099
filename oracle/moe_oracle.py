"""CPU oracle for the NVFP4 sparse-MoE block.  TEST INFRASTRUCTURE -- never imported by the shipped path.

Every function restates one piece of the reference (``SUKUNA-AI/qwen36-moe-16gb``; paths are relative
to that project) in plain torch / numpy and cites the file:line it follows.
"""
from __future__ import annotations

import numpy as np
import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
_E2M1 = torch.tensor(E2M1_VALUES, dtype=torch.float32)
BF16 = torch.bfloat16


def _bf16(x: torch.Tensor) -> torch.Tensor:
    """One round-to-nearest-even bf16 rounding, result kept in fp32."""
    return x.to(BF16).float()


# --------------------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------------------
def router_topk(logits: torch.Tensor, top_k: int, renormalize: bool = True,
                num_token_non_padded: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax over all experts, then ``top_k`` rounds of (highest logit, LOWEST id among equals).

    Follows ``freetoken/python/freetoken/kernel/triton/moe_router.py:56-101``: probabilities are
    ``exp(l - max) / sum``; NaN logits rank as -1e30; weights are the selected probabilities divided
    by their sum (by 1 when the sum is not positive); rows at or past ``num_token_non_padded`` get id -1.
    The torch reference ``freetoken/python/freetoken/moe/fused.py:11-30`` agrees whenever no two
    logits tie.  Returns (weights fp32 [T,k], ids int32 [T,k]) in selection order.
    """
    l32 = logits.float()
    t, n = l32.shape
    row_max = l32.max(dim=1, keepdim=True).values
    ex = torch.exp(l32 - row_max)
    probs = ex / ex.sum(dim=1, keepdim=True)
    ranked = torch.where(l32 == l32, l32, torch.full_like(l32, -1e30))
    # stable sort of -logit keeps the lower expert id first among equal logits
    order = torch.sort(-ranked, dim=1, stable=True).indices[:, :top_k]
    w = torch.gather(probs, 1, order)
    if renormalize:
        s = w.sum(dim=1, keepdim=True)
        w = w / torch.where(s > 0, s, torch.ones_like(s))
    ids = order.to(torch.int32)
    if num_token_non_padded is not None:
        ids[int(num_token_non_padded):] = -1
    return w.contiguous(), ids.contiguous()


# --------------------------------------------------------------------------------------------------
# permutation
# --------------------------------------------------------------------------------------------------
def align_sizes(numel: int, block: int, num_experts: int) -> tuple[int, int]:
    """Buffer sizes of ``freetoken/python/freetoken/moe/fused.py:95-101``."""
    if numel < num_experts + 1:
        cap = numel * block
    else:
        cap = numel + (num_experts + 1) * (block - 1)
    return cap, (cap + block - 1) // block


def align_block_size(topk_ids: torch.Tensor, block: int, num_experts: int):
    """Canonical form of ``moe_align_block_size`` (``freetoken/python/freetoken/kernel/triton/moe_align.py:9-20``).

    effective_E = num_experts + 1; ``cumsum[e+1] = cumsum[e] + ceil(count[e]/block)*block``; flat route
    ids ``t*top_k + k`` land in ``[cumsum[e], cumsum[e]+count[e])``; unwritten entries hold ``numel``.
    The reference fills an expert's region in atomic (nondeterministic) order; the canonical form
    used here and by the CUDA kernel is ASCENDING route id inside each expert.  Routes with a
    negative id are dropped.  Returns (sorted_token_ids, expert_ids, num_tokens_post_pad, counts, offsets)
    where ``offsets`` is the unpadded exclusive prefix sum [effective_E + 1].
    """
    ids = topk_ids.reshape(-1).to(torch.int64).numpy()
    numel = ids.size
    eff = num_experts + 1
    cap, nblocks = align_sizes(numel, block, num_experts)
    sorted_ids = np.full(cap, numel, dtype=np.int32)
    expert_ids = np.full(nblocks, -1, dtype=np.int32)
    counts = np.bincount(ids[ids >= 0], minlength=eff).astype(np.int64)
    assert counts.size == eff, "expert id out of range"
    padded = (counts + block - 1) // block * block
    cumsum = np.concatenate([[0], np.cumsum(padded)])
    offsets = np.concatenate([[0], np.cumsum(counts)])
    for e in range(eff):
        routes = np.nonzero(ids == e)[0]
        sorted_ids[cumsum[e]:cumsum[e] + routes.size] = routes
        expert_ids[cumsum[e] // block:cumsum[e + 1] // block] = e
    return (torch.from_numpy(sorted_ids), torch.from_numpy(expert_ids),
            torch.tensor([cumsum[-1]], dtype=torch.int32),
            torch.from_numpy(counts.astype(np.int32)), torch.from_numpy(offsets.astype(np.int32)))


def sorted_routes(topk_ids: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Unpadded canonical permutation: route ids stably sorted by expert, and offsets [E+1]."""
    ids = topk_ids.reshape(-1).to(torch.int64)
    valid = torch.nonzero(ids >= 0).reshape(-1)
    order = valid[torch.sort(ids[valid], stable=True).indices]
    counts = torch.bincount(ids[valid], minlength=num_experts)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)])
    return order.to(torch.int32), offsets.to(torch.int32)


# --------------------------------------------------------------------------------------------------
# slot cache
# --------------------------------------------------------------------------------------------------
class SlotCacheOracle:
    """Slot tables + LRU policy of the expert offload cache.

    State follows ``freetoken/python/freetoken/moe/offload_cache.py:205-227,263-268``; ``ensure`` restates
    the numpy mirror of ``flashlib.kernels.slot_cache.lru_ensure`` kept in the reference tree
    (``next-update/transport/scripts/d3a_replay.py:21-51``): the clock advances once per call; hits
    get ``usage = step``; DISTINCT misses in ascending id take victims in ascending (usage, slot)
    among the slots this call has not touched.  Plan outputs and the in-place id -> slot rewrite
    follow ``freetoken/python/freetoken/moe/offload_kernels.py:19-40``.  Parity unpinned: ids < 0 (kept
    as they are), more misses than victims (the surplus misses stay unmapped and rewrite to -1).
    """

    def __init__(self, num_layers: int, num_experts: int, cache_size: int):
        self.L, self.E, self.S = num_layers, num_experts, cache_size
        self.reset()

    def reset(self) -> None:
        """``_reset_cache_kernel`` (``offload_kernels.py:273-293``)."""
        self.slot_for_id = np.full(self.L * self.E, -1, dtype=np.int32)
        self.id_of_slot = np.full(self.S, -1, dtype=np.int32)
        self.usage = np.zeros(self.S, dtype=np.int64)
        self.step = 0
        self.stats = np.zeros((self.L, 3), dtype=np.int64)  # active, missing, calls
        self.src_indices = np.zeros(0, dtype=np.int32)
        self.evict_slots = np.zeros(0, dtype=np.int32)

    def ensure(self, layer: int, ids: np.ndarray) -> np.ndarray:
        """Returns the ids rewritten to slot ids (same shape); leaves the miss plan in
        ``src_indices`` / ``evict_slots`` (layer-local expert id, victim slot), in miss order."""
        ids = np.asarray(ids)
        base = layer * self.E
        self.step += 1
        q = np.unique(ids[ids >= 0].astype(np.int64)) + base
        slots = self.slot_for_id[q]
        self.usage[slots[slots >= 0]] = self.step
        miss = q[slots < 0]
        src, dst = [], []
        if miss.size:
            order = np.argsort(self.usage, kind="stable")
            order = order[self.usage[order] != self.step][:miss.size]
            for e, v in zip(miss, order):
                old = self.id_of_slot[v]
                if old >= 0:
                    self.slot_for_id[old] = -1
                self.id_of_slot[v] = e
                self.slot_for_id[e] = v
                self.usage[v] = self.step
                src.append(e - base)
                dst.append(v)
        self.src_indices = np.asarray(src, dtype=np.int32)
        self.evict_slots = np.asarray(dst, dtype=np.int32)
        self.stats[layer] += (q.size, miss.size, 1)
        out = ids.astype(np.int32).copy()
        pos = ids >= 0
        out[pos] = self.slot_for_id[ids[pos].astype(np.int64) + base]
        return out

    def materialize_layer(self, layer: int) -> None:
        """Whole layer into slots [0, E), position == expert id (``offload_kernels.py:296-332``)."""
        base = layer * self.E
        same = (self.id_of_slot >= base) & (self.id_of_slot < base + self.E)
        head = np.arange(self.S) < self.E
        old = self.id_of_slot.copy()
        self.id_of_slot[same] = -1
        self.usage[same] = 0
        evicted = head & (old >= 0) & ~same
        self.slot_for_id[old[evicted]] = -1
        self.step += 1
        e = np.arange(self.E)
        self.id_of_slot[:self.E] = base + e
        self.slot_for_id[base:base + self.E] = e
        self.usage[:self.E] = self.step
        self.src_indices = e.astype(np.int32)
        self.evict_slots = e.astype(np.int32)

    def tables(self) -> dict[str, np.ndarray]:
        return {"slot_for_id": self.slot_for_id.copy(), "id_of_slot": self.id_of_slot.copy(),
                "usage": self.usage.copy(), "step": np.int64(self.step)}


# --------------------------------------------------------------------------------------------------
# NVFP4
# --------------------------------------------------------------------------------------------------
def dequant_nvfp4(packed: torch.Tensor, scale: torch.Tensor, row_global: torch.Tensor | None = None) -> torch.Tensor:
    """``[N, K/2]`` u8 + ``[N, K/16]`` e4m3 (+ ``[N]`` fp32) -> ``[N, K]`` fp32, low nibble = even k.

    ``_dequant_ref`` of ``freetoken/tests/moe/test_nvfp4_backends.py:40-46``.  Without ``row_global``
    the result is ``E2M1 * scale`` only (exact in bf16), the operand the grouped GEMM multiplies."""
    n, k2 = packed.shape[-2:]
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(*packed.shape[:-1], 2 * k2).long()
    w = _E2M1[codes] * scale.float().repeat_interleave(16, dim=-1)
    if row_global is not None:
        w = w * row_global.float().unsqueeze(-1)
    return w


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """fp32 ``gate / (1 + exp(-gate)) * up`` (``freetoken/python/freetoken/kernel/triton/activation.py:98-100``;
    the reference evaluates the exponential with ``ex2.approx``, an error far below one bf16 ulp)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def moe_experts_fp32(x, banks, topk_weights, topk_ids) -> torch.Tensor:
    """The reference test-suite oracle ``_ref_moe`` (``freetoken/tests/moe/test_nvfp4_backends.py:92-115``):
    fp32 dequant, fp32 matmul, ``silu(h[:I]) * h[I:]``, ``out += w * (down @ act)``; fp32 result.
    Vectorised per expert instead of per (token, route); ``topk_ids`` index rows of ``banks``."""
    t_n, h = x.shape
    out = torch.zeros(t_n, h, dtype=torch.float32)
    xf = x.float()
    ids = topk_ids.long()
    inter = banks["down"].shape[-1] * 2
    for e in torch.unique(ids[ids >= 0]).tolist():
        tok, kk = torch.nonzero(ids == e, as_tuple=True)
        gu = dequant_nvfp4(banks["gate_up"][e], banks["gate_up_scale"][e], banks["gate_up_global"][e])
        dn = dequant_nvfp4(banks["down"][e], banks["down_scale"][e], banks["down_global"][e])
        hh = xf[tok] @ gu.t()
        act = torch.nn.functional.silu(hh[:, :inter]) * hh[:, inter:]
        out.index_add_(0, tok, (act @ dn.t()) * topk_weights[tok, kk].float().unsqueeze(1))
    return out


def moe_experts_bf16(x, banks, topk_weights, topk_ids, return_intermediates: bool = False):
    """Production-faithful routed experts: the reference kernels' rounding points.

      ic1 = bf16(acc * global)                      ``kernel/triton/nvfp4_fused_moe.py:214-227,314-325``
      ic2 = bf16(silu(f32 gate) * f32 up)            ``kernel/triton/activation.py:98-119``
      ic3 = bf16((acc * global) * router_weight)     ``nvfp4_fused_moe.py:217-221,317-321``
      out = bf16(sum_k f32(ic3[t,k]) in k order)     ``kernel/triton/fused_moe.py:142-153``

    Accumulation is fp32 over exactly dequantised ``E2M1*scale`` operands (their order is not part
    of the contract).  Negative ids contribute nothing.  Returns bf16 ``[T, H]``."""
    t_n, h = x.shape
    k_n = topk_ids.shape[1]
    inter = banks["down"].shape[-1] * 2
    xf = x.float()
    ids = topk_ids.long()
    ic2 = torch.zeros(t_n, k_n, inter, dtype=torch.float32)
    ic3 = torch.zeros(t_n, k_n, h, dtype=torch.float32)
    for e in torch.unique(ids[ids >= 0]).tolist():
        tok, kk = torch.nonzero(ids == e, as_tuple=True)
        gu = dequant_nvfp4(banks["gate_up"][e], banks["gate_up_scale"][e])
        dn = dequant_nvfp4(banks["down"][e], banks["down_scale"][e])
        ic1 = _bf16((xf[tok] @ gu.t()) * banks["gate_up_global"][e].float())
        a2 = _bf16(silu_mul(ic1[:, :inter], ic1[:, inter:]))
        ic2[tok, kk] = a2
        acc = (a2 @ dn.t()) * banks["down_global"][e].float()
        ic3[tok, kk] = _bf16(acc * topk_weights[tok, kk].float().unsqueeze(1))
    out = torch.zeros(t_n, h, dtype=torch.float32)
    for k in range(k_n):
        out = out + ic3[:, k]
    out = out.to(BF16)
    if return_intermediates:
        return out, ic2.to(BF16), ic3.to(BF16)
    return out


def _linear_bf16(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """bf16 linear: fp32 accumulate, one bf16 rounding (``layers/quantization/linear/unquantized.py:18-24``)."""
    return (x.float() @ w.float().t()).to(BF16)


def shared_expert(x, shared_gate_up, shared_down, shared_gate):
    """``_SharedExpert.forward`` and the gate projection (``models/qwen3_5_moe/moe.py:20-36,99-106``).
    Returns (shared bf16 [T,H], gate logit bf16 [T,1]); every op rounds to bf16."""
    hs = _linear_bf16(x, shared_gate_up).float()
    si = shared_gate_up.shape[0] // 2
    act = silu_mul(hs[:, :si], hs[:, si:]).to(BF16)
    return _linear_bf16(act, shared_down), _linear_bf16(x, shared_gate)


def shared_epilogue(routed, shared, gate):
    """``routed + shared * sigmoid(gate)`` with torch's three bf16 roundings
    (``freetoken/python/freetoken/moe/shared_epilogue.py:7-9``)."""
    sig = _bf16(1.0 / (1.0 + torch.exp(-gate.float())))
    prod = _bf16(shared.float() * sig)
    return (routed.float() + prod).to(BF16)


def moe_block(layer: dict[str, torch.Tensor], top_k: int, logits: torch.Tensor | None = None,
              faithful: bool = True) -> dict[str, torch.Tensor]:
    """The whole block, ``Qwen3_5MoE.forward`` (``models/qwen3_5_moe/moe.py:77-97``): router logits,
    shared expert first, routed experts, merge.  ``logits`` overrides the router GEMV output."""
    x = layer["x"]
    if logits is None:
        logits = x.float() @ layer["router_w"].float().t()
        if "logit_bias" in layer:  # synthetic popularity skew, added before the single bf16 rounding
            logits = logits + layer["logit_bias"]
        logits = logits.to(BF16)
    w, ids = router_topk(logits, top_k, True)
    shared, gate = shared_expert(x, layer["shared_gate_up"], layer["shared_down"], layer["shared_gate"])
    if faithful:
        routed = moe_experts_bf16(x, layer, w, ids)
    else:
        routed = moe_experts_fp32(x, layer, w, ids).to(BF16)
    out = shared_epilogue(routed, shared, gate)
    return {"logits": logits, "topk_weights": w, "topk_ids": ids, "routed": routed,
            "shared": shared, "shared_gate_logit": gate, "out": out}


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                      plus_one: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """``_fused_add_rmsnorm_kernel`` (``freetoken/python/freetoken/kernel/triton/norm.py:78-111``): ``z = f32(x) +
    f32(residual)``; new residual ``bf16(z)``; output ``bf16(z * rsqrt(mean(z*z) + eps) * (w [+ 1]))`` -- the norm
    uses the unrounded sum.  Returns (normed, residual), both bf16."""
    z = x.float() + residual.float()
    w = weight.float() + (1.0 if plus_one else 0.0)
    inv = torch.rsqrt((z * z).mean(dim=-1, keepdim=True) + eps)
    return (z * inv * w).to(BF16), z.to(BF16)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, plus_one: bool = False) -> torch.Tensor:
    """``_rmsnorm_kernel`` (``freetoken/python/freetoken/kernel/triton/norm.py:44-75``)."""
    z = x.float()
    w = weight.float() + (1.0 if plus_one else 0.0)
    return (z * torch.rsqrt((z * z).mean(dim=-1, keepdim=True) + eps) * w).to(BF16)


def pregate_logits(residual: torch.Tensor, norm_w: torch.Tensor, gate_w: torch.Tensor, eps: float) -> torch.Tensor:
    """``_pregate_logits_kernel`` (``freetoken/python/freetoken/moe/pregate.py:77-89``): fp32 logits of the next
    layer's router on ``bf16(rmsnorm(residual) * w)``."""
    x = residual.float().reshape(-1)
    inv = 1.0 / torch.sqrt((x * x).sum() / x.numel() + eps)
    y = (x * inv * norm_w.float()).to(BF16).float()
    return (gate_w.float() * y.unsqueeze(0)).sum(dim=1)


def pregate_select(logits: torch.Tensor, slot_row, cap: int, top_k: int, width: int) -> list[int]:
    """``_pregate_select_kernel`` (``pregate.py:92-117``): the first ``cap`` of the ``top_k`` predictions (score order,
    lowest id among equals, NaN ranks last) whose slot is unmapped, padded to ``width`` with the first of them, or
    with the top-1 prediction when none misses."""
    v = logits.float().clone()
    v[v != v] = float("-inf")
    e = v.numel()
    out, first, top1 = [], 0, 0
    for k in range(top_k):
        best = v.max()
        win = min(int(torch.nonzero(v == best).reshape(-1)[0]), e - 1)
        if k == 0:
            top1 = win
        if int(slot_row[win]) < 0 and len(out) < cap:
            if not out:
                first = win
            out.append(win)
        v[win] = float("-inf")
    pad = first if out else top1
    return out + [pad] * (width - len(out))


def error_metrics(got: torch.Tensor, want: torch.Tensor) -> tuple[float, float]:
    """(max-abs, rel-L2) of ``got`` against ``want`` in fp64."""
    g, w = got.double(), want.double()
    return float((g - w).abs().max()), float((g - w).norm() / w.norm().clamp_min(1e-300))


__all__ = ["E2M1_VALUES", "router_topk", "align_sizes", "align_block_size", "sorted_routes", "SlotCacheOracle",
           "dequant_nvfp4", "silu_mul", "moe_experts_fp32", "moe_experts_bf16", "shared_expert",
           "shared_epilogue", "moe_block", "fused_add_rmsnorm", "rmsnorm", "pregate_logits", "pregate_select", "error_metrics"]
