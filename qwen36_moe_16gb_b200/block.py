"""The MoE block driver: mirror of ``Qwen3_5MoE.forward`` (``freetoken/python/freetoken/models/qwen3_5_moe/moe.py:77-106``).

    out = routed(x) + sigmoid(shared_expert_gate(x)) * shared_expert(x)

Decode (<= 8 tokens): three launches chained by programmatic dependent launch -- dense rows (router logits +
shared gate_up + gate logit), expert GEMM1 with the router top-k in its prologue + SwiGLU (+ shared activation),
expert GEMM2 + route sum + shared down + merge.  With the slot cache in between (offload), routing is a separate
launch so that the LRU can rewrite expert ids to slot ids before the expert kernels.
Prefill: router logits and the shared expert's dense bf16 GEMMs (gate_up with its SwiGLU in the epilogue, down) run
on this package's tcgen05 dense GEMM, like routing, permutation, the grouped expert GEMMs and the merge: no library
GEMM is on the path.
"""
from __future__ import annotations

import torch

from . import ops
from .kernel import DECODE_MAX_TOKENS


class MoEBlock:
    def __init__(self, router_w, shared_gate_up, shared_down, shared_gate, top_k: int, logit_bias=None):
        self.router_w, self.shared_gate_up = router_w, shared_gate_up
        self.shared_down, self.shared_gate = shared_down, shared_gate
        self.top_k = top_k
        self.logit_bias = logit_bias  # synthetic popularity skew (fp32 [E]); None in a real model
        self._bias_f32 = None if logit_bias is None else logit_bias.to(torch.bfloat16).float().contiguous()
        self.dense = ops.make_dense(router_w, shared_gate_up, shared_down, shared_gate)
        self._ws = {}
        self._overlap = {}

    def _decode_ws(self, m, banks):
        key = (m, banks[0].intermediate, torch.cuda.current_stream().cuda_stream)
        if key not in self._ws:
            self._ws[key] = ops.decode_block_workspace(m, self.top_k, banks[0].hidden, banks[0].intermediate,
                                                       self.dense[0].shared_intermediate, self.router_w.device)
        return self._ws[key]

    # ---- pieces (the offload path runs ensure_experts between them) ---------------------------------
    def decode_route(self, x, banks):
        return ops.decode_block_route(x, self.dense, self.top_k, self._decode_ws(x.shape[0], banks))

    def decode_experts(self, x, banks, w, ids, out=None):
        return ops.decode_block_experts(x, banks, self.dense, w, ids, self._decode_ws(x.shape[0], banks), out)

    def decode_fused(self, x, banks, out=None):
        """All experts resident: dense rows -> GEMM1 (routes in its prologue) -> GEMM2 + merge."""
        return ops.decode_block(x, banks, self.dense, self.top_k, self._decode_ws(x.shape[0], banks), out)

    def router_logits(self, x):
        # the synthetic bias is added in the GEMM epilogue (fp32) before the single bf16 rounding
        return ops.dense_linear(x, self.router_w, self._bias_f32)

    def shared_parts(self, x):
        act = ops.dense_linear(x, self.shared_gate_up, swiglu=True)
        return ops.dense_linear(act, self.shared_down), ops.row_dot(x, self.shared_gate)

    # ---- whole block ---------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, bank_tensors: dict[str, torch.Tensor], is_prefill: bool | None = None):
        """``bank_tensors``: whole-layer ``[E, ...]`` banks (position == expert id)."""
        t = x.shape[0]
        banks = ops.make_banks(bank_tensors)
        decode = (not is_prefill) if is_prefill is not None else t <= DECODE_MAX_TOKENS
        if decode and t <= DECODE_MAX_TOKENS and self.logit_bias is None and banks[0].hidden % 512 == 0 \
                and banks[0].intermediate % 512 == 0:
            return self.decode_fused(x, banks)[0]
        return self.prefill(x, bank_tensors)

    def prefill(self, x: torch.Tensor, bank_tensors: dict[str, torch.Tensor], out=None, overlap: bool = False,
                check_status: bool = False):
        """Prefill form of the block.  The shared expert does not depend on the routing, so with ``overlap`` its GEMMs
        run on a side stream next to the router's top-k, the permutation and the token gather, and join before the
        merge -- the prefill counterpart of the decode path's shared-expert overlap
        (``freetoken/python/freetoken/decode_overlap.py:44-59``).  The side stream's work of one call is ordered after
        the router GEMM of that call and therefore after the merge of the previous one, so its buffers can be reused
        call after call.  Off by default: at T = 8192 the two forms take the same time (0.757 against 0.755 ms), because
        a resident dense-GEMM CTA (197 KB of shared memory, 54 K registers) leaves the gather kernel too little of
        the SM to keep HBM busy."""
        logits = self.router_logits(x)
        if not overlap:
            shared, gate = self.shared_parts(x)
            w, ids = ops.fused_topk(x, logits, self.top_k, True)
            return ops.prefill_experts(x, bank_tensors, w, ids, shared=shared, shared_gate_logit=gate, out=out,
                                       check_status=check_status)
        main = torch.cuda.current_stream(x.device)
        side, fork, join = self._overlap_state(x.device)
        fork.record(main)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            shared, gate = self.shared_parts(x)
            join.record(side)
        w, ids = ops.fused_topk(x, logits, self.top_k, True)
        out = ops.prefill_experts(x, bank_tensors, w, ids, out=out, stages=ops.STAGE_PLAN | ops.STAGE_GEMM1 | ops.STAGE_GEMM2)
        main.wait_event(join)
        return ops.prefill_experts(x, bank_tensors, w, ids, shared=shared, shared_gate_logit=gate, out=out,
                                   stages=ops.STAGE_COMBINE, check_status=check_status)

    def _overlap_state(self, device):
        key = torch.device(device).index
        if key not in self._overlap:
            self._overlap[key] = (torch.cuda.Stream(device), torch.cuda.Event(), torch.cuda.Event())
        return self._overlap[key]


class PrefillGraphs:
    """The prefill block as CUDA graphs, one per (input buffer, output buffer) pair: the first call with a pair runs
    the block once eagerly (workspaces and lazy state exist afterwards), captures it, and every later call replays the
    capture -- 14 kernel launches become one graph launch (about 27 us less per step on a B200, whatever T).  The
    buffers' addresses and shapes are baked in: refill ``x`` in place between calls."""

    def __init__(self, block: "MoEBlock", bank_tensors: dict[str, torch.Tensor]):
        self.block, self.banks = block, bank_tensors
        self.graphs: dict[tuple[int, int, int], torch.cuda.CUDAGraph] = {}

    def __call__(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        key = (x.data_ptr(), out.data_ptr(), x.shape[0])
        graph = self.graphs.get(key)
        if graph is None:
            self.block.prefill(x, self.banks, out=out, check_status=True)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.block.prefill(x, self.banks, out=out)
            self.graphs[key] = graph
        graph.replay()
        return out


class DecoderLayerMoE:
    """The part of a decoder layer around the block: the mixer's output joins the residual stream and is normalised
    in one kernel, then the MoE block runs (``Qwen3_5DecoderLayer.forward``,
    ``freetoken/python/freetoken/models/qwen3_5_moe/model.py:63-77``: ``post_attention_layernorm.forward_add_residual``
    followed by ``mlp.forward``).  Returns ``(hidden, residual)`` like the reference layer: the block's output is added
    to the residual by the NEXT layer's fused norm."""

    def __init__(self, block: MoEBlock, post_attention_norm_weight: torch.Tensor, eps: float = 1e-6):
        self.block, self.weight, self.eps = block, post_attention_norm_weight, eps

    def forward(self, mixer_out: torch.Tensor, residual: torch.Tensor, bank_tensors: dict[str, torch.Tensor],
                is_prefill: bool | None = None):
        ops.fused_add_rmsnorm(mixer_out, residual, self.weight, self.eps)   # in place: both tensors are rewritten
        return self.block.forward(mixer_out, bank_tensors, is_prefill), residual


class HostPipeline:
    """Feeds a device step from host memory and returns its result to host memory, step after step, with the
    copies off the compute stream: the host->device copy of step i+1 and the device->host copy of step i-1 run
    while step i computes (two device buffers each way, three streams, events for the hand-overs).

    ``run(x_dev, out_dev)`` runs one step on the current stream and returns the tensor holding its result
    (``out_dev`` or one of its own).  ``x_host`` / ``out_host`` must be pinned."""

    def __init__(self, run, x_host: torch.Tensor, out_host: torch.Tensor, device):
        self.run, self.x_host, self.out_host = run, x_host, out_host
        self.x_dev = [torch.empty(x_host.shape, dtype=x_host.dtype, device=device) for _ in range(2)]
        self.out_dev = [torch.empty(out_host.shape, dtype=out_host.dtype, device=device) for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]    # input buffer b holds the step's tokens
        self.ev_done = [torch.cuda.Event() for _ in range(2)]  # the step that used buffers b has finished computing
        self.ev_out = [torch.cuda.Event() for _ in range(2)]   # output buffer b has been copied to the host
        self.i = 0

    def submit(self) -> None:
        """Enqueue one step; returns at once (the host only issues work)."""
        b = self.i & 1
        main = torch.cuda.current_stream(self.x_dev[0].device)
        if self.i >= 2:
            self.s_in.wait_event(self.ev_done[b])   # the step two back has read input buffer b
        with torch.cuda.stream(self.s_in):
            self.x_dev[b].copy_(self.x_host, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        main.wait_event(self.ev_in[b])
        if self.i >= 2:
            main.wait_event(self.ev_out[b])         # output buffer b has left for the host
        out = self.run(self.x_dev[b], self.out_dev[b])
        self.ev_done[b].record(main)
        self.s_out.wait_event(self.ev_done[b])
        with torch.cuda.stream(self.s_out):
            out.record_stream(self.s_out)
            self.out_host.copy_(out, non_blocking=True)
            self.ev_out[b].record(self.s_out)
        self.i += 1

    def join(self) -> None:
        """The current stream waits for every copy issued so far."""
        main = torch.cuda.current_stream(self.x_dev[0].device)
        main.wait_stream(self.s_in)
        main.wait_stream(self.s_out)


__all__ = ["MoEBlock", "PrefillGraphs", "DecoderLayerMoE", "HostPipeline"]
