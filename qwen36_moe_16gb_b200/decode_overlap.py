"""Device-routed offload decode: the per-layer sequence the reference runs when a layer's experts sit behind the
slot cache and the routing only exists on the device.

Mirror of ``OffloadMoELayer.forward_with_shared`` (``freetoken/python/freetoken/layers/moe.py:286-302``) and
``DecodeSharedOverlap.run`` (``freetoken/python/freetoken/decode_overlap.py:44-59``):

    router logits -> top-k -> ensure_experts (device LRU, ids become slot ids)
        -> fork:  side stream: copy_missing (device gather of the planned misses from the pinned host bank)
                  main stream: the shared expert's rows (gate_up, gate logit)
        -> join -> routed expert GEMVs (+ shared down, merge)

Everything has fixed shapes and never reads a device value on the host, so a whole stack of layers is captured in
ONE CUDA graph (the fork and join are event edges inside the capture).  Nothing here knows a layer's experts
before the layer runs: the fill of layer L overlaps only the shared expert of layer L.
"""
from __future__ import annotations

import torch

from . import ops, synth
from .block import MoEBlock
from .kernel import B200Nvfp4MoEKernel, MoEConfig
from .slot_cache import SlotCache

SEG_ROUTER, SEG_SHARED = 1, 6  # segment masks of ops.decode_dense_rows


class DecodeSharedOverlap:
    """Runs ``copy_missing`` on a side stream while ``shared`` runs on the current one; joins before returning.
    Same contract as the reference class of this name: events are created (and used once) at construction so that
    a later stream capture finds them materialised."""

    def __init__(self, device, high_priority: bool = False):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device, priority=-1 if high_priority else 0)
        self.ready, self.done = torch.cuda.Event(), torch.cuda.Event()
        producer = torch.cuda.current_stream(self.device)
        self.ready.record(producer)
        self.stream.wait_event(self.ready)
        self.done.record(self.stream)
        producer.wait_event(self.done)

    def run(self, copy_missing, shared):
        producer = torch.cuda.current_stream(self.device)
        self.ready.record(producer)  # covers ensure_experts and the previous layer's slot consumer
        try:
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(self.ready)
                try:
                    copy_missing()
                finally:
                    self.done.record(self.stream)
            return shared()
        finally:
            producer.wait_event(self.done)  # join before the routed GEMV and before the next layer reuses slots


class DeviceRoutedDecodeStack:
    """A stack of MoE layers decoded through the slot cache with DEVICE tables: per layer the router, the LRU
    ensure, the miss gather and the expert kernels run back to back on the GPU; the host only replays a graph.

    ``records``: per-layer pinned host banks in record layout (``SlotCache.set_record_sources``); pass the list of
    another stack to share the host memory.  ``routing_override``: when a ``[L, M, top_k]`` int32 device tensor is
    given to :meth:`capture`, every layer takes its expert ids from it instead of from its own router (the
    benchmark prescribes the routing); the ids still reach the cache only on the device, layer by layer."""

    def __init__(self, shape: synth.Shape, num_layers: int, cache_size: int, records, dense_blocks=None, device="cuda",
                 seed: int = 0, log_plans: bool = False):
        self.shape, self.L, self.S = shape, num_layers, cache_size
        self.dev = torch.device(device)
        cfg = MoEConfig(shape.num_experts, shape.hidden, shape.intermediate, shape.top_k)
        layout = B200Nvfp4MoEKernel().layout(cfg)
        self.cache = SlotCache(num_layers, shape.num_experts, cache_size, self.dev, layout=layout, host_tables=False)
        self.cache.collect_stats = True
        self.cache.set_record_sources(records)
        self.cache.decode_shared_overlap = DecodeSharedOverlap(self.dev)
        self.handle = ops.make_banks(self.cache.bank_dict())
        if dense_blocks is None:  # every layer its own dense weights
            g = torch.Generator(device=self.dev).manual_seed(seed + 77)
            h, si, e = shape.hidden, shape.shared_intermediate, shape.num_experts
            dense_blocks = [MoEBlock((torch.randn(e, h, generator=g, device=self.dev) * 0.02).bfloat16(),
                                     (torch.randn(2 * si, h, generator=g, device=self.dev) * 0.02).bfloat16(),
                                     (torch.randn(h, si, generator=g, device=self.dev) * 0.02).bfloat16(),
                                     (torch.randn(1, h, generator=g, device=self.dev) * 0.02).bfloat16(), shape.top_k)
                            for _ in range(num_layers)]
        self.blocks = dense_blocks
        self.log_plans = log_plans
        self.graph = None

    # ---- one layer -----------------------------------------------------------------------------------
    def layer(self, l: int, x: torch.Tensor, out: torch.Tensor, ids_override: torch.Tensor | None = None):
        blk, cache = self.blocks[l], self.cache
        ws = blk._decode_ws(x.shape[0], self.handle)
        logits = ops.decode_dense_rows(x, blk.dense, SEG_ROUTER, ws)
        w, ids = ops.fused_topk_softmax(logits, self.shape.top_k, True)
        if ids_override is not None:
            ids.copy_(ids_override)
            w.fill_(1.0 / self.shape.top_k)
        cache.ensure_experts(l, ids)                       # ids are slot ids from here on
        if self.log_plans:
            self.plan_log[l, 0, :ids.numel()].copy_(cache.src_indices[:ids.numel()])
            self.plan_log[l, 1, :ids.numel()].copy_(cache.evict_slots[:ids.numel()])
            self.plan_count[l].copy_(cache.num_indices[0])
        cache.decode_shared_overlap.run(lambda: cache.copy_planned(l),
                                        lambda: ops.decode_dense_rows(x, blk.dense, SEG_SHARED, ws))
        return ops.decode_block_experts(x, self.handle, blk.dense, w, ids, ws, out)

    def step(self, x: torch.Tensor, outs, routing_override: torch.Tensor | None = None):
        for l in range(self.L):
            self.layer(l, x, outs[l % len(outs)], None if routing_override is None else routing_override[l])

    # ---- whole stack in one graph ----------------------------------------------------------------------
    def capture(self, x: torch.Tensor, routing_override: torch.Tensor | None = None, keep_outputs: bool = False):
        m, k = x.shape[0], self.shape.top_k
        self.x = x
        self.outs = [torch.empty_like(x) for _ in range(self.L if keep_outputs else 2)]
        if self.log_plans:
            self.plan_log = torch.zeros((self.L, 2, m * k), dtype=torch.int32, device=self.dev)
            self.plan_count = torch.zeros((self.L,), dtype=torch.int64, device=self.dev)
        # an eager pass first: workspaces, function attributes and lazy CUDA state exist before the capture
        self.step(x, self.outs, routing_override)
        torch.cuda.synchronize()
        self.cache.reset()
        self.cache.reset_stats()
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step(x, self.outs, routing_override)
        return self.graph

    def run(self, routing: torch.Tensor, ids_buf: torch.Tensor, collect_plans: bool = False):
        """Replays the captured stack once per step of ``routing`` ([steps, L, M*top_k] int32, CPU), copying the
        step's ids into ``ids_buf`` (the ``routing_override`` tensor given to :meth:`capture`) before the replay.
        Returns timing and miss statistics; with ``collect_plans`` also the ordered miss plan of every call (one
        synchronisation per step: not for timing)."""
        steps = routing.shape[0]
        pinned = routing.contiguous().pin_memory()
        plans = []
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for s in range(steps):
            ids_buf.copy_(pinned[s].view_as(ids_buf), non_blocking=True)
            self.graph.replay()
            if collect_plans:
                torch.cuda.synchronize()
                log, cnt = self.plan_log.cpu(), self.plan_count.cpu()
                plans += [(log[l, 0, :int(cnt[l])].tolist(), log[l, 1, :int(cnt[l])].tolist()) for l in range(self.L)]
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        stats = self.cache.decode_routing_stats()
        misses = stats["missing"]
        return {"ms": ms, "steps": steps, "tokens_per_s": steps / (ms * 1e-3), "us_per_layer": ms * 1e3 / (steps * self.L),
                "miss_rate": misses / stats["active"] if stats["active"] else 0.0,
                "h2d_bytes": misses * self.cache.expert_bytes,
                "h2d_gbs": misses * self.cache.expert_bytes / (ms * 1e-3) / 1e9, "plans": plans}


__all__ = ["DecodeSharedOverlap", "DeviceRoutedDecodeStack", "SEG_ROUTER", "SEG_SHARED"]
