"""Decode over a stack of MoE layers whose experts live in pinned host banks behind the slot cache.

Per (step, layer): the LRU policy runs on host tables (the routing of this workload is known on the host),
every miss becomes six ``cudaMemcpyAsync`` (one per bank) on a COPY stream, an event hands the filled slots to
the compute stream, and the decode kernels run with slot ids.  The host never waits for the GPU inside the
loop, so the copy stream runs ahead of the compute stream and layer L+1's fills overlap layer L's kernels.
A fill may only overwrite a slot that no pending kernel still reads: fills of call c wait for the compute of
call c - LOOKAHEAD, and the LRU cannot choose a slot touched in the last LOOKAHEAD calls as long as the cache
has more than top_k * (LOOKAHEAD + 1) slots (checked).
"""
from __future__ import annotations

import torch

from . import ops, synth
from .block import MoEBlock
from .host_banks import HostBank
from .kernel import B200Nvfp4MoEKernel, MoEConfig
from .slot_cache import SlotCache

LOOKAHEAD = 16  # upper bound; a small cache gets a shorter look-ahead


class OffloadDecodeStack:
    def __init__(self, shape: synth.Shape, num_layers: int, cache_size: int, device="cuda", seed: int = 0,
                 lookahead: int = LOOKAHEAD, records=None, per_layer_dense: bool = False):
        """``lookahead``: how many layers the copy stream may run ahead of the compute stream (1 = a layer's fills
        overlap the previous layer only).  ``records``: reuse another stack's pinned host banks.
        ``per_layer_dense``: every layer gets its own router / shared-expert weights (otherwise one set serves all)."""
        self.shape, self.L, self.S = shape, num_layers, cache_size
        self.dev = torch.device(device)
        self.lookahead = min(lookahead, (cache_size - 1) // shape.top_k - 1)  # cache_size > top_k * (lookahead + 1)
        if self.lookahead < 1:
            raise ValueError("slot cache too small for the copy look-ahead")
        cfg = MoEConfig(shape.num_experts, shape.hidden, shape.intermediate, shape.top_k)
        layout = B200Nvfp4MoEKernel().layout(cfg)
        # pinned host banks, one [E, ...] tensor per (role, layer); filled from a device generator (fast)
        # One contiguous record per expert (all six roles back to back): a miss is ONE host-to-device copy.
        g = torch.Generator(device=self.dev).manual_seed(seed)
        rb = SlotCache.record_bytes(layout)
        build = records is None
        records = [] if build else records
        self.host_banks = []
        stage = torch.empty((shape.num_experts, rb), dtype=torch.uint8, device=self.dev)
        for _ in range(num_layers if build else 0):
            dev_banks = synth.make_banks(g, shape, device=self.dev)
            views = SlotCache.record_views(stage, layout)
            for r in synth.ROLES:
                views[r].copy_(dev_banks[r])
            bank = HostBank((shape.num_experts, rb), torch.uint8)   # lazy pages; filled, then pinned
            bank.tensor.copy_(stage)
            bank.pin()
            self.host_banks.append(bank)
            records.append(bank.tensor)
            del dev_banks
        del stage
        self.cache = SlotCache(num_layers, shape.num_experts, cache_size, self.dev, layout=layout, host_tables=True)
        self.cache.collect_stats = True
        self.cache.set_record_sources(records)
        self.records = records
        self.sources = self.cache.bank_sources
        dense = synth.make_layer(seed, 1, shape, with_banks=False)
        d = {k: v.to(self.dev) for k, v in dense.items()}
        self.x = d["x"]
        self.block = MoEBlock(d["router_w"], d["shared_gate_up"], d["shared_down"], d["shared_gate"], shape.top_k)
        self.blocks, self._dense_array, self._dense_stride = [self.block], None, 0
        if per_layer_dense:
            import ctypes as C

            from ._lib import Dense

            gd = torch.Generator(device=self.dev).manual_seed(seed + 77)
            h, si, e = shape.hidden, shape.shared_intermediate, shape.num_experts
            self.blocks = [MoEBlock((torch.randn(e, h, generator=gd, device=self.dev) * 0.02).bfloat16(),
                                    (torch.randn(2 * si, h, generator=gd, device=self.dev) * 0.02).bfloat16(),
                                    (torch.randn(h, si, generator=gd, device=self.dev) * 0.02).bfloat16(),
                                    (torch.randn(1, h, generator=gd, device=self.dev) * 0.02).bfloat16(), shape.top_k)
                           for _ in range(num_layers)]
            self.block = self.blocks[0]
            self._dense_array = (Dense * num_layers)(*[b.dense[0] for b in self.blocks])
            self._dense_stride = C.sizeof(Dense)
        self.handle = ops.make_banks(self.cache.bank_dict())
        self.copy_stream = torch.cuda.Stream(self.dev)
        self.miss_log: list[tuple[list[int], list[int]]] = []

    def _native(self):
        """The C-side step runner (events + host plan + launches in one call per decode step)."""
        import ctypes as C

        from ._lib import check, lib

        if getattr(self, "_handle", None) is None:
            cache = self.cache
            n = len(cache.banks)
            src = (C.c_void_p * (n * self.L))(*[per_layer[l].data_ptr() for l in range(self.L) for per_layer, _ in cache.banks])
            err = C.c_int(0)
            t = cache._tables(None)
            t.stats = cache.lru_stats.data_ptr()  # [L, 3]: the runner offsets it per layer
            self._tables_keep = t
            self._handle = lib().b200moe_offload_create(C.byref(t), n, cache._dst_host, src, cache._row_bytes_host, self.lookahead,
                                                        C.byref(err))
            check(err.value, "b200moe_offload_create")
        return self._handle

    def close(self) -> None:
        from ._lib import lib

        if getattr(self, "_handle", None) is not None:
            lib().b200moe_offload_destroy(self._handle)
            self._handle = None

    def run(self, routing: torch.Tensor, weights: torch.Tensor | None = None, keep_outputs: bool = False,
            log_misses: bool = True):
        """routing: int32 [steps, L, top_k] expert ids (CPU).  One native call per decode step."""
        import ctypes as C

        from ._lib import check, lib, ptr

        steps, L, k = routing.shape
        assert L == self.L and k == self.shape.top_k
        routing = routing.contiguous()
        handle = self._native()
        dev = self.dev
        slots_host = torch.empty((steps, L, k), dtype=torch.int32).pin_memory()
        slots_dev = torch.empty((steps, L, k), dtype=torch.int32, device=dev)
        w_dev = (torch.full((1, k), 1.0 / k, device=dev) if weights is None else weights.to(dev))
        out = torch.empty((L if keep_outputs else 1, 1, self.shape.hidden), dtype=torch.bfloat16, device=dev)
        miss_src = torch.zeros((steps, L, k), dtype=torch.int32)
        miss_dst = torch.zeros((steps, L, k), dtype=torch.int32)
        miss_cnt = torch.zeros((steps, L), dtype=torch.int32)
        banks = self.handle[0]
        dense = self._dense_array if self._dense_array is not None else self.block.dense[0]
        ws = self.block._decode_ws(1, self.handle)
        h2d = C.c_int64(0)
        compute = torch.cuda.current_stream(dev)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record(compute)
        self.copy_stream.wait_stream(compute)
        step_fn = lib().b200moe_offload_decode_step
        out_stride = out.stride(0) * 2 if keep_outputs else 0
        for s in range(steps):
            rc = step_fn(handle, ptr(routing[s]), 1, k, ptr(slots_host[s]), ptr(slots_dev[s]), ptr(w_dev), 0, ptr(self.x),
                         C.byref(banks), dense if self._dense_array is not None else C.byref(dense), self._dense_stride,
                         ptr(out), out_stride, ptr(ws), ws.numel(),
                         ptr(miss_src[s]) if log_misses else None, ptr(miss_dst[s]) if log_misses else None,
                         ptr(miss_cnt[s]), C.byref(h2d), self.copy_stream.cuda_stream, compute.cuda_stream)
            if rc:
                check(rc, "b200moe_offload_decode_step")
        stop.record(compute)
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        self.cache.h2d_bytes += h2d.value
        self.miss_log = [(miss_src[s, l, :int(miss_cnt[s, l])].tolist(), miss_dst[s, l, :int(miss_cnt[s, l])].tolist())
                         for s in range(steps) for l in range(L)] if log_misses else []
        calls = steps * L
        stats = self.cache.decode_miss_stats()
        return {"ms": ms, "steps": steps, "tokens_per_s": steps / (ms * 1e-3), "us_per_layer": ms * 1e3 / calls,
                "miss_rate": stats["miss_rate"], "misses_per_token": stats["missing_per_layer"] * L,
                "h2d_bytes": h2d.value, "h2d_gbs": h2d.value / (ms * 1e-3) / 1e9, "out": out}

    def run_python(self, routing: torch.Tensor, weights: torch.Tensor | None = None, keep_outputs: bool = False):
        """The same loop driven from Python, one layer at a time (reference form of `run`; slower host side)."""
        steps, L, k = routing.shape
        assert L == self.L and k == self.shape.top_k
        cache, blk = self.cache, self.block
        calls = steps * L
        slots_host = torch.empty((calls, 1, k), dtype=torch.int32).pin_memory()
        slots_dev = torch.empty((calls, 1, k), dtype=torch.int32, device=self.dev)
        w_dev = (torch.full((1, k), 1.0 / k, device=self.dev) if weights is None else weights.to(self.dev))
        out = torch.empty((L if keep_outputs else 1, 1, self.shape.hidden), dtype=torch.bfloat16, device=self.dev)
        compute = torch.cuda.current_stream(self.dev)
        la = self.lookahead
        done = [torch.cuda.Event() for _ in range(la + 1)]
        filled = [torch.cuda.Event() for _ in range(la + 1)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.miss_log = []
        torch.cuda.synchronize()
        start.record(compute)
        self.copy_stream.wait_stream(compute)
        c = 0
        for s in range(steps):
            for layer in range(L):
                ids = slots_host[c, 0]
                ids.copy_(routing[s, layer])
                n = cache.ensure_experts_host(layer, ids)                      # ids now hold slot ids
                self.miss_log.append((cache.src_indices[:n].tolist(), cache.evict_slots[:n].tolist()))
                e = c % (la + 1)
                if c >= la:
                    self.copy_stream.wait_event(done[(c - la) % (la + 1)])
                cache.fill_planned(layer, self.copy_stream)
                filled[e].record(self.copy_stream)
                slots_dev[c].copy_(slots_host[c], non_blocking=True)
                compute.wait_event(filled[e])
                blk.decode_route(self.x, self.handle)                          # router logits + shared gate_up (dense part)
                blk.decode_experts(self.x, self.handle, w_dev, slots_dev[c], out[layer if keep_outputs else 0])
                done[e].record(compute)
                c += 1
        stop.record(compute)
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        stats = cache.decode_miss_stats()
        return {"ms": ms, "steps": steps, "tokens_per_s": steps / (ms * 1e-3), "us_per_layer": ms * 1e3 / calls,
                "miss_rate": stats["miss_rate"], "misses_per_token": stats["missing_per_layer"] * L,
                "h2d_bytes": stats["h2d_bytes"], "h2d_gbs": stats["h2d_bytes"] / (ms * 1e-3) / 1e9, "out": out}


__all__ = ["OffloadDecodeStack", "LOOKAHEAD"]
