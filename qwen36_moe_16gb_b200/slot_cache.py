"""Expert-slot offload cache: host-side mirror of the ``OffloadMoeCache`` interface that the reference's
``OffloadMoELayer`` and engine call (``freetoken/python/freetoken/moe/offload_cache.py:139-1533``).

All routed experts of all layers live in pinned host banks; the GPU holds ``cache_size`` slots per bank.
Two ways to serve misses, with identical slot tables:

* device-planned (``ensure_experts`` + ``copy_missing``): the LRU runs in one small kernel on device tables,
  the plan stays on the device (``num_indices`` is a device scalar) and a gather kernel pulls the rows from
  the mapped pinned banks -- fixed-shape launches, no host sync, CUDA-graph capturable;
* host-planned (``ensure_experts_host`` + ``fill_planned``): the same policy runs on host tables and every
  (miss, bank) row becomes one ``cudaMemcpyAsync`` on a copy stream, so layer L+1's fills overlap layer L's
  compute whenever the routing is known ahead of the compute.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ops
from ._lib import SlotTables, check, lib, ptr, stream_ptr
from .kernel import BankSpec

N_STATS = 3  # (active, missing, calls) per layer


class SlotCache:
    def __init__(self, num_layers: int, num_experts: int, cache_size: int, device, cache_policy: str = "lru",
                 prefill_overlap: bool = False, prefill_hit_d2d: bool = False, quant_format: str = "nvfp4",
                 decode_target: str = "gpu", hybrid_max_fetch: int = 1, layout: dict[str, BankSpec] | None = None,
                 max_slots: int | None = None, host_tables: bool = False):
        if cache_policy != "lru":
            raise AssertionError(f"unknown cache policy {cache_policy!r}")
        if decode_target != "gpu":
            raise ValueError("this cache has no CPU executor: decode_target must be 'gpu'")
        self.num_layers, self.num_experts = num_layers, num_experts
        self.device = torch.device(device)
        self.cache_policy, self.quant_format, self.decode_target = cache_policy, quant_format, decode_target
        self.prefill_overlap, self.prefill_hit_d2d = prefill_overlap, prefill_hit_d2d
        self.layout, self.max_slots = layout, max_slots
        self.host_tables = host_tables
        # chunks shorter than this move only the experts their router selected (0 = always whole layers)
        self.prefill_selected_max = 0
        self.prefill_selected_active = False
        self.prefill_selected_chunks = 0
        self.prefill_d2d_rows = self.prefill_h2d_rows = 0
        self.collect_stats = False
        self.decode_shared_overlap = False
        self.layer_major_active = False
        self.refill = None
        self.cpu_layer_ids: frozenset = frozenset()
        self.bank_schema = tuple(layout) if layout is not None else ops.ROLES
        self.bank_sources: dict[str, list[torch.Tensor]] = {}
        self.bank_caches: dict[str, torch.Tensor] = {}
        self.banks: list[tuple[list[torch.Tensor], torch.Tensor]] = []
        self._copy_fused_ok = False
        self._pending_src_layer: int | None = None
        self._pending_whole_layer = False
        self.h2d_bytes = 0
        self.validate_rebuild(cache_size)
        if prefill_overlap and cache_size < 2 * num_experts:
            raise AssertionError("prefill overlap borrows two expert-layer buffers: cache_size must be >= 2 * num_experts")
        self._alloc_tables(cache_size)

    # ---- tables --------------------------------------------------------------------------------------
    def _alloc_tables(self, cache_size: int) -> None:
        self.cache_size = cache_size
        dev = torch.device("cpu") if self.host_tables else self.device
        self.slot_for_id = torch.full((self.num_layers, self.num_experts), -1, dtype=torch.int32, device=dev)
        self.id_of_slot = torch.full((cache_size,), -1, dtype=torch.int32, device=dev)
        self.usage = torch.zeros((cache_size,), dtype=torch.int64, device=dev)
        self.step = torch.zeros((), dtype=torch.int64, device=dev)
        plan = max(self.num_experts, cache_size)
        self.evict_slots = torch.zeros((plan,), dtype=torch.int32, device=dev)
        self.src_indices = torch.zeros((plan,), dtype=torch.int32, device=dev)
        self.num_indices = torch.zeros((1,), dtype=torch.int64, device=dev)
        self.lru_stats = torch.zeros((self.num_layers, N_STATS), dtype=torch.int64, device=dev)

    def _tables(self, layer_id: int | None = None) -> SlotTables:
        stats = self.lru_stats[layer_id] if (self.collect_stats and layer_id is not None) else None
        return SlotTables(ptr(self.slot_for_id), ptr(self.id_of_slot), ptr(self.usage), ptr(self.step),
                          ptr(self.src_indices), ptr(self.evict_slots), ptr(self.num_indices), ptr(stats),
                          self.num_layers, self.num_experts, self.cache_size)

    def validate_rebuild(self, cache_size: int) -> None:
        if cache_size < self.num_experts:
            raise ValueError(f"cache_size {cache_size} < num_experts {self.num_experts}")
        if self.max_slots is not None and cache_size > self.max_slots:
            raise ValueError(f"moe_cache_size={cache_size} exceeds the expert kernel's slot limit of {self.max_slots}")

    def rebuild(self, cache_size: int) -> None:
        """Resize the slot cache in place; host banks stay, every slot cold-starts."""
        self.validate_rebuild(cache_size)
        sources = self.bank_sources
        self.bank_caches, self.banks = {}, []
        self._alloc_tables(cache_size)
        if sources:
            self.set_bank_sources(sources)

    def reset(self) -> None:
        if self.host_tables:
            self.slot_for_id.fill_(-1); self.id_of_slot.fill_(-1); self.usage.zero_(); self.step.zero_()
            self.num_indices.zero_()
        else:
            t = self._tables()
            check(lib().b200moe_slot_reset(C.byref(t), stream_ptr()), "b200moe_slot_reset")
        self._pending_src_layer = None

    def reset_stats(self) -> None:
        self.lru_stats.zero_()
        self.h2d_bytes = 0

    # ---- banks ---------------------------------------------------------------------------------------
    def set_bank_sources(self, sources: dict[str, list[torch.Tensor]], layer_residency=None) -> None:
        """Attach per-layer host banks (pinned ``[E, ...]`` tensors, or device tensors) and allocate the slots."""
        if set(sources) != set(self.bank_schema):
            raise AssertionError(f"banks {sorted(sources)} do not match the schema {self.bank_schema}")
        for name in self.bank_schema:
            per_layer = sources[name]
            assert len(per_layer) == self.num_layers, (name, len(per_layer))
            head = per_layer[0]
            if self.layout is not None:
                spec = self.layout[name]
                if tuple(head.shape[1:]) != tuple(spec.shape) or head.dtype != spec.dtype:
                    raise ValueError(f"bank {name!r} rows are {tuple(head.shape[1:])} {head.dtype} but the expert "
                                     f"kernel's layout wants {tuple(spec.shape)} {spec.dtype}")
            for layer_id, src in enumerate(per_layer):
                assert src.is_contiguous() and src.size(0) == self.num_experts, (name, layer_id, src.shape)
                assert src.shape == head.shape and src.dtype == head.dtype
                if not src.is_cuda and not src.is_pinned():
                    raise ValueError(f"bank {name!r} layer {layer_id} must be pinned host memory or a device tensor")
            self.bank_sources[name] = list(per_layer)
            self.bank_caches[name] = torch.empty((self.cache_size, *head.shape[1:]), dtype=head.dtype, device=self.device)
        self.banks = [(self.bank_sources[n], self.bank_caches[n]) for n in self.bank_schema]
        self._build_copy_plan()

    # ---- record layout: the six roles of a slot in ONE contiguous record, so a miss is one copy -----------
    @staticmethod
    def record_views(records: torch.Tensor, layout: dict[str, BankSpec]) -> dict[str, torch.Tensor]:
        """Role views ``[N, *shape]`` into ``records [N, record_bytes]`` (uint8); slots are strided by the record."""
        out, off = {}, 0
        n = records.shape[0]
        for role, spec in layout.items():
            nbytes = int(torch.tensor([], dtype=spec.dtype).element_size())
            for d in spec.shape:
                nbytes *= d
            out[role] = records[:, off:off + nbytes].view(spec.dtype).view(n, *spec.shape)
            off += nbytes
        assert off <= records.shape[1]
        return out

    @staticmethod
    def record_bytes(layout: dict[str, BankSpec]) -> int:
        total = 0
        for spec in layout.values():
            n = int(torch.tensor([], dtype=spec.dtype).element_size())
            for d in spec.shape:
                n *= d
            total += n
        return total

    def set_record_sources(self, records: list[torch.Tensor]) -> None:
        """Attach per-layer host banks given as ``[E, record_bytes]`` uint8 tensors (pinned, or on the device) and
        allocate the slot cache as ``[cache_size, record_bytes]``.  ``bank_caches`` / ``bank_views`` expose the
        usual role tensors as strided views; a miss fill moves one contiguous record."""
        if self.layout is None:
            raise ValueError("the record layout needs the kernel's bank layout")
        rb = self.record_bytes(self.layout)
        assert len(records) == self.num_layers
        for r in records:
            assert r.dtype == torch.uint8 and r.shape == (self.num_experts, rb) and r.is_contiguous()
            if not r.is_cuda and not r.is_pinned():
                raise ValueError("records must be pinned host memory or device tensors")
        self.records = list(records)
        self.record_cache = torch.empty((self.cache_size, rb), dtype=torch.uint8, device=self.device)
        self.bank_caches = self.record_views(self.record_cache, self.layout)
        self.bank_sources = {role: [self.record_views(r, self.layout)[role] for r in records] for role in self.layout}
        self.banks = [(self.records, self.record_cache)]  # one "bank": the whole record
        self._build_copy_plan()

    def _build_copy_plan(self) -> None:
        rows = [c[0].numel() * c.element_size() for _, c in self.banks]
        self._row_bytes_host = (C.c_int64 * len(rows))(*rows)
        self._dst_host = (C.c_void_p * len(rows))(*[c.data_ptr() for _, c in self.banks])
        self._src_host = [(C.c_void_p * len(rows))(*[per_layer[l].data_ptr() for per_layer, _ in self.banks])
                          for l in range(self.num_layers)]
        self._row_bytes_dev = torch.tensor(rows, dtype=torch.int64, device=self.device)
        self._dst_dev = torch.tensor([c.data_ptr() for _, c in self.banks], dtype=torch.int64, device=self.device)
        self._src_dev = [torch.tensor([per_layer[l].data_ptr() for per_layer, _ in self.banks], dtype=torch.int64,
                                      device=self.device) for l in range(self.num_layers)]
        self.expert_bytes = sum(rows)
        self._copy_fused_ok = all(r % 16 == 0 for r in rows)

    def bank_views(self, n: int | None = None) -> tuple[torch.Tensor, ...]:
        assert self.banks, "set_bank_sources must register the banks first"
        caches = [self.bank_caches[r] for r in self.bank_schema]
        return tuple(c if n is None else c[:n] for c in caches)

    def bank_dict(self, n: int | None = None) -> dict[str, torch.Tensor]:
        return dict(zip(self.bank_schema, self.bank_views(n)))

    def alphas_for_slots(self, layer_id: int):
        return None  # this layout keeps its global scales inside the banks

    alphas_for_layer = alphas_for_slots

    def set_alphas(self, *args, **kwargs) -> None:
        return None

    def is_cpu_layer(self, layer_id: int) -> bool:
        return False

    def is_unpinned_layer(self, layer_id: int) -> bool:
        return False

    # ---- device-planned path -------------------------------------------------------------------------
    def ensure_experts(self, layer_id: int, expert_ids: torch.Tensor) -> None:
        """LRU ensure on the device tables; rewrites ``expert_ids`` IN PLACE to slot ids."""
        if self.host_tables:
            raise RuntimeError("this cache keeps host tables: use ensure_experts_host")
        assert expert_ids.dtype == torch.int32 and expert_ids.is_cuda and expert_ids.is_contiguous()
        t = self._tables(layer_id)
        check(lib().b200moe_slot_ensure(C.byref(t), layer_id, ptr(expert_ids), expert_ids.numel(), ptr(expert_ids),
                                        stream_ptr()), "b200moe_slot_ensure")
        self._pending_src_layer, self._pending_whole_layer = layer_id, False

    def materialize_layer(self, layer_id: int) -> None:
        if self.host_tables:
            raise RuntimeError("materialize_layer needs device tables")
        t = self._tables(layer_id)
        check(lib().b200moe_slot_materialize(C.byref(t), layer_id, stream_ptr()), "b200moe_slot_materialize")
        self._pending_src_layer, self._pending_whole_layer = layer_id, True

    def copy_missing(self) -> None:
        layer_id = self._pending_src_layer
        assert self.banks, "set_bank_sources must register the banks first"
        assert layer_id is not None, "no staged misses (ensure_experts/materialize_layer first)"
        if self._pending_whole_layer:
            for per_layer, cache in self.banks:  # position == expert id: one plain copy per bank
                cache[: self.num_experts].copy_(per_layer[layer_id], non_blocking=True)
            return
        self.copy_planned(layer_id)

    def copy_planned(self, layer_id: int, tma: bool = True, blocks_per_bank: int = 8) -> None:
        """Gather the staged plan from ``layer_id``'s banks with one fixed-shape launch."""
        if not self._copy_fused_ok:
            raise RuntimeError("bank rows must be multiples of 16 bytes")
        check(lib().b200moe_slot_gather(len(self.banks), ptr(self._dst_dev), ptr(self._src_dev[layer_id]),
                                        ptr(self._row_bytes_dev), ptr(self.evict_slots), ptr(self.src_indices),
                                        ptr(self.num_indices), min(self.cache_size, self.evict_slots.numel()),
                                        blocks_per_bank, stream_ptr()), "b200moe_slot_gather")

    # ---- host-planned path ---------------------------------------------------------------------------
    def ensure_experts_host(self, layer_id: int, expert_ids: torch.Tensor) -> int:
        """Same policy on host tables; ``expert_ids`` (CPU int32) is rewritten in place. Returns the miss count."""
        if not self.host_tables:
            raise RuntimeError("this cache keeps device tables: use ensure_experts")
        assert expert_ids.dtype == torch.int32 and not expert_ids.is_cuda and expert_ids.is_contiguous()
        t = self._tables(layer_id)
        check(lib().b200moe_slot_ensure_host(C.byref(t), layer_id, ptr(expert_ids), expert_ids.numel(), ptr(expert_ids)),
              "b200moe_slot_ensure_host")
        self._pending_src_layer, self._pending_whole_layer = layer_id, False
        return int(self.num_indices[0])

    def fill_planned(self, layer_id: int, stream: torch.cuda.Stream | None = None) -> int:
        """One cudaMemcpyAsync per (miss, bank) of the host plan, on ``stream`` (default: current). Returns bytes."""
        n = int(self.num_indices[0])
        if n == 0:
            return 0
        s = stream.cuda_stream if stream is not None else stream_ptr()
        check(lib().b200moe_slot_fill(len(self.banks), self._dst_host, self._src_host[layer_id], self._row_bytes_host,
                                      ptr(self.evict_slots), ptr(self.src_indices), n, s), "b200moe_slot_fill")
        self.h2d_bytes += n * self.expert_bytes
        return n * self.expert_bytes

    # ---- prefill double buffer: slots [0, 2E) as two whole-layer buffers ---------------------------------
    def begin_prefill(self) -> None:
        if not self.prefill_overlap:
            raise RuntimeError("prefill_overlap is off")
        if not hasattr(self, "_copy_stream"):
            self._copy_stream = torch.cuda.Stream(self.device)
            self._ready = [torch.cuda.Event(), torch.cuda.Event()]
            self._released = [torch.cuda.Event(), torch.cuda.Event()]
            self._buffer_layer = [None, None]
        self._invalidate_prefill_buffer()
        for ev in self._released:
            ev.record(torch.cuda.current_stream(self.device))

    def _invalidate_prefill_buffer(self) -> None:
        """Slots [0, 2E) stop being LRU residents: unmap their owners and zero their usage."""
        two_e = 2 * self.num_experts
        owners = self.id_of_slot[:two_e]
        flat = self.slot_for_id.view(-1)
        valid = owners >= 0
        flat[owners[valid].long()] = -1
        self.id_of_slot[:two_e] = -1
        self.usage[:two_e] = 0

    def prefetch_prefill_layer(self, layer_id: int) -> None:
        b = layer_id % 2
        if self._buffer_layer[b] == layer_id:
            return
        self._copy_stream.wait_event(self._released[b])
        with torch.cuda.stream(self._copy_stream):
            for per_layer, cache in self.banks:
                cache[b * self.num_experts:(b + 1) * self.num_experts].copy_(per_layer[layer_id], non_blocking=True)
            self._ready[b].record(self._copy_stream)
        self._buffer_layer[b] = layer_id
        self.h2d_bytes += self.num_experts * self.expert_bytes

    # ---- selected-experts form and hit/miss split --------------------------------------------------------
    def select_prefill_route(self, tokens: int) -> None:
        """Decide, before this chunk's ``begin_prefill``, whether it moves only the experts its router selects
        (short chunks) instead of whole layers."""
        self.prefill_selected_active = bool(self.prefill_overlap and not self.host_tables
                                            and 0 < tokens < self.prefill_selected_max and self._copy_fused_ok)
        if self.prefill_selected_active:
            self.prefill_selected_chunks += 1

    def _split_lists(self):
        if not hasattr(self, "_xfer_lists"):
            e = self.num_experts
            self._xfer_lists = [tuple(torch.zeros((e,), dtype=torch.int32, device=self.device) for _ in range(4))
                                + (torch.zeros((2,), dtype=torch.int64, device=self.device),) for _ in range(2)]
            self._xfer_event = torch.cuda.Event()
        return self._xfer_lists

    def _split_and_fill(self, layer_id: int, topk_ids, select_all: bool) -> None:
        """Residents of ``layer_id`` (slots outside the two buffers) are gathered cache -> buffer on the current
        stream; the rest come from the host bank on the copy stream (device gather over the pinned bank); the
        current stream then waits for both.  Reads the slot map only."""
        b = layer_id % 2
        e = self.num_experts
        hit_dst, hit_src, miss_dst, miss_src, counts = self._split_lists()[b]
        ids = topk_ids.reshape(-1) if topk_ids is not None else None
        check(lib().b200moe_prefill_split(ptr(ids), 0 if ids is None else ids.numel(), ptr(self.slot_for_id[layer_id]), e,
                                          2 * e, b * e, int(select_all), ptr(hit_dst), ptr(hit_src), ptr(miss_dst),
                                          ptr(miss_src), ptr(counts), stream_ptr()), "b200moe_prefill_split")
        compute = torch.cuda.current_stream(self.device)
        self._xfer_event.record(compute)
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._xfer_event)
            check(lib().b200moe_slot_gather(len(self.banks), ptr(self._dst_dev), ptr(self._src_dev[layer_id]),
                                            ptr(self._row_bytes_dev), ptr(miss_dst), ptr(miss_src), ptr(counts[1:]), e, 8,
                                            stream_ptr()), "b200moe_slot_gather")
            self._ready[b].record(self._copy_stream)
        # hits: cache rows -> buffer rows of the same tensors (a wide grid: this is an HBM-to-HBM copy)
        check(lib().b200moe_slot_gather(len(self.banks), ptr(self._dst_dev), ptr(self._dst_dev), ptr(self._row_bytes_dev),
                                        ptr(hit_dst), ptr(hit_src), ptr(counts[:1]), e, 64, stream_ptr()),
              "b200moe_slot_gather")
        compute.wait_event(self._ready[b])

    def selected_prefill_layer(self, layer_id: int, topk_ids: torch.Tensor) -> dict[str, torch.Tensor]:
        """Fill this layer's buffer with only the experts ``topk_ids`` routes to (after the router) and return its
        bank views (row == expert id, like the whole-layer path); rows of experts nobody routes to are stale."""
        assert self.prefill_selected_active, "select_prefill_route first"
        self._split_and_fill(layer_id, topk_ids, select_all=False)
        self._buffer_layer[layer_id % 2] = None
        b, e = layer_id % 2, self.num_experts
        return {n: self.bank_caches[n][b * e:(b + 1) * e] for n in self.bank_schema}

    def prefetch_prefill_layer_split(self, layer_id: int) -> None:
        """Whole layer into its buffer with the resident experts copied device-to-device and only the others
        crossing the bus (``prefill_hit_d2d``)."""
        b = layer_id % 2
        if self._buffer_layer[b] == layer_id:
            return
        torch.cuda.current_stream(self.device).wait_event(self._released[b])
        self._copy_stream.wait_event(self._released[b])
        self._split_and_fill(layer_id, None, select_all=True)
        self._buffer_layer[b] = layer_id

    def prefill_transfer_stats(self) -> dict:
        """Rows moved by the last split calls: (device-to-device hits, host-to-device misses) per buffer."""
        out = {}
        for b, lists in enumerate(self._split_lists()):
            hits, misses = (int(v) for v in lists[4].cpu())
            out[b] = {"d2d_rows": hits, "h2d_rows": misses}
        return out

    def wait_prefill_layer(self, layer_id: int) -> dict[str, torch.Tensor]:
        b = layer_id % 2
        assert self._buffer_layer[b] == layer_id, "prefetch_prefill_layer first"
        torch.cuda.current_stream(self.device).wait_event(self._ready[b])
        e = self.num_experts
        # the per-role cache views work for both layouts (separate banks, or one record per slot)
        return {n: self.bank_caches[n][b * e:(b + 1) * e] for n in self.bank_schema}

    def release_prefill_layer(self, layer_id: int) -> None:
        b = layer_id % 2
        self._released[b].record(torch.cuda.current_stream(self.device))
        self._buffer_layer[b] = None

    # ---- stats ---------------------------------------------------------------------------------------
    def decode_miss_stats_per_layer(self) -> list[dict]:
        """Per-layer (active, missing, calls) as the reference's per-layer reader reports them."""
        rows = self.lru_stats.cpu().tolist()
        return [{"layer": l, "active": int(a), "missing": int(m), "calls": int(c),
                 "miss_rate": (m / a) if a else 0.0} for l, (a, m, c) in enumerate(rows)]

    def decode_routing_stats(self) -> dict:
        """Totals over all layers: distinct experts asked for, misses among them, ensure calls."""
        active, missing, calls = (int(v) for v in self.lru_stats.sum(0))
        return {"active": active, "missing": missing, "calls": calls}

    def decode_miss_stats(self) -> dict:
        active, missing, calls = (int(v) for v in self.lru_stats.sum(0))
        return {"layer_calls": calls, "active_per_layer": active / calls if calls else 0.0,
                "missing_per_layer": missing / calls if calls else 0.0,
                "miss_rate": missing / active if active else 0.0, "h2d_bytes": self.h2d_bytes}


__all__ = ["SlotCache", "N_STATS"]
