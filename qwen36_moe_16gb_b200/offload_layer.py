"""The movement decision tree of a MoE layer whose experts sit behind the slot cache.

Mirror of ``OffloadMoELayer`` (``freetoken/python/freetoken/layers/moe.py:286-339,390-459``): the routed experts of a
layer are computed by the expert kernels on whatever view of the banks the movement step produced.

  decode   ``ensure_experts`` rewrites the ids to slot ids, ``copy_missing`` fills the planned misses, the GEMVs
           read the whole slot cache (``_decode_routed``); with the shared expert given, the fill is forked to a
           side stream while the shared rows run (``forward_with_shared``).
  prefill  whole layers stream through the two prefill buffers behind the previous layer's GEMMs
           (``prefill_overlap``: prefetch L and L+1, wait L, GEMMs, release L); short chunks move only the experts
           their router selected (``select_prefill_route`` / ``selected_prefill_layer``); with ``prefill_hit_d2d``
           resident experts are copied device-to-device and only the others cross the bus; without overlap the
           layer is materialised synchronously.  Position == expert id in every prefill view, so the routing ids
           pass through unmapped.
"""
from __future__ import annotations

import torch

from . import ops
from .kernel import DECODE_MAX_TOKENS


class OffloadMoELayer:
    def __init__(self, layer_id: int, num_experts: int, top_k: int, cache):
        self.layer_id, self.num_experts, self.top_k, self.offload_cache = layer_id, num_experts, top_k, cache

    # ---- the expert kernels on a view ---------------------------------------------------------------------
    def _expert_gemm(self, x, topk_weights, topk_ids, views: dict[str, torch.Tensor], is_prefill: bool):
        if not is_prefill and x.shape[0] <= DECODE_MAX_TOKENS:
            return ops.decode_experts(x, views, topk_weights, topk_ids)
        return ops.prefill_experts(x, views, topk_weights, topk_ids)

    # ---- decode ---------------------------------------------------------------------------------------------
    def _decode_routed(self, x, topk_weights, topk_ids):
        cache = self.offload_cache
        cache.ensure_experts(self.layer_id, topk_ids)      # ids become slot ids, in place
        cache.copy_missing()
        return self._expert_gemm(x, topk_weights, topk_ids, cache.bank_dict(), is_prefill=False)

    def forward_with_shared(self, x, topk_weights, topk_ids, shared_forward):
        """Same kernels and merge order; only the transport moves to the side stream."""
        cache = self.offload_cache
        cache.ensure_experts(self.layer_id, topk_ids)
        shared = cache.decode_shared_overlap.run(cache.copy_missing, lambda: shared_forward(x))
        routed = self._expert_gemm(x, topk_weights, topk_ids, cache.bank_dict(), is_prefill=False)
        return routed, shared

    # ---- prefill --------------------------------------------------------------------------------------------
    def _wait_prefill_overlap(self, cache):
        if self.layer_id == 0:
            cache.begin_prefill()
        fetch = cache.prefetch_prefill_layer_split if cache.prefill_hit_d2d else cache.prefetch_prefill_layer
        fetch(self.layer_id)
        if self.layer_id + 1 < cache.num_layers:
            fetch(self.layer_id + 1)
        return cache.wait_prefill_layer(self.layer_id)

    def _prefill_routed(self, x, topk_weights, topk_ids):
        cache = self.offload_cache
        if cache.prefill_overlap:
            if self.layer_id == 0:
                cache.select_prefill_route(x.shape[0])
            if cache.prefill_selected_active:
                if self.layer_id == 0:
                    cache.begin_prefill()
                views = cache.selected_prefill_layer(self.layer_id, topk_ids)
            else:
                views = self._wait_prefill_overlap(cache)
            out = self._expert_gemm(x, topk_weights, topk_ids, views, is_prefill=True)
            cache.release_prefill_layer(self.layer_id)
            return out
        cache.materialize_layer(self.layer_id)
        cache.copy_missing()
        return self._expert_gemm(x, topk_weights, topk_ids, cache.bank_dict(self.num_experts), is_prefill=True)

    def forward(self, x, topk_weights, topk_ids, is_prefill: bool):
        if is_prefill:
            return self._prefill_routed(x, topk_weights, topk_ids)
        return self._decode_routed(x, topk_weights, topk_ids)


__all__ = ["OffloadMoELayer"]
