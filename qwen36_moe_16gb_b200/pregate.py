"""One-layer-ahead speculative expert prefetch for single-token decode through the slot cache, and the route trace
that measures what such a predictor would have fetched.

Mirror of ``DecodePregate`` (``freetoken/python/freetoken/moe/pregate.py:120-227``) and ``RouteTrace``
(``freetoken/python/freetoken/moe/route_trace.py:31-118``).  At the start of decoder layer L+1 (after its input
norm, before its mixer) layer L+1's router is applied to ``post_attention_layernorm`` of the residual stream that
leaves layer L; the first ``cap`` predicted misses go through the unchanged LRU ensure into the shared copy plan
and the unchanged gather copies them from the host bank, all on a side stream while the mixer runs:

  compute: input_norm -> fork -> mixer -> wait(read) -> post_norm -> router -> top-k -> wait(done) -> ensure -> ...
  side:    wait(fork) -> predict -> read -> ensure(predicted misses) -> gather -> done

The real ``ensure_experts`` still runs on the real routing, so a wrong prediction costs bus traffic and residency,
never correctness.  Speculative admissions are counted in ``rows`` and not in the cache's miss statistics.
"""
from __future__ import annotations

import ctypes as C
import pathlib

import torch

from ._lib import check, lib, ptr, stream_ptr

MAX_CAP = 8


class DecodePregate:
    """Owns the side-stream fork/join of the speculative plan; one instance per cache."""

    def __init__(self, cache, device, linear_cap: int, attn_cap: int | None = None, stream=None, high_priority: bool = False):
        attn_cap = linear_cap if attn_cap is None else attn_cap
        if not (0 <= linear_cap <= MAX_CAP and 0 <= attn_cap <= MAX_CAP):
            raise ValueError(f"pre-gate caps must be 0..{MAX_CAP}")
        self.cache, self.device = cache, torch.device(device)
        self.linear_cap, self.attn_cap = linear_cap, attn_cap
        # fixed query width: duplicates collapse in the LRU ensure, so padding never adds a copy
        self.width = max(2, linear_cap, attn_cap)
        if high_priority:
            self.stream = torch.cuda.Stream(self.device, priority=-1)
        else:
            self.stream = stream if stream is not None else torch.cuda.Stream(self.device)
        self.fork, self.read, self.done = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        e = cache.num_experts
        self.logits = torch.zeros((e,), dtype=torch.float32, device=self.device)
        self.query = torch.zeros((self.width,), dtype=torch.int32, device=self.device)
        self.rows = torch.zeros((cache.num_layers,), dtype=torch.int64, device=self.device)
        self._pending = self._reading = False
        # materialise the CUDA handles before any capture
        producer = torch.cuda.current_stream(self.device)
        for event in (self.fork, self.read, self.done):
            event.record(producer)
            self.stream.wait_event(event)
        self.done.record(self.stream)
        producer.wait_event(self.done)

    def cap(self, attention: bool) -> int:
        return self.attn_cap if attention else self.linear_cap

    @staticmethod
    def predictor_ok(residual: torch.Tensor, norm_weight: torch.Tensor, gate_weight: torch.Tensor, num_experts: int) -> bool:
        h = residual.shape[-1]
        return (residual.dim() == 2 and residual.shape[0] == 1 and residual.stride(-1) == 1
                and residual.dtype == torch.bfloat16 and gate_weight.dim() == 2
                and tuple(gate_weight.shape) == (num_experts, h) and gate_weight.stride(-1) == 1
                and gate_weight.dtype == torch.bfloat16 and norm_weight.numel() == h and norm_weight.is_contiguous()
                and norm_weight.dtype == torch.bfloat16 and num_experts % 8 == 0 and num_experts <= 512)

    def launch(self, layer_id: int, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float, gate_weight: torch.Tensor,
               cap: int, top_k: int) -> None:
        """Fork the speculative plan of ``layer_id`` off the compute stream."""
        producer = torch.cuda.current_stream(self.device)
        self.join()
        self.fork.record(producer)
        self._pending = self._reading = True
        try:
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(self.fork)
                try:
                    try:
                        self._predict(layer_id, residual, norm_weight, eps, gate_weight, cap, top_k)
                    finally:
                        self.read.record(self.stream)
                    self._admit_and_copy(layer_id)
                finally:
                    self.done.record(self.stream)
        except BaseException:
            self.join()
            raise

    def release_input(self) -> None:
        """Before the compute stream rewrites the residual the predictor read."""
        if self._reading:
            torch.cuda.current_stream(self.device).wait_event(self.read)
            self._reading = False

    def join(self) -> None:
        """Before anything reuses the shared plan buffers, slot maps or slot bytes."""
        if self._pending:
            torch.cuda.current_stream(self.device).wait_event(self.done)
            self._pending = self._reading = False

    def _predict(self, layer_id, residual, norm_weight, eps, gate_weight, cap, top_k):
        cache = self.cache
        check(lib().b200moe_pregate_predict(ptr(residual), ptr(norm_weight), float(eps), ptr(gate_weight), gate_weight.stride(0),
                                            residual.shape[-1], cache.num_experts, ptr(cache.slot_for_id[layer_id]), cap, top_k,
                                            ptr(self.logits), ptr(self.query), self.width, stream_ptr()),
              "b200moe_pregate_predict")

    def _admit_and_copy(self, layer_id):
        cache = self.cache
        t = cache._tables(layer_id)
        t.stats = None                                     # speculative admissions are not the cache's misses
        check(lib().b200moe_slot_ensure(C.byref(t), layer_id, ptr(self.query), self.width, ptr(self.query), stream_ptr()),
              "b200moe_slot_ensure")
        cache.copy_planned(layer_id)
        if cache.collect_stats:
            self.rows[layer_id] += cache.num_indices[0]

    def reset_stats(self) -> None:
        self.rows.zero_()


class RouteTrace:
    """Records, per decode step and layer, the real routing, which of it missed the slot cache, and what a
    one-layer-ahead predictor would have picked, plus a snapshot of the LRU state at the first step, so the trace can
    be replayed offline through the policy with and without the speculative prefetch.  One ``.npz`` per request."""

    def __init__(self, cache, out_dir):
        self.cache, self.out = cache, pathlib.Path(out_dir)
        self.out.mkdir(parents=True, exist_ok=True)
        self.requests = 0
        self._reset()

    def _reset(self):
        self.snapshot, self.steps, self.pred = None, [], {}

    def on_prefill(self):
        self.flush()

    def predict(self, layer_id: int, predicted_ids: torch.Tensor):
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the route trace needs eager decode (it reads device values on the host)")
        self.pred[layer_id] = predicted_ids.to(torch.int32).reshape(-1)

    def observe(self, layer_id: int, expert_ids: torch.Tensor):
        c = self.cache
        if self.snapshot is None:
            self.snapshot = {k: t.detach().cpu().clone() for k, t in (("slot_for_id", c.slot_for_id), ("id_of_slot", c.id_of_slot),
                                                                      ("usage", c.usage), ("step", c.step))}
        if layer_id == 0 or not self.steps:
            self.steps.append({})
        ids = expert_ids.reshape(-1).to(torch.int32)
        missed = c.slot_for_id[layer_id][ids.long().to(c.slot_for_id.device)] < 0
        self.steps[-1][layer_id] = (ids.clone(), missed, self.pred.pop(layer_id, None))

    def flush(self):
        if self.snapshot is None or not self.steps:
            self._reset()
            return None
        import numpy as np

        c = self.cache
        n, layers = len(self.steps), c.num_layers
        k = next(iter(self.steps[0].values()))[0].numel()
        actual = np.full((n, layers, k), -1, np.int32)
        missed = np.zeros((n, layers, k), np.bool_)
        pred = np.full((n, layers, k), -1, np.int32)
        for s, step in enumerate(self.steps):
            for layer, (ids, miss, p) in step.items():
                actual[s, layer] = ids.cpu().numpy()
                missed[s, layer] = miss.cpu().numpy()
                if p is not None:
                    pred[s, layer, :min(k, p.numel())] = p.cpu().numpy()[:k]
        path = self.out / f"req{self.requests:04d}.npz"
        np.savez_compressed(path, actual=actual, missed=missed, predicted=pred, num_experts=c.num_experts,
                            cache_size=c.cache_size, **{k_: v.numpy() for k_, v in self.snapshot.items()})
        self.requests += 1
        self._reset()
        return path


__all__ = ["DecodePregate", "RouteTrace", "MAX_CAP"]
