"""Expert-parallel prefill across the GPUs of one box (the reference has no expert parallelism; this is the
multi-GPU form of its prefill path ``fused_experts_nvfp4``, ``freetoken/python/freetoken/moe/fused_nvfp4.py:287-333``).

Partition: rank r owns experts ``[r*E/N, (r+1)*E/N)`` (banks of its experts only); tokens are split evenly;
router and shared-expert weights are replicated.  One step on every rank:

  1. route locally (logits GEMM, shared expert, top-k);
  2. DISPATCH (all-to-all-v): a token row travels ONCE to every rank that owns at least one of its routes,
     with its 8 local expert ids (-1 where the route lives elsewhere) and router weights;
  3. run the local grouped GEMMs on what arrived -> one bf16 row per (token, route), router weight applied;
  4. COMBINE (all-to-all-v): every per-route row goes back to the token's home rank;
  5. home rank sums its token's routes in k order and merges the shared expert.

Step 5 adds exactly the rows the single-GPU path adds, in the same order, so the result is bit-identical to
the single-GPU result.  Collectives are NCCL (NVLink/NVSwitch) through ``torch.distributed``; received rows
always land in local HBM before a kernel reads them.  ``expert_fn`` / ``combine_fn`` can be replaced (the CPU
tests run the same plan over gloo with the oracle as the expert function).
"""
from __future__ import annotations

import torch


def plan_dispatch(topk_ids: torch.Tensor, num_experts: int, world: int):
    """Host-free index plan (pure tensor ops, any device).

    Returns dict with
      send_tok   [n_send]      token index of every (token, destination) pair, grouped by destination, token-ascending
      send_counts[world]       rows per destination
      local_ids  [n_send, k]   expert id local to the destination, -1 for routes that live elsewhere
      route_perm [T*k]         flat route ids grouped by destination rank ((t,k) ascending inside a group)
      route_counts[world]      routes per destination
    """
    t, k = topk_ids.shape
    epr = num_experts // world
    valid = topk_ids >= 0
    dest = torch.where(valid, torch.div(topk_ids, epr, rounding_mode="floor"), torch.full_like(topk_ids, -1))
    ranks = torch.arange(world, device=topk_ids.device, dtype=dest.dtype)
    hit = (dest.unsqueeze(0) == ranks.view(world, 1, 1)).any(dim=2)       # [world, T]
    pair = hit.nonzero()                                                  # rows sorted by (rank, token)
    send_rank, send_tok = pair[:, 0], pair[:, 1]
    send_counts = hit.sum(dim=1)
    ids_sel = topk_ids[send_tok]
    mine = dest[send_tok] == send_rank.unsqueeze(1).to(dest.dtype)
    local_ids = torch.where(mine, ids_sel - (send_rank.unsqueeze(1) * epr).to(ids_sel.dtype), torch.full_like(ids_sel, -1))
    flat_dest = dest.reshape(-1)
    order = torch.sort(torch.where(flat_dest >= 0, flat_dest, torch.full_like(flat_dest, world)), stable=True).indices
    route_counts = torch.bincount(flat_dest[flat_dest >= 0].long(), minlength=world)
    route_perm = order  # valid routes first (grouped by destination), dropped routes at the end
    return {"send_tok": send_tok, "send_counts": send_counts, "local_ids": local_ids.to(torch.int32).contiguous(),
            "route_perm": route_perm, "route_counts": route_counts}


def _a2a(dist, out, inp, out_splits, in_splits, group=None):
    """all-to-all-v of rows; rows travel as raw bytes (every backend moves uint8)."""
    out, inp = out.view(torch.uint8), inp.view(torch.uint8)
    dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


def ep_prefill_step(dist, x, topk_weights, topk_ids, num_experts, expert_fn, combine_fn, group=None):
    """One expert-parallel pass.  ``expert_fn(x_recv, w_recv, local_ids) -> [n_recv, k, H]`` per-route rows
    (rows of -1 routes are ignored); ``combine_fn(ic3 [T,k,H], topk_ids) -> [T,H]``.  Returns (out, stats)."""
    world = dist.get_world_size(group)
    t, k = topk_ids.shape
    h = x.shape[1]
    dev = x.device
    plan = plan_dispatch(topk_ids, num_experts, world)
    counts = torch.stack([plan["send_counts"], plan["route_counts"]]).to(torch.int64)        # [2, world]
    got = torch.empty_like(counts)
    dist.all_to_all_single(got.view(-1), counts.t().contiguous().view(-1), group=group)       # [world, 2] each way
    got = got.view(world, 2)
    send_rows, send_routes = plan["send_counts"].tolist(), plan["route_counts"].tolist()
    recv_rows, recv_routes = got[:, 0].tolist(), got[:, 1].tolist()
    n_recv = sum(recv_rows)

    # ---- dispatch ------------------------------------------------------------------------------------
    tok = plan["send_tok"]
    x_send = x[tok]
    meta_send = torch.cat([plan["local_ids"].view(torch.float32), topk_weights[tok]], dim=1).contiguous()  # [n, 2k] 4-byte words
    x_recv = torch.empty((n_recv, h), dtype=x.dtype, device=dev)
    meta_recv = torch.empty((n_recv, 2 * k), dtype=torch.float32, device=dev)
    _a2a(dist, x_recv, x_send, recv_rows, send_rows, group)
    _a2a(dist, meta_recv, meta_send, recv_rows, send_rows, group)
    ids_recv = meta_recv[:, :k].contiguous().view(torch.int32)
    w_recv = meta_recv[:, k:].contiguous()

    # ---- local experts ---------------------------------------------------------------------------------
    if n_recv:
        ic3_local = expert_fn(x_recv, w_recv, ids_recv)                   # [n_recv, k, H]
        back = ic3_local.reshape(n_recv * k, h)[(ids_recv.reshape(-1) >= 0).nonzero().reshape(-1)]
    else:
        back = torch.empty((0, h), dtype=x.dtype, device=dev)

    # ---- combine ---------------------------------------------------------------------------------------
    n_routes = sum(send_routes)
    rows = torch.empty((n_routes, h), dtype=x.dtype, device=dev)
    _a2a(dist, rows, back.contiguous(), send_routes, recv_routes, group)
    ic3 = torch.empty((t * k, h), dtype=x.dtype, device=dev)
    ic3[plan["route_perm"][:n_routes]] = rows
    out = combine_fn(ic3.view(t, k, h), topk_ids)
    stats = {"dispatch_rows": int(sum(send_rows)), "recv_rows": n_recv, "recv_routes": int(sum(recv_routes)),
             "dispatch_bytes": int(sum(send_rows)) * (h * 2 + 8 * k), "combine_bytes": n_routes * h * 2}
    return out, stats


class PeerCombine:
    """Symmetric (peer-mapped) buffers of one rank: the per-route output rows `ic3` that every rank's second
    grouped GEMM stores into, and this rank's tokens + routing (`x`, `meta`) that the other ranks pull."""

    def __init__(self, dist, tokens: int, top_k: int, hidden: int, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.dist, self.world, self.rank = dist, dist.get_world_size(), dist.get_rank()
        self.tokens, self.top_k, self.hidden = tokens, top_k, hidden
        ic3_bytes = tokens * top_k * hidden * 2
        x_bytes = tokens * hidden * 2
        meta_bytes = tokens * 2 * top_k * 4
        self._offsets = (0, ic3_bytes, ic3_bytes + x_bytes)
        self.buf = symm_mem.empty((ic3_bytes + x_bytes + meta_bytes,), dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buf, dist.group.WORLD)
        self.ic3 = self.buf[:ic3_bytes].view(torch.bfloat16).view(tokens * top_k, hidden)
        self.x = self.buf[ic3_bytes:ic3_bytes + x_bytes].view(torch.bfloat16).view(tokens, hidden)
        self.meta = self.buf[ic3_bytes + x_bytes:].view(torch.float32).view(tokens, 2 * top_k)
        self.peer_ptrs = torch.tensor(list(self.handle.buffer_ptrs), dtype=torch.int64, device=device)
        self.copy_stream = torch.cuda.Stream(device)
        self.x_stage = torch.empty((self.world, tokens, hidden), dtype=torch.bfloat16, device=device)
        self.meta_stage = torch.empty((self.world, tokens, 2 * top_k), dtype=torch.float32, device=device)
        self.events = [torch.cuda.Event() for _ in range(self.world)]
        self.tokens_published = False

    def peer_x(self, r):
        return self.handle.get_buffer(r, (self.tokens, self.hidden), torch.bfloat16, self._offsets[1] // 2)

    def peer_meta(self, r):
        return self.handle.get_buffer(r, (self.tokens, 2 * self.top_k), torch.float32, self._offsets[2] // 4)

    def barrier(self):
        self.handle.barrier()  # on the current stream: all ranks' earlier stores are visible afterwards

    def publish_tokens(self, x: torch.Tensor) -> None:
        """Early half of the exchange: the tokens do not depend on the routing, so a rank can publish them and start
        pulling the other ranks' tokens (copy stream, ring order) BEFORE it runs its router and shared expert; the
        pulls then hide behind those GEMMs.  :func:`ep_prefill_step_peer` notices and only exchanges the routing."""
        main = torch.cuda.current_stream(x.device)
        self.x.copy_(x)
        self.barrier()
        self.x_stage[0].copy_(self.x)
        self.copy_stream.wait_stream(main)
        with torch.cuda.stream(self.copy_stream):
            for j in range(1, self.world):
                self.x_stage[j].copy_(self.peer_x((self.rank + j) % self.world), non_blocking=True)
        self.tokens_published = True


def source_groups(world: int, sizes) -> list[list[int]]:
    """Ring positions 0 .. world-1 (position j = rank + j modulo world; position 0 is the rank itself) cut into
    consecutive chunks: ``sizes`` is one chunk length for all, or a list of lengths (the last one repeats).  The
    tokens of a chunk are one contiguous (wrapping) slice of the box's tokens, which one grouped-GEMM call takes
    together."""
    if isinstance(sizes, int):
        sizes = [sizes]
    out, i, n = [], 0, 0
    while i < world:
        step = max(1, sizes[min(n, len(sizes) - 1)])
        out.append(list(range(i, min(world, i + step))))
        i += step
        n += 1
    return out


def default_group_size(world: int):
    """Ring positions per grouped-GEMM call.  A call costs a fixed ~0.1 ms (permutation, tile list, pipeline fill and
    drain of two kernels, a shorter tile list to balance), more than the NVLink pull of a few ranks' tokens: up to
    four ranks everything goes into one call after the pulls have landed; beyond, two calls of half the ring each,
    the second one's pulls hidden behind the first (measured on 8 GPUs: 4+4 1.84-1.93 ms, 2+6 1.86, 1+7 2.03,
    one call 2.06, four calls 2.20)."""
    import os

    env = os.environ.get("B200MOE_EP_GROUP")
    if env:
        return [max(1, int(v)) for v in env.split(",")]
    return world if world <= 4 else (world + 1) // 2


def balanced_placement(counts, world: int, max_per_rank: int | None = None):
    """Which rank owns which expert, from observed (or prior) per-expert route counts: experts in descending count
    go to the least loaded rank that still has room (longest-processing-time rule).  A rank may hold up to
    ``max_per_rank`` experts (default: twice the even share), so the rank with the hottest expert holds fewer of
    them: with an even share the hottest expert plus 31 of the coldest already exceed the mean load by 20 % on
    8 ranks.  Returns int32 tensors ``owner[e]`` and ``local[e]`` (the expert's row in its owner's banks)."""
    counts = [float(c) for c in counts]
    e = len(counts)
    cap = max_per_rank if max_per_rank is not None else 2 * ((e + world - 1) // world)
    order = sorted(range(e), key=lambda i: (-counts[i], i))
    load, fill = [0.0] * world, [0] * world
    owner, local = [0] * e, [0] * e
    members: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min((r for r in range(world) if fill[r] < cap), key=lambda r: (load[r], r))
        members[r].append(i)
        fill[r] += 1
        load[r] += counts[i]
    for r in range(world):
        for j, i in enumerate(sorted(members[r])):
            owner[i], local[i] = r, j
    return torch.tensor(owner, dtype=torch.int32), torch.tensor(local, dtype=torch.int32)


def ep_prefill_step_peer(dist, peer: PeerCombine, x, topk_weights, topk_ids, num_experts, local_banks, shared=None,
                         gate=None, placement=None, out=None, marks: list | None = None):
    """Expert-parallel pass with both exchanges off the critical path (GPU only).

    Every rank publishes its tokens and routing in symmetric memory; after a barrier it (a) runs the local grouped
    GEMMs for chunks of ring positions (see :func:`source_groups`; position 0 is its own tokens) and (b) pulls the
    other ranks' tokens over NVLink on a copy stream in ring order; a chunk runs as soon as its copies have landed.
    The second GEMM stores each per-route row into the home GPU's buffer; a second barrier, then the local sum
    over routes.

    ``placement``: optional ``(owner, local)`` int32 device tensors from :func:`balanced_placement`; without it rank
    r owns the contiguous experts [r * E / world, (r + 1) * E / world).

    ``marks``: a list that receives ``(phase name, timing event)`` pairs recorded on the current stream at the phase
    boundaries (diagnostics: the events cost a few microseconds)."""
    from . import ops

    def mark(name):
        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(x.device))
            marks.append((name, ev))

    mark("start")
    world, rank = peer.world, peer.rank
    t, k = topk_ids.shape
    h = x.shape[1]
    epr = num_experts // world
    lo = rank * epr
    main = torch.cuda.current_stream(x.device)
    early = peer.tokens_published                    # publish_tokens(x) ran before the router: the pulls are under way
    peer.tokens_published = False
    if not early:
        peer.x.copy_(x)
    peer.meta.copy_(torch.cat([topk_ids.view(torch.float32), topk_weights], dim=1))
    peer.barrier()                                   # everyone's routing (and tokens) are published
    mark("publish_and_barrier")
    # staging buffers in ring order: slot j holds the tokens of rank (rank + j) % world; slot 0 is a local copy
    if not early:
        peer.x_stage[0].copy_(peer.x)
    peer.meta_stage[0].copy_(peer.meta)
    peer.copy_stream.wait_stream(main)
    with torch.cuda.stream(peer.copy_stream):
        for j in range(1, world):
            s = (rank + j) % world
            if not early:
                peer.x_stage[j].copy_(peer.peer_x(s), non_blocking=True)
            peer.meta_stage[j].copy_(peer.peer_meta(s), non_blocking=True)
            peer.events[j].record(peer.copy_stream)  # the copy stream is in order: the token pulls are covered too

    lut = None
    if placement is not None:  # expert id -> row in this rank's banks, or -1; cached on the peer object
        key = (id(placement[0]), id(placement[1]))
        if getattr(peer, "_lut_key", None) != key:
            owner, local = placement
            peer._lut = torch.cat([torch.where(owner == rank, local, torch.full_like(local, -1)),
                                   torch.full((1,), -1, dtype=local.dtype, device=local.device)])
            peer._lut_key = key
        lut = peer._lut

    def run(xs, meta, first_token):
        ids = meta[:, :k].contiguous().view(torch.int32)
        w = meta[:, k:].contiguous()
        if placement is None:
            local_ids = torch.where((ids >= lo) & (ids < lo + epr), ids - lo, torch.full_like(ids, -1))
        else:
            local_ids = lut[ids.clamp(-1, num_experts).long()]  # -1 and num_experts both index the trailing -1
        return ops.prefill_ep_routes(xs, local_banks, w, local_ids, first_token, peer.peer_ptrs, world, t)

    status = None
    for grp in source_groups(world, default_group_size(world)):
        if grp[-1] > 0:
            main.wait_event(peer.events[grp[-1]])    # pulls were issued in ring order: the last one covers the chunk
            mark("wait_tokens_of_ring_%d_%d" % (grp[0], grp[-1]))
        a, b = grp[0], grp[-1] + 1
        st = run(peer.x_stage[a:b].view(-1, h), peer.meta_stage[a:b].view(-1, 2 * k), ((rank + a) % world) * t)
        mark("grouped_gemms_ring_%d_%d" % (grp[0], grp[-1]))
        status = st if status is None else status
    peer.barrier()                                   # all rows have landed; all peers are done reading my tokens
    mark("barrier_rows_landed")
    out = ops.combine_routes(peer.ic3.view(t, k, h), topk_ids, num_experts, shared, gate, out=out)
    mark("combine")
    return out, status


class EpPrefill:
    """Synthetic expert-parallel prefill workload: T tokens per rank, Zipf(1.1) routing, local banks on the GPU."""

    # dense GEMM 3 (router, shared gate_up + SwiGLU, shared down), gate logit 1, router top-k 1, permutation 4,
    # tile list 1, grouped GEMM 2, combine 1 (the token gather between ranks is extra and depends on the ring)
    launches_per_step = 13

    early_tokens = True   # publish the tokens and start the pulls before the router and the shared expert run

    def __init__(self, dist, shape, block, banks, x, top_k):
        self.dist, self.shape, self.block, self.banks, self.x, self.top_k = dist, shape, block, banks, x, top_k
        self.world = dist.get_world_size()
        self.x_host = x.cpu().pin_memory()
        self.out_host = torch.empty_like(self.x_host).pin_memory()
        self.x_stage = torch.empty_like(x)
        self.info = {"h2d": x.numel() * 2, "d2h": x.numel() * 2}
        self.last_stats = None
        self.peer = PeerCombine(dist, x.shape[0], top_k, shape.hidden, x.device)
        self.placement = None
        self.last_status = torch.zeros(4, dtype=torch.int32, device=x.device)

    @classmethod
    def synthetic(cls, dist, shape, tokens: int, seed: int = 0, placement: str = "contiguous"):
        """``placement``: "contiguous" -- rank r owns experts [r*E/N, (r+1)*E/N) (the stated workload); "balanced" --
        experts dealt by the route counts of this batch (see :func:`balanced_placement`)."""
        from . import synth
        from .block import MoEBlock

        rank, world = dist.get_rank(), dist.get_world_size()
        dev = torch.device("cuda", torch.cuda.current_device())
        host = synth.make_layer(seed, 8, shape, zipf_alpha=1.1, with_banks=False)     # replicated dense weights + bias
        d = {k: v.to(dev) for k, v in host.items()}
        g = torch.Generator(device=dev).manual_seed(1000 + rank)
        x = torch.randn(tokens, shape.hidden, generator=g, device=dev).to(torch.bfloat16)
        block = MoEBlock(d["router_w"], d["shared_gate_up"], d["shared_down"], d["shared_gate"], shape.top_k,
                         logit_bias=d["logit_bias"])
        epr = shape.num_experts // world
        if placement == "balanced":
            # every rank counts its routes per expert, the counts are summed over the ranks, and the experts are
            # dealt so that the ranks' loads are even
            from . import ops

            _, ids = ops.fused_topk(x, block.router_logits(x), shape.top_k, True)
            counts = torch.bincount(ids.reshape(-1).long().clamp_(0, shape.num_experts - 1),
                                    minlength=shape.num_experts).float()
            dist.all_reduce(counts)
            owner, local = balanced_placement(counts.cpu().tolist(), world)
        else:
            e = torch.arange(shape.num_experts, dtype=torch.int32)
            owner, local = torch.div(e, epr, rounding_mode="floor").to(torch.int32), (e % epr).to(torch.int32)
        mine = int((owner == rank).sum())
        # the banks are synthetic: a rank draws as many experts as it owns
        banks = synth.make_banks(g, shape, num_experts=mine, device=dev)
        self = cls(dist, shape, block, banks, x, shape.top_k)
        self.placement = (owner.to(dev), local.to(dev)) if placement == "balanced" else None
        self.owner, self.local = owner, local
        self.placement_name = placement
        self.experts_here = mine
        return self

    def status_ok(self) -> bool:
        """True when no rank's grouped GEMM gave up on a bounded wait in the last step (max over the ranks)."""
        st = self.last_status.to(torch.int32).abs().max().reshape(1).clone()
        self.dist.all_reduce(st, op=self.dist.ReduceOp.MAX)
        return int(st) == 0

    def gather_banks_to_host(self):
        """Every rank's banks, collected on every rank and put in expert-id order on the host (a checker's helper:
        456 MB for the Qwen shape)."""
        from . import synth

        world = self.world
        most = int(torch.bincount(self.owner.long(), minlength=world).max())
        full = {}
        for role in synth.ROLES:
            mine = self.banks[role]
            pad = torch.zeros((most, *mine.shape[1:]), dtype=mine.dtype, device=mine.device)
            pad[:mine.shape[0]] = mine
            wire = pad.view(torch.uint8) if pad.element_size() == 1 else pad   # fp8 travels as bytes
            parts = [torch.empty_like(wire) for _ in range(world)]
            self.dist.all_gather(parts, wire)
            stacked = torch.stack([p_.cpu() for p_ in parts]).view(mine.dtype)  # [world, most, ...]
            full[role] = stacked[self.owner.long(), self.local.long()].contiguous()
        return full

    def _run(self, x, out=None, marks=None):
        from . import ops

        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(("begin", ev))
        if self.early_tokens:
            self.peer.publish_tokens(x)
        logits = self.block.router_logits(x)
        shared, gate = self.block.shared_parts(x)
        w, ids = ops.fused_topk(x, logits, self.top_k, True)
        out, self.last_status = ep_prefill_step_peer(self.dist, self.peer, x, w, ids, self.shape.num_experts, self.banks,
                                                     shared, gate, placement=self.placement, out=out, marks=marks)
        self.last_routing = (w, ids)
        return out

    def step(self):
        return self._run(self.x)

    def phases_ms(self) -> dict:
        """One more step with timing events at the phase boundaries: milliseconds per phase on this rank's compute
        stream (``dense_and_router`` = router logits, shared expert, top-k; the token pulls run on the copy stream and
        show up only as ``wait_tokens_*``)."""
        marks: list = []
        self._run(self.x, marks=marks)
        torch.cuda.synchronize()
        names = {"start": "dense_and_router"}
        return {names.get(n1, n1): round(e0.elapsed_time(e1), 4) for (_, e0), (n1, e1) in zip(marks, marks[1:])}

    def e2e_step(self):
        self.x_stage.copy_(self.x_host, non_blocking=True)
        out = self._run(self.x_stage)
        self.out_host.copy_(out, non_blocking=True)

    def pipeline(self):
        """Host tokens in, host result out, with the copies of neighbouring steps overlapping the compute."""
        from .block import HostPipeline

        # the result goes into the pipeline's own buffer: a tensor allocated per step and read on another stream
        # would make the caching allocator grow (and synchronise) inside the timed region
        return HostPipeline(lambda xd, od: self._run(xd, od), self.x_host, self.out_host, self.x.device)


__all__ = ["plan_dispatch", "ep_prefill_step", "ep_prefill_step_peer", "source_groups", "default_group_size", "balanced_placement", "PeerCombine",
           "EpPrefill"]
