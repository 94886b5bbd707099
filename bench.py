"""Benchmark of the NVFP4 sparse-MoE block on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the whole MoE block (router, permutation, expert GEMMs with SwiGLU, shared expert,
weighted combine + merge) over one batch of synthetic tokens.  N=1 runs the prefill workload the headline
metric is quoted on (T=8192, Zipf(1.1) routing over 256 experts) plus the T=1024/32768/65536 points, the decode
layer and the slot-cache workload; N>1 runs expert-parallel prefill of T=65536 tokens split evenly over the
ranks, experts in contiguous blocks.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "moe_prefill_tokens_per_s"
UNIT = "tokens/s"
TOKENS_PER_GPU = 8192
EP_TOTAL_TOKENS = 65536
NVFP4_DENSE_PEAK_TFLOPS = 9000.0  # nominal dense NVFP4 tensor peak of one B200
# DRAM traffic of one gate_up grouped-GEMM launch at T=8192 (dram__bytes_read.sum + dram__bytes_write.sum of a
# one-kernel ncu capture of this command with --steps 1); the JSON line names the capture it came from.
NCU_TRAFFIC_GEMM1_T8192 = {"bytes": 758_626_560, "read": 694_373_632, "write": 64_252_928,
                           "capture": "ncu --set full -k regex:grouped_gemm -s 6 -c 2 on `bench.py --steps 1 --warmup 3 --no-decode "
                                      "--no-cpu --no-cache --no-sweep` (summary: profiles/grouped_gemm_prefill_T8192.md)"}
CPU_TOKENS = 8192  # the CPU arms run the same T as the headline


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Polls NVML for SM clocks and throttle reasons from a thread while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.0005):
        self.index, self.period, self.rows, self.stop = index, period_s, [], threading.Event()
        self.thread, self.max_mhz = None, None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if visible:
                entry = visible.split(",")[self.index].strip()
                if entry.isdigit():
                    phys = int(entry)
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:  # NVML missing: the summary says so
            self.thread = None
        return self

    def _poll(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)))
            except Exception:
                pass
            time.sleep(self.period)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        flags = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = [n for n, bit in flags.items() if any(r[1] & bit for r in self.rows)]
        return {"sm_mhz": statistics.median(r[0] for r in self.rows), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.rows)}


def cpu_baseline(tokens: int, threads: int, warmup: int = 1, reps: int = 3) -> dict:
    """The oracle (a port of the reference's torch dequantise-and-matmul path) on this box's host cores, on the
    SAME workload as the GPU arm: whole block, T tokens, seeded Zipf(1.1) routing."""
    import torch

    import oracle
    from qwen36_moe_16gb_b200 import synth

    torch.set_num_threads(threads)
    layer = synth.make_layer(0, tokens, zipf_alpha=1.1)
    for _ in range(warmup):
        oracle.moe_block(layer, 8)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.moe_block(layer, 8)
        times.append(time.perf_counter() - t0)
    return {"value": tokens / statistics.median(times), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"whole MoE block, T={tokens} (the headline workload: same seed, same Zipf(1.1) routing), median of "
                      f"{reps} after {warmup} warm-up, torch {torch.__version__} fp32 on {threads} threads"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    import torch

    import oracle
    from qwen36_moe_16gb_b200 import synth

    torch.set_num_threads(threads)
    tokens = CPU_TOKENS  # the same workload as the GPU arm (one step is a few seconds of CPU work)
    layer = synth.make_layer(0, tokens, zipf_alpha=1.1)
    for _ in range(args.warmup):
        oracle.moe_block(layer, 8)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.moe_block(layer, 8)
    dt = (time.perf_counter() - t0) / args.steps
    val = tokens / dt
    cb = {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
          "sample": f"T={tokens} tokens per step: the whole seeded Zipf(1.1) prefill workload (CPU oracle, fp32 torch)"}
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"prefill_T{TOKENS_PER_GPU}_zipf1.1", "tokens_per_step": tokens},
                      "cpu_baseline": cb,
                      "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def time_events(fn, steps: int, torch) -> float:
    """Average milliseconds per call, CUDA events on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def time_pipeline(pipe, steps: int, torch) -> float:
    """Average milliseconds per step of a HostPipeline: from before the first step's host->device copy is issued
    until the last step's device->host copy has finished."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    pipe.s_in.wait_event(start)  # the first copy does not start before the clock
    for _ in range(steps):
        pipe.submit()
    pipe.join()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def decode_microbench(torch, peaks, layers: int = 40, reps: int = 20, token_counts=(1, 2, 4, 8)) -> dict:
    """Decode layer time over `layers` DISTINCT banks (18 GB: every replay streams weights from HBM, not L2),
    replayed as one CUDA graph, for M in {1, 2, 4, 8}."""
    from qwen36_moe_16gb_b200 import ops, synth
    from qwen36_moe_16gb_b200.block import MoEBlock, PrefillGraphs

    shape = synth.QWEN36
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    stacks = []
    for _ in range(layers):
        stacks.append(synth.make_banks(g, shape, device=dev))
    host = synth.make_layer(0, 8, with_banks=False)
    d = {k: v.to(dev) for k, v in host.items()}
    dense = []
    for l in range(layers):  # distinct dense weights per layer as well
        dense.append(MoEBlock((torch.randn(256, 2048, generator=g, device=dev) * 0.02).bfloat16(),
                              (torch.randn(1024, 2048, generator=g, device=dev) * 0.02).bfloat16(),
                              (torch.randn(2048, 512, generator=g, device=dev) * 0.02).bfloat16(),
                              (torch.randn(1, 2048, generator=g, device=dev) * 0.02).bfloat16(), 8))
    handles = [ops.make_banks(s) for s in stacks]
    out = {}
    for m in token_counts:
        x = d["x"][:m].contiguous()
        outs = [torch.empty_like(x), torch.empty_like(x)]

        def stack_pass():
            for l in range(layers):
                dense[l].decode_fused(x, handles[l], outs[l % 2])

        stack_pass()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack_pass()
        graph.replay()
        ms = time_events(graph.replay, reps, torch)
        distinct = 0
        for l in range(layers):
            ids = dense[l].decode_fused(x, handles[l])[3]
            distinct += int(torch.unique(ids).numel())
        torch.cuda.synchronize()
        us_layer = ms * 1e3 / layers
        bytes_layer = synth.algorithmic_bytes(m, distinct / layers, shape)
        gbs = bytes_layer / (us_layer * 1e-6) / 1e9
        out[f"M{m}"] = {"us_per_layer": round(us_layer, 3), "hbm_gbs": round(gbs, 1),
                        "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4),
                        "distinct_experts_per_layer": round(distinct / layers, 2),
                        "algorithmic_bytes_per_layer": int(bytes_layer)}
    del stacks, handles, dense
    torch.cuda.empty_cache()
    return out


def cache_bench(torch, steps: int = 512, layers: int = 40, slots: int = 4603) -> dict:
    """Expert-slot offload cache: 40 layers x 256 experts (18.2 GB NVFP4) in pinned host memory, 4603 GPU slots,
    `steps` decode steps at M=1 with Zipf(1.1) routing and 70 % reuse of the previous step's experts; every layer
    has its own router and shared-expert weights.  Three forms of the same workload:
      host_planned_lookahead16  the routing of the whole step is known on the host; fills run up to 16 layers ahead
      host_planned_lookahead1   fills of layer L overlap layer L-1 only
      device_routed             nothing is known before a layer runs: device LRU + device gather of the misses,
                                overlapped with the layer's own shared expert, 40 layers in one CUDA graph"""
    from qwen36_moe_16gb_b200 import synth
    from qwen36_moe_16gb_b200.decode_overlap import DeviceRoutedDecodeStack
    from qwen36_moe_16gb_b200.offload_runner import OffloadDecodeStack

    t0 = time.perf_counter()
    stack = OffloadDecodeStack(synth.QWEN36, layers, slots, per_layer_dense=True)
    setup_s = time.perf_counter() - t0
    routing = synth.cache_routing(seed=0, steps=steps, layers=layers)

    def host_planned(st):
        st.run(routing[:8])                       # warm-up (also warms the cache, as a served model would be)
        st.cache.reset_stats()
        res = st.run(routing)
        r = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items() if k != "out"}
        r["policy_bit_exact"] = cache_policy_check(st, routing, warm=8)
        return r

    out = host_planned(stack)
    out["form"] = "host_planned_lookahead16"
    one = OffloadDecodeStack(synth.QWEN36, layers, slots, lookahead=1, records=stack.records, per_layer_dense=True)
    out["host_planned_lookahead1"] = host_planned(one)
    one.close()
    del one
    torch.cuda.empty_cache()
    dev_stack = DeviceRoutedDecodeStack(synth.QWEN36, layers, slots, stack.records, dense_blocks=stack.blocks)
    ids_buf = torch.zeros((layers, 1, synth.QWEN36.top_k), dtype=torch.int32, device="cuda")
    dev_stack.capture(stack.x, ids_buf)
    dev_stack.run(routing[:8], ids_buf)
    dev_stack.cache.reset_stats()
    res = dev_stack.run(routing, ids_buf)
    out["device_routed"] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items() if k != "plans"}
    out.update(layers=layers, slots=slots, host_bank_gb=round(layers * 256 * synth.QWEN36.expert_bytes / 1e9, 3),
               setup_s=round(setup_s, 1), routing="Zipf(1.1), 70% reuse, seed 0", dense_weights="one set per layer",
               plan="host LRU + cudaMemcpyAsync on a copy stream (host-planned forms); device LRU kernel + gather kernel "
                    "reading the pinned bank (device-routed form)")
    stack.close()
    del stack, dev_stack
    torch.cuda.empty_cache()
    return out


def cache_policy_check(stack, routing, warm: int) -> dict:
    """NOT timed: replays the same routing (warm-up steps, then the measured steps) through the CPU policy oracle
    and compares the ordered miss plan of every (step, layer) of the measured run and the final slot tables."""
    import numpy as np

    import oracle

    cache = stack.cache
    o = oracle.SlotCacheOracle(cache.num_layers, cache.num_experts, cache.cache_size)
    for s_ in range(warm):
        for layer in range(cache.num_layers):
            o.ensure(layer, routing[s_, layer].numpy())
    plans_equal, c = True, 0
    for s_ in range(routing.shape[0]):
        for layer in range(cache.num_layers):
            o.ensure(layer, routing[s_, layer].numpy())
            src, dst = stack.miss_log[c]
            plans_equal &= src == o.src_indices.tolist() and dst == o.evict_slots.tolist()
            c += 1
    tables_equal = (np.array_equal(cache.slot_for_id.view(-1).numpy(), o.slot_for_id)
                    and np.array_equal(cache.id_of_slot.numpy(), o.id_of_slot)
                    and np.array_equal(cache.usage.numpy(), o.usage) and int(cache.step) == o.step)
    return {"miss_plans": bool(plans_equal), "tables": bool(tables_equal), "calls_compared": c,
            "checker": "oracle.SlotCacheOracle replay, outside the timed region"}


def prefill_point(torch, ops, synth, blk, banks, tokens: int, peaks: dict, steps: int, seed: int) -> dict:
    """One more point of the prefill curve on the layer that is already on the device: `tokens` fresh tokens
    (seeded), whole-block time and the time of every stage of the expert path."""
    shape = synth.QWEN36
    dev = blk.router_w.device
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(tokens, shape.hidden, generator=g, device=dev).to(torch.bfloat16)
    out = torch.empty_like(x)

    from qwen36_moe_16gb_b200.block import PrefillGraphs

    graphs = PrefillGraphs(blk, banks)

    def step():
        graphs(x, out)

    for _ in range(3):
        step()
    ms = time_events(step, steps, torch)
    logits = blk.router_logits(x)
    shared, gate = blk.shared_parts(x)
    w, ids = ops.fused_topk(x, logits, shape.top_k, True)
    ops.prefill_experts(x, banks, w, ids, shared=shared, shared_gate_logit=gate, out=out, check_status=True)
    stage = {}
    for name, mask in (("plan", ops.STAGE_PLAN), ("gemm1_gate_up_swiglu", ops.STAGE_GEMM1), ("gemm2_down", ops.STAGE_GEMM2),
                       ("combine_merge", ops.STAGE_COMBINE)):
        stage[name] = time_events(lambda: ops.prefill_experts(x, banks, w, ids, shared=shared, shared_gate_logit=gate,
                                                              out=out, stages=mask), steps, torch)
    distinct = int(torch.unique(ids).numel())
    flops = synth.routed_flops(tokens, shape)
    gemm_ms = stage["gemm1_gate_up_swiglu"] + stage["gemm2_down"]
    tf = flops / (gemm_ms * 1e-3) / 1e12
    gbs = synth.algorithmic_bytes(tokens, distinct, shape) / (ms * 1e-3) / 1e9
    res = {"tokens": tokens, "ms_per_step": round(ms, 4), "tokens_per_s": round(tokens / (ms * 1e-3), 1),
           "stages_ms": {k: round(v, 4) for k, v in stage.items()}, "routed_tflops": round(tf, 1),
           "frac_of_measured_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
           "frac_of_nominal_nvfp4_peak": round(tf / NVFP4_DENSE_PEAK_TFLOPS, 4),
           "distinct_experts": distinct, "hbm_gbs_algorithmic": round(gbs, 1),
           "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4)}
    del x, out
    torch.cuda.empty_cache()
    return res


def ep_checks(torch, dist, runner, rank: int, sample: int = 16) -> dict:
    """NOT timed.  (1) no rank's kernels gave up on a bounded wait; (2) rank 0's output rows of `sample` of its
    tokens against the CPU oracle fed the same routing and the banks collected from their owners."""
    out = runner.step().clone()
    torch.cuda.synchronize()
    status_ok = runner.status_ok()
    w, ids = runner.last_routing
    banks = runner.gather_banks_to_host()   # collective: every rank takes part
    res = {"status_ok": status_ok}
    if rank == 0:
        import oracle

        t = runner.x.shape[0]
        pick = torch.linspace(0, t - 1, sample).long()
        x = runner.x[pick.to(runner.x.device)].cpu()
        blk = runner.block
        layer = dict(banks)
        routed = oracle.moe_experts_bf16(x, layer, w[pick.to(w.device)].cpu(), ids[pick.to(ids.device)].cpu())
        shared, gate = oracle.shared_expert(x, blk.shared_gate_up.cpu(), blk.shared_down.cpu(), blk.shared_gate.cpu())
        want = oracle.shared_epilogue(routed, shared, gate)
        max_abs, rel_l2 = oracle.error_metrics(out[pick.to(out.device)].float().cpu(), want.float())
        res["parity"] = {"tokens": sample, "max_abs": max_abs, "rel_l2": rel_l2, "ok": bool(max_abs <= 2e-2 and rel_l2 <= 1e-3),
                         "gate": "max-abs 2e-2, rel-L2 1e-3 against oracle.moe_experts_bf16 + shared expert"}
    return res


def run_ours(args) -> None:
    import torch

    from qwen36_moe_16gb_b200 import build as b

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rank == 0:
        b.build()
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    from qwen36_moe_16gb_b200 import ops, synth
    from qwen36_moe_16gb_b200.block import MoEBlock, PrefillGraphs

    peaks = load_peaks()
    shape = synth.QWEN36
    # one GPU: the headline workload (T=8192); expert parallel: the stated T=65536 split evenly over the ranks
    T = TOKENS_PER_GPU if world == 1 else EP_TOTAL_TOKENS // world
    dev = torch.device("cuda", local)
    if args.only_decode:
        ms_ = tuple(int(v) for v in args.decode_m.split(","))
        print(json.dumps({"decode": decode_microbench(torch, peaks, args.decode_layers, args.decode_reps, ms_)}))
        return

    if world > 1:
        from qwen36_moe_16gb_b200 import ep

        runner = ep.EpPrefill.synthetic(dist, shape, T, seed=0, placement="contiguous")
        step, pipe, info = runner.step, runner.pipeline(), runner.info
        launches_per_step = runner.launches_per_step
        stage_ms = None
    else:
        layer = synth.make_layer(0, T, zipf_alpha=1.1)
        d = {k: v.to(dev) for k, v in layer.items()}
        banks = {r: d[r] for r in synth.ROLES}
        blk = MoEBlock(d["router_w"], d["shared_gate_up"], d["shared_down"], d["shared_gate"], shape.top_k,
                       logit_bias=d["logit_bias"])
        x_dev = d["x"]
        x_host = layer["x"].pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()
        out_dev = torch.empty_like(x_dev)

        graphs = PrefillGraphs(blk, banks)   # one captured step per (input, output) buffer pair

        def step():
            graphs(x_dev, out_dev)

        def run_block(xd, od):
            return graphs(xd, od)

        from qwen36_moe_16gb_b200.block import HostPipeline

        pipe = HostPipeline(run_block, x_host, out_host, dev)

        info = {"h2d": x_host.numel() * 2, "d2h": out_host.numel() * 2}
        # this package's kernels per step: 3 dense GEMMs (router, shared gate_up + SwiGLU, shared down), gate logit,
        # router top-k, 4 permutation, tile list, token gather, 2 grouped GEMMs, combine; no library kernel runs
        launches_per_step = 14

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    with ClockSampler(local) as clocks:
        ms = time_events(step, args.steps, torch)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    # end to end: host tokens in, host result out, every step; the copies of neighbouring steps overlap the compute
    for _ in range(3):
        pipe.submit()
    pipe.join()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_ms = time_pipeline(pipe, args.steps, torch)
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)

    total_tokens = T * world
    ep_extra = {}
    if world > 1:
        ep_extra = ep_checks(torch, dist, runner, rank)
        ep_extra["phases_ms_rank0"] = runner.phases_ms()   # every rank runs it (the step has two ring-wide barriers)
        if not args.no_balanced:
            # the same step with the experts dealt by route count instead of contiguous blocks (a deployment
            # choice, reported beside the stated workload)
            del pipe
            balanced = ep.EpPrefill.synthetic(dist, shape, T, seed=0, placement="balanced")
            for _ in range(3):
                balanced.step()
            torch.cuda.synchronize()
            dist.barrier()
            bms = torch.tensor([time_events(balanced.step, args.steps, torch)], device=dev)
            dist.all_reduce(bms, op=dist.ReduceOp.MAX)
            ep_extra["value_balanced"] = total_tokens / (float(bms) * 1e-3)
            ep_extra["status_ok_balanced"] = balanced.status_ok()
    result = {"metric": METRIC, "value": total_tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
              "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
              "scaling": "weak" if world == 1 else "strong",
              "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
              "config": {"workload": f"prefill_T{T}_zipf1.1" if world == 1 else f"ep_prefill_T{total_tokens}_zipf1.1",
                         "tokens_per_gpu": T, "hidden": 2048, "moe_intermediate": 512, "experts": 256, "top_k": 8,
                         "weights": "NVFP4 (E2M1 + E4M3 per 16 + fp32 per row), bf16 activations (fp16 inside the MMA, rows "
                                    "rescaled by powers of two), fp32 accumulate",
                         "l2": "inputs larger than L2 (456 MB of expert weights per step)",
                         "launch": "the step's 14 kernels replayed as one CUDA graph" if world == 1 else "eager launches",
                         "parallelism": "single GPU" if world == 1 else f"ep{world}"},
              "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": info["h2d"],
                      "d2h_bytes_per_step": info["d2h"]},
              "gpu_launches": launches_per_step * args.steps, "clocks": clocks.summary()}
    if world > 1:
        result["config"]["expert_placement"] = "contiguous blocks of %d experts per GPU" % (shape.num_experts // world)
        result["collective"] = ("symmetric-memory peer copies (token dispatch) + peer stores from the down GEMM's "
                                "epilogue (combine); NCCL only for set-up, timing and the checks")
        result.update(ep_extra)

    if world == 1:
        # per-stage device time of the expert path (same stream, events), for the roofline of the dominant kernel
        logits = blk.router_logits(x_dev)
        shared, gate = blk.shared_parts(x_dev)
        w, ids = ops.fused_topk(x_dev, logits, shape.top_k, True)
        ops.prefill_experts(x_dev, banks, w, ids, shared=shared, shared_gate_logit=gate, out=out_dev, check_status=True)
        stage_ms = {}
        for name, mask in (("plan", ops.STAGE_PLAN), ("gemm1_gate_up_swiglu", ops.STAGE_GEMM1),
                           ("gemm2_down", ops.STAGE_GEMM2), ("combine_merge", ops.STAGE_COMBINE)):
            stage_ms[name] = time_events(lambda: ops.prefill_experts(x_dev, banks, w, ids, shared=shared,
                                                                     shared_gate_logit=gate, out=out_dev, stages=mask),
                                         args.steps, torch)
        flops1 = T * shape.top_k * 2 * shape.hidden * 2 * shape.intermediate
        flops2 = T * shape.top_k * 2 * shape.intermediate * shape.hidden
        ach = flops1 / (stage_ms["gemm1_gate_up_swiglu"] * 1e-3) / 1e12
        result["roofline"] = {"bound": "tensor", "kernel": "grouped_gemm_kernel<0> (gate_up + SwiGLU)", "achieved": ach,
                              "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                              "peak_source": f"{peaks['source']} cuBLAS bf16 burst (the kernel multiplies in kind::f16)",
                              "frac_of_nominal_nvfp4_peak": ach / NVFP4_DENSE_PEAK_TFLOPS,
                              "traffic": NCU_TRAFFIC_GEMM1_T8192["bytes"], "traffic_unit": "bytes per launch",
                              "traffic_source": NCU_TRAFFIC_GEMM1_T8192,
                              "algorithmic_bytes": int(256 * (1048576 + 131072 + 4096) + T * 2048 * 2 + T * 8 * 512 * 2)}
        result["stages_ms"] = {k: round(v, 4) for k, v in stage_ms.items()}
        # the same step with the shared expert's GEMMs on a side stream next to top-k / permutation / gather
        for _ in range(3):
            blk.prefill(x_dev, banks, out=out_dev, overlap=True)
        result["ms_per_step_shared_on_side_stream"] = round(
            time_events(lambda: blk.prefill(x_dev, banks, out=out_dev, overlap=True), args.steps, torch), 4)
        result["stages_tflops"] = {"gemm1": round(ach, 1),
                                   "gemm2": round(flops2 / (stage_ms["gemm2_down"] * 1e-3) / 1e12, 1),
                                   "routed_total": round((flops1 + flops2) / ((stage_ms["gemm1_gate_up_swiglu"] +
                                                                                stage_ms["gemm2_down"]) * 1e-3) / 1e12, 1)}
        if not args.no_sweep:
            # the other points of the prefill curve (same layer, fresh seeded tokens); T=65536 is the one-GPU
            # baseline of the expert-parallel workload
            for t_, st_ in ((1024, max(args.steps, 5)), (32768, 5), (65536, 3)):
                result[f"prefill_T{t_}"] = prefill_point(torch, ops, synth, blk, banks, t_, peaks, st_, seed=100 + t_)
        del d, banks, blk
        torch.cuda.empty_cache()
        if not args.no_decode:
            result["decode"] = decode_microbench(torch, peaks, args.decode_layers, args.decode_reps)
        if not args.no_cache:
            result["cache"] = cache_bench(torch)
        if not args.no_cpu:
            result["cpu_baseline"] = cpu_baseline(CPU_TOKENS, os.cpu_count() or 1)
    if rank == 0:
        print(json.dumps(result))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--no-decode", action="store_true", help="skip the decode micro-benchmark block")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-cache", action="store_true", help="skip the slot-cache offload workload")
    ap.add_argument("--no-sweep", action="store_true", help="skip the T=1024/32768/65536 prefill points")
    ap.add_argument("--no-balanced", action="store_true", help="N>1: skip the balanced-placement figure")
    ap.add_argument("--only-decode", action="store_true", help="run only the decode micro-benchmark (profiling aid)")
    ap.add_argument("--decode-layers", type=int, default=40, help="distinct layer banks in the decode stack")
    ap.add_argument("--decode-reps", type=int, default=20)
    ap.add_argument("--decode-m", default="1,2,4,8", help="token counts of the decode micro-benchmark (with --only-decode)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
