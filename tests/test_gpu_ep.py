"""Expert-parallel prefill on 2 GPUs (NCCL): bit-identical to the single-GPU grouped GEMM path."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
TOKENS = 300


def _worker(rank, world, port, ret, group=None):
    import torch.distributed as dist

    from qwen36_moe_16gb_b200 import ep, ops, synth

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if group:
        os.environ["B200MOE_EP_GROUP"] = str(group)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        shape = synth.Shape(hidden=1024, intermediate=512, num_experts=16, top_k=4, shared_intermediate=256)
        layer = synth.make_layer(5, TOKENS * world, shape, zipf_alpha=1.1)
        d = {k: v.cuda() for k, v in layer.items()}
        logits = synth.router_logits(d["x"], d["router_w"], d["logit_bias"])
        w, ids = ops.fused_topk_softmax(logits, shape.top_k, True)
        ids[3, 1] = -1
        banks = {r: d[r] for r in synth.ROLES}
        want = ops.prefill_experts(d["x"], banks, w, ids, check_status=True)
        epr = shape.num_experts // world
        local = {r: d[r][rank * epr:(rank + 1) * epr].contiguous() for r in synth.ROLES}
        sl = slice(rank * TOKENS, (rank + 1) * TOKENS)
        out, stats = ep.ep_prefill_step(
            dist, d["x"][sl].contiguous(), w[sl].contiguous(), ids[sl].contiguous(), shape.num_experts,
            expert_fn=lambda xr, wr, idr: ops.prefill_route_rows(xr, local, wr, idr),
            combine_fn=lambda ic3, tid: ops.combine_routes(ic3, tid, shape.num_experts))
        torch.cuda.synchronize()
        ok_a2a = bool(torch.equal(out.view(torch.int16), want[sl].view(torch.int16)))
        # combine fused into the GEMM epilogue (stores into the home GPU's buffer), twice in a row
        peer = ep.PeerCombine(dist, TOKENS, shape.top_k, shape.hidden, d["x"].device)
        ok_peer = True
        for _ in range(2):
            out2, status = ep.ep_prefill_step_peer(dist, peer, d["x"][sl].contiguous(), w[sl].contiguous(),
                                                   ids[sl].contiguous(), shape.num_experts, local)
            torch.cuda.synchronize()
            ok_peer = ok_peer and int(status[0]) == 0 and bool(torch.equal(out2.view(torch.int16), want[sl].view(torch.int16)))
        # experts dealt round-robin to the ranks instead of in contiguous blocks
        owner = (torch.arange(shape.num_experts, dtype=torch.int32) % world).cuda()
        local_idx = (torch.arange(shape.num_experts, dtype=torch.int32) // world).cuda()
        dealt = {r: d[r][rank::world].contiguous() for r in synth.ROLES}
        out3, status3 = ep.ep_prefill_step_peer(dist, peer, d["x"][sl].contiguous(), w[sl].contiguous(),
                                                ids[sl].contiguous(), shape.num_experts, dealt, placement=(owner, local_idx))
        torch.cuda.synchronize()
        ok_placed = int(status3[0]) == 0 and bool(torch.equal(out3.view(torch.int16), want[sl].view(torch.int16)))
        # tokens published (and the pulls started) ahead of the routing exchange
        peer.publish_tokens(d["x"][sl].contiguous())
        out4, status4 = ep.ep_prefill_step_peer(dist, peer, d["x"][sl].contiguous(), w[sl].contiguous(),
                                                ids[sl].contiguous(), shape.num_experts, local)
        torch.cuda.synchronize()
        ok_early = int(status4[0]) == 0 and bool(torch.equal(out4.view(torch.int16), want[sl].view(torch.int16)))
        ret[rank] = ok_a2a and ok_peer and ok_placed and ok_early
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_prefill_two_gpus_bit_identical():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_ep_prefill_four_gpus_grouped_sources_bit_identical():
    """Remote sources taken two at a time per grouped-GEMM call (the form used on 8 GPUs)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(4, port, ret, 2), nprocs=4, join=True)
    assert dict(ret) == {r: True for r in range(4)}
