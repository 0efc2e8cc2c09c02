"""Ring sequence partition on two real GPUs over NCCL (skipped on a single-GPU box)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    import numpy as np
    import torch.distributed as dist
    from jaxmodules_b200 import masks as M, sharding as S
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator().manual_seed(0)
        B, L, H, d = 1, 2048, 4, 128
        Q, K, V = (torch.randn(B, L, H, d, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
        n = L // world
        terms = M.MaskTerms(causal=True)
        full, full_lse = S.cuda_attend(Q, K, V, terms)
        dO = torch.randn(B, L, H, d, generator=g).cuda()
        want = S.cuda_backward(Q, K, V, full, full_lse, dO, terms)
        worst = [0.0, 0.0, 0.0]
        for make_layout in (S.contiguous_layout, S.zigzag_layout):
            layout = make_layout(n)
            idx = torch.cat([torch.arange(g0, g0 + m) for g0, m in layout(rank, world)]).cuda()   # global ids of the local tokens
            loc = lambda t: t[:, idx].contiguous()
            O, lse = S.ring_attention_forward(loc(Q), loc(K), loc(V), rank=rank, world=world, terms=terms, layout=layout)
            got = S.ring_attention_backward(loc(Q), loc(K), loc(V), O, lse, loc(dO), rank=rank, world=world, terms=terms,
                                            layout=layout)
            torch.cuda.synchronize()
            worst[0] = max(worst[0], float((O - full[:, idx]).abs().max()))
            worst[1] = max(worst[1], float((lse - full_lse[:, :, idx]).abs().max()))
            worst[2] = max(worst[2], max(float(((a.float() - b[:, idx].float()).abs() / b[:, idx].float().abs().clamp(min=1.0)).max())
                                         for a, b in zip(got, want)))
        results[rank] = tuple(worst)
    finally:
        dist.destroy_process_group()


def test_ring_forward_and_backward_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    for r in range(2):
        assert results[r][0] < 2e-3 and results[r][1] < 1e-4 and results[r][2] < 3e-2, dict(results)
