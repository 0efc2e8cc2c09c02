"""Multi-rank host logic on CPU (gloo, world size 2): batch x head sharding without a collective,
and the ring sequence partition (K/V rotation, global offsets, log-sum-exp merge).  The CUDA
kernels are replaced by the float64 oracle as the per-shard stand-in; what is under test is the
partitioning, offset and merge logic of jaxmodules_b200/sharding.py."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jaxmodules_b200 import masks as M
from jaxmodules_b200 import sharding as S
from oracle import attention_oracle as ao


def test_shard_ranges_cover_everything_once():
    for units in (1, 7, 8, 64, 65):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = S.shard_range(units, r, world)
                seen += list(range(lo, hi))
            assert seen == list(range(units))
    # a kv head never splits, ranges follow the flattened (b, hk) order
    slices = [S.shard_units(3, 4, r, 5) for r in range(5)]
    flat = [(b, h) for sl in slices for (b, h0, h1) in sl for h in range(h0, h1)]
    assert flat == [(b, h) for b in range(3) for h in range(4)]
    assert S.ring_schedule(2, 4) == [2, 1, 0, 3]


def _terms_mask(terms, B, H, nq, nk):
    q = np.arange(nq)[:, None] + terms.q_offset
    k = np.arange(nk)[None, :] + terms.k_offset
    m = np.ones((nq, nk), dtype=bool)
    if terms.causal:
        m &= k <= q
    if terms.band is not None:
        m &= (k >= q - terms.band[0]) & (k <= q + terms.band[1])
    return np.broadcast_to(m, (B, H, nq, nk))


def _oracle_attend(Q, K, V, terms):
    out = ao.dense_attention(Q.numpy(), K.numpy(), V.numpy(), _terms_mask(terms, Q.shape[0], Q.shape[2], Q.shape[1], K.shape[1]))
    return torch.from_numpy(out["O"]), torch.from_numpy(out["lse"])


def _oracle_merge(O, lse, O2, lse2):
    la, lb = lse.numpy(), lse2.numpy()
    mx = np.maximum(la, lb)
    safe = np.where(np.isfinite(mx), mx, 0.0)
    ea, eb = np.exp(la - safe), np.exp(lb - safe)
    tot = ea + eb
    with np.errstate(divide="ignore", invalid="ignore"):
        l = np.where(tot > 0, safe + np.log(tot), -np.inf)
        wa = np.where(tot > 0, ea / tot, 0.0)
        wb = np.where(tot > 0, eb / tot, 0.0)
    w = lambda x: torch.from_numpy(np.transpose(x, (0, 2, 1))[..., None])   # [B,H,N] -> [B,N,H,1]
    return w(wa) * O + w(wb) * O2, torch.from_numpy(l)


def _oracle_backward(Q, K, V, O, lse, dO, terms):
    """Gradients of one (query chunk, key chunk) pair from the GLOBAL lse and output of the queries."""
    B, nq, Hq, d = Q.shape
    nk, Hkv = K.shape[1], K.shape[2]
    G = Hq // Hkv
    m = torch.from_numpy(np.ascontiguousarray(_terms_mask(terms, B, Hq, nq, nk)))
    Kr, Vr = K.repeat_interleave(G, dim=2), V.repeat_interleave(G, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", Q, Kr) / math.sqrt(d)
    safe_lse = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    P = torch.where(m & torch.isfinite(lse)[..., None], torch.exp(s - safe_lse[..., None]), torch.zeros_like(s))
    dP = torch.einsum("bqhd,bkhd->bhqk", dO, Vr)
    delta = (dO * O).sum(-1).permute(0, 2, 1)
    dS = P * (dP - delta[..., None])
    dQ = torch.einsum("bhqk,bkhd->bqhd", dS, Kr) / math.sqrt(d)
    dK = (torch.einsum("bhqk,bqhd->bkhd", dS, Q) / math.sqrt(d)).reshape(B, nk, Hkv, G, d).sum(3)
    dV = torch.einsum("bhqk,bqhd->bkhd", P, dO).reshape(B, nk, Hkv, G, d).sum(3)
    return dQ, dK, dV


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)           # same data on every rank
        B, L, Hq, Hkv, d = 2, 64, 4, 2, 16
        Q = torch.from_numpy(rng.standard_normal((B, L, Hq, d)))
        K = torch.from_numpy(rng.standard_normal((B, L, Hkv, d)))
        V = torch.from_numpy(rng.standard_normal((B, L, Hkv, d)))

        # --- batch x head shards: no collective in the data path; gathered only for the check
        head_mask = lambda b, h, q, k: (q >= k) | ((h + b) % 2 == 0)
        oracle_call = lambda q, k, v, **kw: torch.from_numpy(ao.masked_attention_dense(q.numpy(), k.numpy(), v.numpy(), **kw)["O"])
        mine = S.sharded_attention(Q, K, V, rank=rank, world=world, attend=oracle_call, mask_fn=head_mask)
        gathered = [None] * world
        dist.all_gather_object(gathered, [(sl, o.numpy()) for sl, o in mine])
        full = np.zeros((B, L, Hq, d))
        for part in gathered:
            for (b, h0, h1), o in part:
                full[b:b + 1, :, h0:h1] = o
        want = ao.masked_attention_dense(Q.numpy(), K.numpy(), V.numpy(), mask_fn=head_mask)["O"]
        ok_shard = np.abs(full - want).max() < 1e-10

        # --- ring sequence partition, causal and banded, contiguous and zig-zag token layouts
        n = L // world
        ok_ring = ok_bwd = True
        dO = torch.from_numpy(np.random.default_rng(1).standard_normal((B, L, Hq, d)))
        for make_layout in (S.contiguous_layout, S.zigzag_layout):
            layout = make_layout(n)
            idx = torch.cat([torch.arange(g0, g0 + m) for g0, m in layout(rank, world)])   # global ids of the local tokens
            for terms in (M.MaskTerms(causal=True), M.MaskTerms(band=(20, 5)), M.MaskTerms(causal=True, band=(17, 1 << 20))):
                O, lse = S.ring_attention_forward(Q[:, idx], K[:, idx], V[:, idx], rank=rank, world=world, terms=terms,
                                                  attend=_oracle_attend, merge=_oracle_merge, layout=layout)
                ref = ao.dense_attention(Q.numpy(), K.numpy(), V.numpy(), _terms_mask(terms, B, Hq, L, L), dO.numpy())
                ok_ring &= np.abs(O.numpy() - ref["O"][:, idx]).max() < 1e-10
                ok_ring &= np.abs(lse.numpy() - ref["lse"][:, :, idx]).max() < 1e-10
                # backward round the same ring: dK / dV accumulators travel with their tokens and come home
                grads = S.ring_attention_backward(Q[:, idx], K[:, idx], V[:, idx], O, lse, dO[:, idx], rank=rank, world=world,
                                                  terms=terms, backward=_oracle_backward, layout=layout)
                for got, name in zip(grads, ("dQ", "dK", "dV")):
                    ok_bwd &= np.abs(got.numpy() - ref[name][:, idx]).max() < 1e-5     # float32 accumulators
        results[rank] = (bool(ok_shard), bool(ok_ring), bool(ok_bwd))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_gloo(world):
    # four ranks: the receive buffers of the ring (two pairs used in turn) and the accumulators that travel one step
    # behind their tokens are reused, which two ranks never do
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {r: (True, True, True) for r in range(world)}


# ---- failure detection on the host (CPU ranks, nothing faults): a neighbour with a chunk of the wrong size, and a
# ---- neighbour that never enters the call.  Either way the ring must raise RingTransferError within its deadline.

def _failing_worker(rank, world, port, results, scenario):
    from datetime import timedelta
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    rng = np.random.default_rng(rank)
    B, Hq, Hkv, d = 1, 2, 2, 8
    n = 32 if not (scenario == "wrong_size" and rank == 1) else 24      # rank 1 holds a shorter chunk
    Q, K, V = (torch.from_numpy(rng.standard_normal((B, n, h, d))) for h in (Hq, Hkv, Hkv))
    t0 = time.monotonic()
    outcome = "completed"
    if scenario in ("absent_peer", "absent_peer_backward") and rank == 1:
        time.sleep(6.0)                                                  # never posts its send
        outcome = "absent"
    elif scenario == "absent_peer_backward":
        # the backward posts its accumulators a step behind the tokens: its deadline must still end the very first wait
        O = torch.zeros((B, n, Hq, d), dtype=torch.float64)
        lse = torch.zeros((B, Hq, n), dtype=torch.float64)
        try:
            S.ring_attention_backward(Q, K, V, O, lse, torch.ones_like(O), rank=rank, world=world, terms=M.MaskTerms(causal=True),
                                      backward=_oracle_backward, timeout_s=3.0)
        except S.RingTransferError as e:
            outcome = "RingTransferError: " + str(e)[:60]
    else:
        try:
            S.ring_attention_forward(Q, K, V, rank=rank, world=world, terms=M.MaskTerms(causal=True), attend=_oracle_attend,
                                     merge=_oracle_merge, timeout_s=3.0)
        except S.RingTransferError as e:
            outcome = "RingTransferError: " + str(e)[:60]
    results[rank] = (outcome, time.monotonic() - t0)
    os._exit(0)      # a transfer may still be pending: leave without the collective teardown


@pytest.mark.parametrize("scenario", ["wrong_size", "absent_peer", "absent_peer_backward"])
def test_ring_reports_a_failed_neighbour(scenario):
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    results = mgr.dict()
    ctx = mp.spawn(_failing_worker, args=(world, port, results, scenario), nprocs=world, join=False)
    for p in ctx.processes:
        p.join(60)
        assert not p.is_alive(), "a rank hung instead of reporting the failure"
    res = dict(results)
    assert res[0][0].startswith("RingTransferError") and res[0][1] < 15.0, res
    if scenario == "wrong_size":
        assert res[1][0].startswith("RingTransferError") and "shape" in res[0][0] + res[1][0], res
