"""Host-side multi-rank logic on CPU: the unit partition, the ring schedule, and a world-size-2 gloo
run of the ring loop with the oracle standing in for the CUDA kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagattention_b200 import ring, sharding
from oracle.attention import attention_forward


def test_unit_ranges_cover_everything_once():
    for units in (1, 7, 8, 32, 256):
        for world in (1, 2, 3, 4, 8):
            got = []
            for r in range(world):
                lo, hi = sharding.unit_range(units, r, world)
                assert hi - lo in (units // world, units // world + 1)
                got.extend(range(lo, hi))
            assert got == list(range(units))


def test_shard_pieces_match_units():
    q = torch.arange(4 * 8 * 2 * 2, dtype=torch.float32).reshape(4, 8, 2, 2)
    k = torch.arange(4 * 2 * 2 * 2, dtype=torch.float32).reshape(4, 2, 2, 2)
    seen_q, seen_k = 0, 0
    for r in range(3):
        for qp, kp, vp, dop in sharding.shard(q, k, k, r, 3, q):
            assert qp.shape[1] == kp.shape[1] * 4 and torch.equal(qp, dop)
            seen_q += qp.numel()
            seen_k += kp.numel()
    assert seen_q == q.numel() and seen_k == k.numel()


def test_ring_plan_is_balanced_and_complete():
    for world in (1, 2, 4, 8):
        seen = set()
        for rank in range(world):
            cost = 0
            lo, hi = ring.zigzag_chunks(rank, world)
            for step in range(world):
                src = (rank - step) % world
                slo, shi = ring.zigzag_chunks(src, world)
                for q_half, kv_halves, causal in ring.plan_step(rank, src):
                    qs = {"lo": [lo], "hi": [hi], "both": [lo, hi]}[q_half]
                    ks = [slo] if kv_halves == "lo" else [slo, shi]
                    for a in qs:
                        for c in ks:
                            if causal and c > a:
                                continue  # masked part of a bottom-right aligned causal call
                            assert c <= a and (causal or c < a)
                            seen.add((a, c))
                            cost += 1 if c < a else 0.5
            if rank == 0:
                ref_cost = cost
            assert cost == ref_cost
        assert seen == {(a, c) for a in range(2 * world) for c in range(a + 1)}


def _torch_merge(o_acc, lse_acc, acc_row0, o_part, lse_part, part_row0, rows, first):
    oa = o_acc[:, :, acc_row0:acc_row0 + rows]
    la = lse_acc[:, :, acc_row0:acc_row0 + rows]
    ob = o_part[:, :, part_row0:part_row0 + rows]
    lb = lse_part[:, :, part_row0:part_row0 + rows]
    if first:
        oa.copy_(ob)
        la.copy_(lb)
        return
    new = torch.logaddexp(la, lb)
    wa = torch.exp(la - new).nan_to_num(0.0).unsqueeze(-1)
    wb = torch.exp(lb - new).nan_to_num(0.0).unsqueeze(-1)
    oa.copy_(oa * wa + ob * wb)
    la.copy_(new)


def _oracle_partial(q, k, v, causal, sm_scale):
    o, lse, _ = attention_forward(q, k, v, causal, sm_scale=sm_scale, upcast=True, return_log_normalizer=True)
    return o.float(), lse


def _worker(rank, world, port, q, k, v, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ql, kl, vl = (ring.zigzag_shard(t, rank, world) for t in (q, k, v))
        o, lse = ring.ring_attention_forward(ql, kl, vl, partial_fn=_oracle_partial, merge_fn=_torch_merge)
        out[rank] = (o, lse)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ring_loop_world2_gloo(world):
    torch.manual_seed(0)
    B, Hq, Hk, S, D = 1, 4, 2, 64 * world // 2, 16
    q = torch.randn(B, Hq, S, D)
    k = torch.randn(B, Hk, S, D)
    v = torch.randn(B, Hk, S, D)
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), q, k, v, out), nprocs=world, join=True)
    o = ring.zigzag_unshard([out[r][0] for r in range(world)])
    lse = ring.zigzag_unshard([out[r][1] for r in range(world)])
    o_ref, lse_ref, _ = attention_forward(q, k, v, True, upcast=True, return_log_normalizer=True)
    torch.testing.assert_close(o, o_ref, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lse, lse_ref, atol=1e-5, rtol=1e-5)
