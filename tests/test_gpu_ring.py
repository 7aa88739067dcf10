"""Ring-KV sequence-parallel forward and the partial-result merge kernel on the GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagattention_b200 import flash_attention, ring
from oracle.attention import attention_forward, max_abs_diff

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_merge_kernel_matches_logsumexp_algebra():
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    B, H, L, c, D = 2, 3, 96, 48, 64
    o_acc = torch.randn(B, H, L, D, device=dev, generator=g)
    lse_acc = torch.randn(B, H, L, device=dev, generator=g)
    o_part = torch.randn(B, H, c, D, device=dev, generator=g)
    lse_part = torch.randn(B, H, c, device=dev, generator=g)
    lse_part[0, 0, :5] = float("-inf")        # partial with no visible key
    want_o, want_l = o_acc.clone(), lse_acc.clone()
    new = torch.logaddexp(lse_acc[:, :, c:], lse_part)
    want_o[:, :, c:] = (o_acc[:, :, c:] * torch.exp(lse_acc[:, :, c:] - new).unsqueeze(-1)
                        + o_part * torch.exp(lse_part - new).unsqueeze(-1))
    want_l[:, :, c:] = new
    ring._cuda_merge(o_acc, lse_acc, c, o_part, lse_part, 0, c, False)
    torch.testing.assert_close(o_acc, want_o, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lse_acc, want_l, atol=1e-5, rtol=1e-5)
    ring._cuda_merge(o_acc, lse_acc, 0, o_part, lse_part, 0, c, True)   # first: overwrite
    torch.testing.assert_close(o_acc[:, :, :c][torch.isfinite(lse_part)], o_part[torch.isfinite(lse_part)])
    assert torch.equal(lse_acc[:, :, :c], lse_part)


def _ring_worker(rank, world, port, backend, q, k, v, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank if backend == "nccl" else 0)
    torch.cuda.set_device(dev)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ql, kl, vl = (ring.zigzag_shard(t.to(dev), rank, world) for t in (q, k, v))
        o, lse = ring.ring_attention_forward(ql, kl, vl)
        torch.cuda.synchronize(dev)
        out[rank] = (o.cpu(), lse.cpu())
    finally:
        dist.destroy_process_group()


def _check(world, backend, S):
    g = torch.Generator().manual_seed(world)
    B, Hq, Hk, D = 1, 8, 2, 128
    q, k, v = (torch.randn(B, h, S, D, generator=g).to(torch.bfloat16) for h in (Hq, Hk, Hk))
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ring_worker, args=(world, _free_port(), backend, q, k, v, out), nprocs=world, join=True)
    o = ring.zigzag_unshard([out[r][0] for r in range(world)])
    lse = ring.zigzag_unshard([out[r][1] for r in range(world)])
    o_ref, lse_ref, _ = attention_forward(q.cuda(), k.cuda(), v.cuda(), True, upcast=True, return_log_normalizer=True)
    o_low = attention_forward(q.cuda(), k.cuda(), v.cuda(), True, upcast=False)
    assert max_abs_diff(o.cuda(), o_ref) <= 2 * max_abs_diff(o_low, o_ref) + 1e-5
    assert max_abs_diff(lse.cuda(), lse_ref) <= 1e-4
    single = flash_attention(q.cuda(), k.cuda(), v.cuda(), causal=True)
    assert max_abs_diff(o.cuda(), single) <= 2 ** -6


def test_ring_world1_equals_plain_forward():
    _check(1, "gloo", 2048)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ring_two_gpus_nccl():
    _check(2, "nccl", 4096)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_ring_four_gpus_nccl():
    _check(4, "nccl", 8192)
