"""Two-GPU runs (skipped on a single-GPU box): head partition without a collective, and the optional
Ulysses mode (sequence-sharded activations, NCCL all-to-all before and after the path)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    import paroatten_b200 as pb
    from paroatten_b200 import dist as pd
    from oracle import paro_oracle as po
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, H, D, grid, n_text = 1, 4, 128, (2, 8, 16), 0
        N = grid[0] * grid[1] * grid[2]
        q, k, v, orders = po.make_inputs(B, H, N, D, torch.bfloat16, seed=5)     # same on every rank
        mask = po.make_mask(H, (N + 63) // 64, 0.5, seed=5)
        tabs = pb.rope_tables(grid, D, "wan", device=dev)
        full = pb.paro_attention(q.to(dev), k.to(dev), v.to(dev), torch.tensor(orders), mask.to(dev), grid_fhw=grid,
                                 rope=tabs)
        # (1) head partition: each rank computes its heads only, no exchange
        h0, h1 = pd.head_range(H, rank, world)
        mine = pb.paro_attention(q[:, h0:h1].to(dev), k[:, h0:h1].to(dev), v[:, h0:h1].to(dev),
                                 torch.tensor(orders[h0:h1]), mask[h0:h1].to(dev), grid_fhw=grid, rope=tabs)
        ok_heads = torch.equal(mine, full[:, h0:h1])
        # (2) Ulysses: this rank starts with a slice of the sequence of ALL heads
        n_loc = N // world
        sl = slice(rank * n_loc, (rank + 1) * n_loc)
        qs, ks, vs = (pd.ulysses_seq_to_heads(t[:, :, sl].contiguous().to(dev)) for t in (q, k, v))
        o_heads = pb.paro_attention(qs, ks, vs, torch.tensor(orders[h0:h1]), mask[h0:h1].to(dev), grid_fhw=grid, rope=tabs)
        o_seq = pd.ulysses_heads_to_seq(o_heads)
        ok_ulysses = torch.equal(o_seq, full[:, :, sl])
        pb.check_status(dev)
        q_out.put((rank, bool(ok_heads), bool(ok_ulysses)))
    finally:
        dist.destroy_process_group()


def test_head_partition_and_ulysses_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res == [(0, True, True), (1, True, True)]
