"""Host-side multi-rank logic on CPU: head partition and the Ulysses exchanges over gloo, world size 2."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from paroatten_b200 import dist as pd


def test_head_range_covers_all_heads():
    for heads, world in [(40, 8), (40, 3), (12, 4), (5, 8)]:
        got = [h for r in range(world) for h in range(*pd.head_range(heads, r, world))]
        assert got == list(range(heads))
        sizes = [pd.head_range(heads, r, world)[1] - pd.head_range(heads, r, world)[0] for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def test_balanced_partition():
    kept = [100, 10, 10, 10, 90, 20, 20, 60]
    parts = pd.balanced_head_partition(kept, 2)
    assert sorted(h for p in parts for h in p) == list(range(8))
    loads = [sum(kept[h] for h in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 20


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, N, D = 2, 4, 12, 3
        full = torch.arange(B * H * N * D, dtype=torch.float32).reshape(B, H, N, D)
        n_loc = N // world
        mine = full[:, :, rank * n_loc:(rank + 1) * n_loc].contiguous()       # sequence shard
        heads = pd.ulysses_seq_to_heads(mine)                                  # -> head shard, full sequence
        h0, h1 = pd.head_range(H, rank, world)
        ok1 = torch.equal(heads, full[:, h0:h1])
        back = pd.ulysses_heads_to_seq(heads * 2.0)
        ok2 = torch.equal(back, mine * 2.0)
        # a rank-local "attention" on its heads gives the same rows as the unsharded computation
        attn = torch.softmax(heads @ heads.transpose(-1, -2), dim=-1) @ heads
        ref = torch.softmax(full @ full.transpose(-1, -2), dim=-1) @ full
        ok3 = torch.allclose(pd.ulysses_heads_to_seq(attn), ref[:, :, rank * n_loc:(rank + 1) * n_loc])
        q.put((rank, ok1 and ok2 and ok3))
    finally:
        dist.destroy_process_group()


def test_ulysses_roundtrip_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(res) == [(0, True), (1, True)]


def test_ulysses_rejects_uneven_heads():
    class FakeGroup:
        pass
    # world size comes from the process group; without one, torch raises before any exchange
    with pytest.raises(Exception):
        pd.ulysses_seq_to_heads(torch.zeros(1, 3, 4, 2))


def test_host_pipeline_head_groups():
    """The host pipeline's groups cover the heads once, in order, never exceed the requested size and
    shrink towards the end (the last group's kernels and copy back are the un-overlapped tail)."""
    from paroatten_b200.host import head_groups
    for H in (1, 2, 3, 5, 6, 7, 10, 12, 20, 40, 48):
        for g in (None, 1, 2, 3, 4, 5, 8):
            groups = head_groups(H, g)
            sizes = [b - a for a, b in groups]
            assert groups[0][0] == 0 and groups[-1][1] == H and sum(sizes) == H and min(sizes) > 0
            assert all(groups[i][1] == groups[i + 1][0] for i in range(len(groups) - 1))
            if g is not None:
                assert max(sizes) <= g
            tail = sizes[1:]
            assert all(tail[i] >= tail[i + 1] for i in range(len(tail) - 1))
    assert [b - a for a, b in head_groups(40)] == [5, 5, 5, 5, 5, 5, 4, 3, 2, 1]
    assert len(head_groups(5)) >= 3
