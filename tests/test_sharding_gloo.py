"""The N > 1 path on CPU: two gloo ranks shard the units of the hot path, compute their
shard (with the oracle standing in for the GPU kernels, since this box has none), gather, and
must reproduce the unsharded result exactly -- there is no collective on the forward path, so
sharded == unsharded bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O

from torch_paras import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1234)          # same inputs on every rank
        if case == "attn_batch":
            q, k, v = (torch.randn(4, 8, 24, 32, generator=g), torch.randn(4, 2, 24, 32, generator=g),
                       torch.randn(4, 2, 24, 32, generator=g))
        else:                                             # fewer batches than ranks: split kv heads
            q, k, v = (torch.randn(1, 8, 24, 32, generator=g), torch.randn(1, 4, 24, 32, generator=g),
                       torch.randn(1, 4, 24, 32, generator=g))
        qs, ks, vs, (kind, lo, hi) = sharding.attention_shard(q, k, v, rank, world)
        local = O.sdpa(qs, ks, vs, is_causal=True, enable_gqa=True)
        if kind == "batch":
            sizes = [b - a for a, b in (sharding.shard_bounds(q.shape[0], r, world) for r in range(world))]
            full = sharding.gather_shards(local, sizes, dim=0)
        else:
            grp = q.shape[1] // k.shape[1]
            sizes = [(b - a) * grp for a, b in (sharding.shard_bounds(k.shape[1], r, world) for r in range(world))]
            full = sharding.gather_shards(local, sizes, dim=1)
        want = O.sdpa(q, k, v, is_causal=True, enable_gqa=True)
        assert torch.equal(full, want), f"rank {rank}: gathered attention differs"

        x = torch.randn(37, 64, generator=g)              # 37 rows: uneven split
        w = torch.randn(64, generator=g)
        xs, (a, b) = sharding.rows_shard(x, rank, world)
        y_local, _ = O.rms_norm_fused(xs, w, 1e-6)
        sizes = [hi_ - lo_ for lo_, hi_ in (sharding.shard_bounds(37, r, world) for r in range(world))]
        y = sharding.gather_shards(y_local, sizes, dim=0)
        assert torch.equal(y, O.rms_norm_fused(x, w, 1e-6)[0])
        gate = torch.randn(37, 64, generator=g)
        z = sharding.gather_shards(O.swiglu_fused(gate[a:b], xs), sizes, dim=0)
        assert torch.equal(z, O.swiglu_fused(gate, x))
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["attn_batch", "attn_heads"])
def test_two_rank_sharding_matches_unsharded(case, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_bounds_cover_everything_once():
    for n in (0, 1, 7, 8, 64, 1000):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def test_attention_shard_keeps_gqa_groups_together():
    q, k, v = torch.zeros(1, 16, 4, 8), torch.zeros(1, 4, 4, 8), torch.zeros(1, 4, 4, 8)
    for rank in range(4):
        qs, ks, vs, (kind, lo, hi) = sharding.attention_shard(q, k, v, rank, 4)
        assert kind == "kv_head" and qs.shape[1] == 4 and ks.shape[1] == 1 and (lo, hi) == (rank, rank + 1)
    q8 = torch.zeros(8, 16, 4, 8)
    qs, ks, vs, (kind, lo, hi) = sharding.attention_shard(q8, torch.zeros(8, 4, 4, 8), torch.zeros(8, 4, 4, 8), 3, 8)
    assert kind == "batch" and (lo, hi) == (3, 4) and qs.shape[0] == 1


def _leaver(rank, world, port, mode, out_dir):
    """Step 0: both ranks gather.  Then rank 1 leaves between steps, with nothing in flight.  Rank 0
    must find that out on the host ("announce") or through the group's timeout ("timeout"), and
    raise instead of waiting forever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    store = dist.distributed_c10d._get_default_store()
    x = torch.full((3, 4), float(rank))
    got = sharding.gather_shards_checked(store, rank, 0, x, [3, 3])
    assert torch.equal(got[:3], torch.zeros(3, 4)) and torch.equal(got[3:], torch.ones(3, 4))
    store.set(f"done0/{rank}", "1")
    if rank == 1:
        store.wait(["done0/0"])   # rank 0 has its step-0 result too: nothing is in flight any more
        open(os.path.join(out_dir, "left"), "w").write("left")
        os._exit(0)           # gone without a word
    try:
        if mode == "announce":
            sharding.gather_shards_checked(store, rank, 1, x, [3, 3], wait_s=1.0)
        else:
            sharding.gather_shards(x, [3, 3])     # straight into the collective: the timeout ends it
    except RuntimeError as e:
        open(os.path.join(out_dir, "raised"), "w").write(str(e))
    os._exit(0)               # (destroy_process_group would wait for the dead peer)


@pytest.mark.parametrize("mode", ["announce", "timeout"])
def test_a_rank_that_leaves_is_noticed_on_the_host(mode, tmp_path):
    ctx = mp.spawn(_leaver, args=(2, _free_port(), mode, str(tmp_path)), nprocs=2, join=False)
    import time
    deadline = time.monotonic() + 90
    while not ctx.join(timeout=5):          # join() returns as each process ends; wait for both
        assert time.monotonic() < deadline, "a rank is still waiting for the one that left"
    assert (tmp_path / "left").exists()
    msg = (tmp_path / "raised").read_text()
    if mode == "announce":
        assert "rank(s) [1] did not reach step 1" in msg
    else:
        assert msg      # gloo's own error: the peer closed the connection or the wait timed out
