"""World-size-2 gloo rehearsal of the data-parallel plumbing (no GPU): partition of a batch, gather
of per-rank embeddings in rank order, ragged last shard, and a rank that fails before the gather."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from segment_anything_fast_b200.dist import gather_embeddings, gather_ragged, shard_range


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, fail_rank, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        n_items = 5                                           # ragged: rank 0 gets 3, rank 1 gets 2
        a, b = shard_range(n_items, rank, world)
        local = torch.arange(a, b, dtype=torch.float32).view(-1, 1, 1, 1).expand(-1, 2, 3, 3).contiguous()
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the gather")
        counts = [shard_range(n_items, r, world)[1] - shard_range(n_items, r, world)[0] for r in range(world)]
        full = gather_ragged(local, counts)
        ok = full.shape == (n_items, 2, 3, 3) and torch.equal(full[:, 0, 0, 0], torch.arange(n_items, dtype=torch.float32))
        even = gather_embeddings(torch.full((2, 1, 1, 1), float(rank)))
        ok = ok and torch.equal(even.flatten(), torch.tensor([0., 0., 1., 1.]))
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as e:                                    # the surviving rank must see an error, not hang
        q.put((rank, f"error:{type(e).__name__}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(fail_rank, port):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_rank, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "rank did not finish"
    return dict(q.get(timeout=5) for _ in range(2))


def test_two_rank_gather_in_rank_order():
    res = _run(fail_rank=-1, port=29611)
    assert res == {0: "ok", 1: "ok"}


def test_rank_failing_before_gather_surfaces_as_error_on_the_peer():
    res = _run(fail_rank=1, port=29612)
    assert res[1].startswith("error:RuntimeError")
    assert res[0].startswith("error:")          # timeout / connection error, not a hang
