"""World-size-2 gloo tests (CPU) of the data-parallel plumbing: bucketing of the flat gradient buffer, the SUM
all-reduce giving every rank the same averaged gradient, and host-side failure detection (a rank that never joins
the collective makes the others fail with an error after a short timeout instead of hanging)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cgpt_b200 import dp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=30):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _worker_allreduce(rank, world, port, out):
    _init(rank, world, port)
    torch.manual_seed(100 + rank)
    flat = torch.randn(10_007, dtype=torch.float32) * dp.gradient_scale(1024.0, world)
    mine = flat.clone()
    buckets = dp.make_buckets(flat, 4096 * 4)           # 3 buckets, last one ragged
    assert len(buckets) == 3 and sum(b.numel() for b in buckets) == flat.numel()
    assert buckets[1].data_ptr() == flat.data_ptr() + 4096 * 4, "buckets must alias the flat buffer"
    for w in dp.allreduce_buckets(buckets, async_op=True):
        w.wait()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    want = sum(gathered)
    ok = torch.allclose(flat, want, rtol=0, atol=1e-5)
    others = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(others, flat)
    same = all(torch.equal(others[0], o) for o in others)   # every rank holds identical reduced gradients
    out.put((rank, bool(ok), bool(same)))
    dist.destroy_process_group()


def test_bucketed_allreduce_world2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_allreduce, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok and same for _, ok, same in results)


def _worker_failure(rank, world, port, out):
    _init(rank, world, port, timeout_s=5)
    flat = torch.ones(1024)
    dist.all_reduce(flat)                     # one healthy step
    if rank == 1:
        out.put((rank, "left"))
        out.close(); out.join_thread()        # flush the queue's feeder thread before the hard exit
        os._exit(0)                           # the rank dies between steps, nothing in flight
    try:
        dist.all_reduce(flat)                 # the survivor's next collective must end with an error
        out.put((rank, "no error"))
    except Exception as exc:                  # noqa: BLE001 - any backend error is the expected outcome
        out.put((rank, "error:" + type(exc).__name__))
    out.close(); out.join_thread()
    os._exit(0)


def test_peer_loss_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_failure, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results[1] == "left"
    assert results[0].startswith("error:"), results


def test_bucket_helpers_validate():
    with pytest.raises(ValueError):
        dp.make_buckets(torch.zeros(4, 4), 64)
    with pytest.raises(ValueError):
        dp.gradient_scale(1024.0, 0)
    assert dp.gradient_scale(1024.0, 8) == 128.0
    assert [b.numel() for b in dp.make_buckets(torch.zeros(10, dtype=torch.float16), 8)] == [4, 4, 2]


def test_final_gradient_prefix_follows_backward_order():
    """ModelStorage.final_gradient_elements: after k backward steps exactly the tensors those steps finish lie below
    the mark, in the flat buffer's order (final norm, blocks from last to first, embedding-side tensors last)."""
    from cgpt_b200 import model as M
    for tied in (True, False):
        st = M.ModelStorage(M.preset("tiny", vocabulary_size=64), torch.float16, seed=0, tied=tied, device="cpu")
        L = st.options.num_layers
        marks = [st.final_gradient_elements(k) for k in range(L + 3)]
        assert marks[0] == 0 and marks[-1] == st.flat_gradients.numel() and marks == sorted(marks)
        assert marks[1] >= st.final_norm.numel() and marks[1] <= st.gradient_offsets[f"layers.{L - 1}.down_proj"]
        for k in range(1, L + 1):          # after step k (block L-k) every tensor of blocks >= L-k lies below the mark
            for li in range(L - k, L):
                for name, t in st.layers[li].items():
                    assert st.gradient_offsets[f"layers.{li}.{name}"] + t.numel() <= marks[k + 1]
            for li in range(0, L - k):     # ... and no tensor of an unfinished block does
                for name in st.layers[li]:
                    assert st.gradient_offsets[f"layers.{li}.{name}"] >= marks[k + 1]
        assert st.gradient_offsets["token_embedding"] >= marks[L + 1]     # the embedding step is the last one


def _bucket_reducer_worker(rank, world, port, out):
    import torch.distributed as dist
    from cgpt_b200 import dp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        flat = torch.arange(1000, dtype=torch.float32) * (rank + 1)
        buckets = dp.make_buckets(flat, 4 * 300)               # 300, 300, 300, 100 elements
        red = dp.BucketReducer(buckets, dist.group.WORLD)
        started = [red.advance(n) for n in (0, 299, 300, 650, 899, 900)]
        red.finish()
        want = torch.arange(1000, dtype=torch.float32) * sum(r + 1 for r in range(world))
        out.put((rank, started, bool(torch.equal(flat, want)), red.started))
        out.close(); out.join_thread()
    finally:
        dist.destroy_process_group()


def test_bucket_reducer_starts_only_complete_buckets():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_bucket_reducer_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, started, equal, left in results:
        assert started == [0, 0, 1, 1, 0, 1], started      # a bucket goes out only when its last element is final
        assert equal and left == 0
