"""World-size-2 CPU (gloo) tests of the data-parallel plumbing, mirroring the reference's
multi-process tests (test/distributed/{common,optimizer,synchronize,data}_distributedtest.jl)."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, q):
    try:
        sys.path.insert(0, os.path.join(ROOT, "lux.jl_b200"))
        os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LOCAL_RANK=str(rank))
        from luxlib_b200 import distributed as D
        D.initialize(D.GlooBackend, timeout_s=60)
        be = D.get_distributed_backend(D.GlooBackend)
        globals()[fn_name](D, be, rank, world)
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the parent
        import traceback
        q.put((rank, "FAIL: " + traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def _spawn(fn_name, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    for rank, res in results:
        assert res == "ok", f"rank {rank}: {res}"


def _primitives(D, be, rank, world):
    # test/distributed/common_distributedtest.jl:36-106: 512-element buffers
    assert D.local_rank(be) == rank and D.total_workers(be) == world
    buf = torch.full((512,), float(rank + 1))
    D.bcast_(be, buf, root=0)
    assert (buf == 1).all()
    buf = torch.full((512,), float(rank + 1))
    D.allreduce_(be, buf, "+")
    assert (buf == sum(range(1, world + 1))).all()
    buf = torch.full((512,), float(rank + 1))
    D.allreduce_(be, buf, D.avg)
    assert torch.allclose(buf, torch.full((512,), sum(range(1, world + 1)) / world))
    col = torch.full((4, 6), float(rank + 1)).T   # column-major (non-contiguous) array
    D.allreduce_(be, col, D.avg)
    assert torch.allclose(col, torch.full((6, 4), sum(range(1, world + 1)) / world))
    buf = torch.full((512,), float(rank + 1))
    D.reduce_(be, buf, "+", root=0)
    if rank == 0:
        assert (buf == sum(range(1, world + 1))).all()
    buf = torch.full((512,), float(rank + 1))
    D.reduce_(be, buf, D.avg, root=0)
    if rank == 0:
        assert torch.allclose(buf, torch.full((512,), sum(range(1, world + 1)) / world))


def _synchronize(D, be, rank, world):
    # test/distributed/synchronize_distributedtest.jl:34-118: nested containers, scalars, symbols
    from collections import namedtuple
    NT = namedtuple("NT", "a b")
    ps = {"w": torch.full((3, 2), float(rank)), "nested": NT(torch.full((4,), float(rank)), (torch.tensor([rank]), "sym")),
          "scalar": float(rank) + 0.5, "count": rank + 7, "flag": rank == 0, "none": None, "empty": ()}
    out = D.synchronize(be, ps, root=0)
    assert (out["w"] == 0).all() and (out["nested"].a == 0).all() and out["nested"].b[0].item() == 0
    assert out["nested"].b[1] == "sym" and out["scalar"] == 0.5 and out["count"] == 7 and out["flag"] is True
    assert out["none"] is None and out["empty"] == ()


def _optimizer(D, be, rank, world):
    # test/distributed/optimizer_distributedtest.jl:27-47: equal gradients on all ranks -> same step as the plain rule
    def sgd(state, p, g):
        return state, p - 0.1 * g
    params = [torch.ones(5), torch.arange(6.0).reshape(2, 3)]
    grads_equal = [torch.full((5,), 2.0), torch.ones(2, 3)]
    for bucketed in (False, True):
        opt = D.DistributedOptimizer(be, sgd, bucketed=bucketed)
        out = opt.apply_all([None, None], params, [g.clone() for g in grads_equal])
        for (st, newp), p, g in zip(out, params, grads_equal):
            assert torch.allclose(newp, p - 0.1 * g)
        # rank-dependent gradients are averaged
        gr = [torch.full((5,), float(rank)), torch.full((2, 3), float(2 * rank))]
        out = opt.apply_all([None, None], params, gr)
        mean_r = sum(range(world)) / world
        assert torch.allclose(out[0][1], params[0] - 0.1 * mean_r)
        assert torch.allclose(out[1][1], params[1] - 0.1 * 2 * mean_r)


def _data(D, be, rank, world):
    # test/distributed/data_distributedtest.jl:35-53: partition sizes and global sum
    data = list(range(1, 11))
    dc = D.DistributedDataContainer(be, data)
    assert len(dc) == 5
    s = torch.tensor([float(sum(dc[i] for i in range(len(dc))))])
    D.allreduce_(be, s, "+")
    assert s.item() == sum(data)


@pytest.mark.parametrize("fn", ["_primitives", "_synchronize", "_optimizer", "_data"])
def test_gloo_world_size_2(fn):
    _spawn(fn, 2)


def test_data_container_partition_sizes_without_processes():
    sys.path.insert(0, os.path.join(ROOT, "lux.jl_b200"))
    from luxlib_b200 import distributed as D
    data = list(range(10))
    sizes = [len(D.DistributedDataContainer(None, data, rank=r, workers=3)) for r in range(3)]
    assert sizes == [4, 4, 2]   # ceil(10/3) = 4 per worker, the last one takes the rest
    assert [len(D.DistributedDataContainer(None, data, rank=r, workers=4)) for r in range(4)] == [3, 3, 3, 1]
    assert len(D.DistributedDataContainer(None, [], rank=0, workers=2)) == 0


def test_fused_optimizer_buckets_follow_dtype_and_size_without_reordering():
    # host logic only: which leaves share one collective + one optimiser launch
    import torch
    from luxlib_b200 import distributed as D
    opt = D.FusedOptimizer(D.GlooBackend, "adam", bucket_bytes=1000)
    params = [torch.zeros(100), torch.zeros(100), torch.zeros(10, dtype=torch.bfloat16), torch.zeros(200), torch.zeros(5)]
    # fp32 leaves: 400 B + 400 B fit, the 800 B leaf starts a new bucket, the 20 B leaf joins it; bf16 apart
    assert opt.buckets(params) == [[0, 1], [3, 4], [2]]
    st = opt.init(params)
    assert st[0][0].shape == params[0].shape and st[0][1] is not None and st[0][2] is None
    assert D.FusedOptimizer(D.GlooBackend, "descent").init(params)[0] == (None, None, None)
    assert D.FusedOptimizer(D.GlooBackend, "momentum", master=True).init(params)[2][2].dtype == torch.float32
    with pytest.raises(ValueError):
        D.FusedOptimizer(D.GlooBackend, "rmsprop")
