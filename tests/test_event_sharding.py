"""Event sharding: partition table, local/global id mapping and the result gather, run as
world_size-2 gloo ranks on CPU with the CPU oracle standing in for the CUDA kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastgraphcompute_b200 import event_sharding as es


def test_partition_is_balanced_and_complete():
    g = torch.Generator().manual_seed(0)
    sizes = torch.randint(50000, 150001, (64,), generator=g)
    rs = torch.zeros(65, dtype=torch.int64)
    rs[1:] = torch.cumsum(sizes, 0)
    for world in (1, 2, 4, 8):
        p = es.partition_events(rs, world)
        assert sorted(e for ev in p.events for e in ev) == list(range(64))
        assert sum(p.points) == int(rs[-1])
        assert max(p.points) <= 1.05 * (int(rs[-1]) / world) + 150000 / world
        assert p.events == es.partition_events(rs, world).events   # deterministic


def test_partition_edge_cases():
    p = es.partition_events([0, 0, 5, 5, 9], 3)
    assert sorted(e for ev in p.events for e in ev) == [0, 1, 2, 3] and sum(p.points) == 9
    p = es.partition_events([0, 7], 4)
    assert p.points.count(7) == 1 and sum(p.points) == 7
    with pytest.raises(ValueError):
        es.partition_events([0, 5, 3], 2)
    with pytest.raises(ValueError):
        es.partition_events([0, 5], 0)


def test_shard_rows():
    rows, local = es.shard_rows([0, 3, 3, 7, 9], [0, 2])
    assert rows.tolist() == [0, 1, 2, 3, 4, 5, 6] and local.tolist() == [0, 3, 7]
    rows, local = es.shard_rows([0, 3, 3, 7, 9], [])
    assert rows.numel() == 0 and local.tolist() == [0]


def test_chunk_events():
    rs = [0, 10, 10, 40, 45, 100]
    assert es.chunk_events([0, 1, 2, 3, 4], rs, 1) == [[0, 1, 2, 3, 4]]
    c = es.chunk_events([0, 2, 4], rs, 2)
    assert sorted(e for g in c for e in g) == [0, 2, 4] and len(c) == 2
    assert es.chunk_events([], rs, 3) == [[], [], []]
    assert es.chunk_events([1], rs, 2) == [[1], []]          # an empty event lands in the first group


def _cpu_knn(K, coords, row_splits, direction=None, torch_compatible_indices=False):
    from oracle import oracle
    idx, d = oracle.binned_select_knn(K, coords.numpy(), row_splits.numpy(),
                                      direction=None if direction is None else direction.numpy(),
                                      torch_compatible_indices=torch_compatible_indices)
    return torch.from_numpy(idx), torch.from_numpy(d)


def _cpu_replace(idx, table):
    from oracle import oracle
    return torch.from_numpy(oracle.index_replacer(idx.numpy(), table.numpy()))


def _join_all(procs, limit):
    """Join the workers; whoever is still alive after the limit is terminated (then killed)
    before anything is asserted, so that a stuck rank never outlives the test."""
    try:
        for p in procs:
            p.join(limit)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
    assert [p.exitcode for p in procs] == [0] * len(procs)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fail_rank, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        rs = torch.tensor([0, 300, 300, 520, 900, 1000])
        coords = torch.rand((1000, 3), generator=g)
        if fail_rank is None:
            idx, dsq = es.sharded_binned_select_knn(9, coords, rs, knn_fn=_cpu_knn, replace_fn=_cpu_replace)
            ref_idx, ref_d = _cpu_knn(9, coords, rs)
            import sys
            sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__))))
            import parity
            parity.assert_knn_parity(idx.numpy(), dsq.numpy(), ref_idx.numpy(), ref_d.numpy())
            rows, lidx, _ = es.sharded_binned_select_knn(9, coords, rs, gather=False, knn_fn=_cpu_knn,
                                                         replace_fn=_cpu_replace)
            assert torch.equal(lidx[:, 0], rows)
            # the same in two groups per rank (rows of group 1 travel while group 2 is searched)
            idx2, dsq2 = es.sharded_binned_select_knn(9, coords, rs, n_chunks=2, knn_fn=_cpu_knn,
                                                      replace_fn=_cpu_replace)
            assert idx2.dtype == torch.int64
            parity.assert_knn_parity(idx2.numpy(), dsq2.numpy(), ref_idx.numpy(), ref_d.numpy())
            # the point-to-point exchange for rows on every rank (the default is the collective one)
            idx3, dsq3 = es.sharded_binned_select_knn(9, coords, rs, n_chunks=2, knn_fn=_cpu_knn,
                                                      replace_fn=_cpu_replace, exchange="p2p")
            assert idx3.dtype == torch.int64
            parity.assert_knn_parity(idx3.numpy(), dsq3.numpy(), ref_idx.numpy(), ref_d.numpy())
            # and gathered on rank 1 only
            ridx, rdsq = es.sharded_binned_select_knn(9, coords, rs, gather="root", root=1, knn_fn=_cpu_knn,
                                                      replace_fn=_cpu_replace)
            if rank == 1:
                parity.assert_knn_parity(ridx.numpy(), rdsq.numpy(), ref_idx.numpy(), ref_d.numpy())
            else:
                assert ridx is None and rdsq is None
            out[rank] = "ok"
        else:
            # a rank whose shard disagrees with the partition table must be detected on the host
            part = es.partition_events(rs, world)
            rows, idx, dsq = es.local_binned_select_knn(9, coords, rs, part.events[rank], knn_fn=_cpu_knn,
                                                        replace_fn=_cpu_replace)
            if rank == fail_rank:
                rows, idx, dsq = rows[:-1], idx[:-1], dsq[:-1]
            try:
                es.gather_rows(rows, [idx, dsq], 1000, part.points, row_splits=rs, part=part)
                out[rank] = "no error"
            except RuntimeError as e:
                out[rank] = "raised: " + str(e)[:40]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [None, 1])
def test_two_rank_gloo(fail_rank):
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, fail_rank, out)) for r in range(world)]
    for p in procs:
        p.start()
    _join_all(procs, 120)
    if fail_rank is None:
        assert dict(out) == {0: "ok", 1: "ok"}
    else:
        assert out[fail_rank].startswith("raised")


def _grad_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.ReLU(), torch.nn.Linear(7, 2))
        frozen = torch.nn.Parameter(torch.zeros(3))           # never used: no gradient
        g = torch.Generator().manual_seed(3)
        x = torch.randn((90, 5), generator=g)
        rs = torch.tensor([0, 20, 50, 50, 90])
        part = es.partition_events(rs, world)
        rows, _ = es.shard_rows(rs, part.events[rank])
        (model(x[rows]) ** 2).sum().backward()
        es.allreduce_gradients(list(model.parameters()) + [frozen])
        ref = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.ReLU(), torch.nn.Linear(7, 2))
        ref.load_state_dict(model.state_dict())
        (ref(x) ** 2).sum().backward()
        ok = all(torch.allclose(a.grad, b.grad, rtol=1e-5, atol=1e-6)
                 for a, b in zip(model.parameters(), ref.parameters()))
        out[rank] = "ok" if ok and bool((frozen.grad == 0).all()) else "mismatch"
    finally:
        dist.destroy_process_group()


def test_allreduce_gradients_two_rank_gloo():
    """Data-parallel step over event shards: summed parameter gradients == whole-batch gradients."""
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_grad_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    _join_all(procs, 120)
    assert dict(out) == {0: "ok", 1: "ok"}
