"""Event sharding on real GPUs: two ranks (one process per GPU, NCCL) search their own events
and gather; the result must equal the single-GPU result bit for bit.  Skipped on a box with
fewer than two GPUs (the CPU twin of this test runs on gloo ranks in test_event_sharding.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import fastgraphcompute_b200 as fgc
        from fastgraphcompute_b200 import synthetic, event_sharding as es
        w = synthetic.c3_event_batch(scale=0.05, n_events=12)
        coords, rs = w.coords.to(dev), w.row_splits.to(dev)
        idx, dsq = es.sharded_binned_select_knn(w.K, coords, rs, n_chunks=2)
        ref_idx, ref_dsq = fgc.binned_select_knn(w.K, coords, rs)
        # distances are bit-identical; the neighbour sets too (slot order may differ because a
        # shard builds its own grid)
        same = torch.equal(torch.sort(dsq, 1).values, torch.sort(ref_dsq, 1).values) and \
            torch.equal(torch.sort(idx, 1).values, torch.sort(ref_idx, 1).values)
        # the point-to-point form of the exchange and the gather to one rank give the same rows
        pidx, pdsq = es.sharded_binned_select_knn(w.K, coords, rs, n_chunks=3, exchange="p2p")
        def same_rows(i2, d2):
            return torch.equal(torch.sort(d2, 1).values, torch.sort(ref_dsq, 1).values) and \
                torch.equal(torch.sort(i2, 1).values, torch.sort(ref_idx, 1).values)
        same = same and same_rows(pidx, pdsq)
        ridx, rdsq = es.sharded_binned_select_knn(w.K, coords, rs, gather="root", root=1)
        same = same and ((ridx is None and rdsq is None) if rank != 1 else same_rows(ridx, rdsq))
        part = es.partition_events(w.row_splits, world)
        # data-parallel GravNet step over the event shards: summed parameter gradients must equal
        # the gradients of the whole batch on one GPU
        from fastgraphcompute_b200.gnn_ops import GravNetOp
        gw = synthetic.c4_gravnet(scale=0.02, n_events=6)
        gpart = es.partition_events(gw.row_splits, world)
        torch.manual_seed(0)
        layer = synthetic.init_gravnet_weights(
            GravNetOp(gw.in_channels, gw.out_channels, gw.space_dimensions, gw.propagate_dimensions, gw.k)).to(dev)
        x = gw.x.to(dev)
        rows, local_rs = es.shard_rows(gw.row_splits, gpart.events[rank], device=dev)
        (layer(x.index_select(0, rows), local_rs)[0] ** 2).sum().backward()
        es.allreduce_gradients(layer.parameters())
        mine = [p.grad.clone() for p in layer.parameters()]
        layer.zero_grad(set_to_none=True)
        (layer(x, gw.row_splits.to(dev))[0] ** 2).sum().backward()
        grads_ok = all(float((a - p.grad).abs().max()) <= 2e-4 * (float(p.grad.abs().max()) + 1e-30)
                       for a, p in zip(mine, layer.parameters()) if p.dim() > 1)
        out[rank] = "ok" if same and grads_ok and sum(part.points) == w.n_points else (
            "mismatch knn=%s grads=%s" % (same, grads_ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_knn_matches_single_gpu():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(300)
    finally:
        # a rank that is still alive (stuck in a collective after its peer failed, say) must not
        # outlive the test with a GPU in its hands
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
                    p.join(10)
    assert [p.exitcode for p in procs] == [0] * world
    assert dict(out) == {0: "ok", 1: "ok"}
