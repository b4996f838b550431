"""Generate the committed golden vectors by running the reference's own CPU ops.

    python oracle/build_ref.py && python tests/golden/make_golden.py

Needs oracle/_ref/binned_knn_ops.so (built from the unmodified reference
sources).  Writes tests/golden/{knn,binning,gravnet,misc,stacked,oc,select,pyg}.npz
(`python make_golden.py stacked` / `oc` / `select` / `pyg` write only that file).  The tests only
read those files; they never need the reference checkout.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import cases  # noqa: E402
from oracle import build_ref, ref_ops  # noqa: E402
from fastgraphcompute_b200 import synthetic  # noqa: E402


def run_knn(c):
    coords = torch.tensor(c["coords"], requires_grad="grad" in c)
    rs = torch.tensor(c["row_splits"], dtype=torch.int64)
    kw = {}
    if "n_bins" in c:
        kw["n_bins"] = torch.tensor(c["n_bins"], dtype=torch.int64)
    if "direction" in c:
        kw["direction"] = torch.tensor(c["direction"], dtype=torch.int64)
    if "max_bin_dims" in c:
        kw["max_bin_dims"] = int(c["max_bin_dims"])
    if c.get("tf_compat"):
        kw["torch_compatible_indices"] = True
    idx, dist = ref_ops.ref_binned_select_knn(int(c["K"]), coords, rs, **kw)
    out = dict(idx=idx.numpy().astype(np.int32), distsq=dist.detach().numpy())
    if "grad" in c:
        # slot-order independent loss: weights apply to the row sorted by distance
        dist.retain_grad()
        sorted_d, _ = torch.sort(dist, dim=1, stable=True)
        (sorted_d * torch.tensor(c["grad"])).sum().backward()
        out["grad_coords"] = coords.grad.numpy()
        out["grad_dist_slots"] = dist.grad.numpy()   # the same weights in the reference's slot order
    return out


STACKED = dict(n=700, row_splits=[0, 300, 700], in_dim=16, prop_dim=8, space_dim=3, k=10, hidden_dim=32,
               output_dim=5, num_gravnet_layers=2)


def make_pyg():
    """row_splits <-> batch conversions recorded from the reference's own functions
    (fastgraphcompute/torch_geometric_interface.py, loaded from its file: the module is plain
    tensor code).  Inputs: the shapes its unit tests use (three events, one event, no points,
    one point per event) and seeded random event sizes with empty events and non-consecutive
    ids."""
    import importlib.util
    path = os.path.join(build_ref.default_reference_root(), "fastgraphcompute", "torch_geometric_interface.py")
    spec = importlib.util.spec_from_file_location("ref_pyg_interface", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    rng = np.random.RandomState(7)
    batches = {
        "three_events": np.array([0, 0, 0, 1, 1, 2, 2, 2]),
        "one_event": np.zeros(4, np.int64),
        "no_points": np.zeros(0, np.int64),
        "one_point_each": np.arange(4),
        "ids_with_gaps": np.repeat(np.array([3, 4, 9, 10, 40]), [5, 1, 7, 2, 3]),
        "random_5000": np.repeat(np.arange(300) * 2, rng.randint(1, 40, size=300)),
    }
    splits = {
        "three_events": np.array([0, 3, 5, 8]),
        "one_event": np.array([0, 4]),
        "no_points": np.array([0, 0]),
        "one_point_each": np.arange(5),
        "with_empty_events": np.array([0, 0, 4, 4, 4, 9, 9]),
        "random_sizes": np.concatenate([[0], np.cumsum(rng.randint(0, 50, size=400))]),
    }
    store = {}
    for name, b in batches.items():
        store["batch_to_rs/%s/in" % name] = b.astype(np.int64)
        store["batch_to_rs/%s/out" % name] = ref.row_splits_from_strict_batch(torch.tensor(b, dtype=torch.int64)).numpy()
    for name, r in splits.items():
        store["rs_to_batch/%s/in" % name] = r.astype(np.int64)
        store["rs_to_batch/%s/out" % name] = ref.strict_batch_from_row_splits(torch.tensor(r, dtype=torch.int64)).numpy()
    np.savez_compressed(os.path.join(HERE, "pyg.npz"), **store)
    print("pyg done:", len(batches), "+", len(splits), "cases")


def make_stacked():
    """The stacked-GravNet model (performance/gravnet_perfm.py:20-96 of the reference) with the
    reference's CPU ops inside every GravNet layer: output and gradients of one step."""
    from fastgraphcompute_b200.gravnet_model import GravNetModel
    torch.set_num_threads(1)
    c = STACKED
    torch.manual_seed(21)
    m = GravNetModel(c["in_dim"], c["prop_dim"], c["space_dim"], c["k"], c["hidden_dim"], c["output_dim"],
                     num_gravnet_layers=c["num_gravnet_layers"], the_op=ref_ops.RefGravNetOp)
    g = torch.Generator().manual_seed(22)
    x = torch.randn((c["n"], c["in_dim"]), generator=g, requires_grad=True)
    rs = torch.tensor(c["row_splits"], dtype=torch.int64)
    out = m(x, rs)
    (out ** 2).sum().backward()
    store = {"in/x": x.detach().numpy(), "out/out": out.detach().numpy(), "out/grad_x": x.grad.numpy()}
    for k, v in c.items():
        store["in/" + k] = np.asarray(v)
    for k, v in m.state_dict().items():
        store["weights/" + k] = v.numpy()
    for k, p in m.named_parameters():
        store["grad/" + k] = p.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "stacked.npz"), **store)
    print("stacked done")


def oc_cases():
    rng = np.random.RandomState(77)
    cases = {}

    def mk(name, sizes, lo, hi, scale=1):
        rs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        asso = rng.randint(lo, hi, size=int(rs[-1])).astype(np.int64)
        asso[asso >= 0] *= scale
        cases[name] = dict(asso=asso, row_splits=rs)

    mk("two_splits", [40, 25], -2, 6)
    mk("empty_split_between", [30, 0, 50], -1, 9)
    mk("large_truth_indices", [60, 60, 10], -3, 12, scale=10 ** 12 + 7)
    mk("many_small_objects", [300], 0, 150)
    mk("one_object_per_split", [20, 20, 20], 5, 6)
    mk("noise_only_split", [25, 40], -4, 0)
    cases["noise_only_split"]["asso"][25:] = rng.randint(0, 4, size=40)
    mk("bigger", [700, 900, 400], -1, 40)
    return cases


def make_oc():
    """oc_helper_matrices of the reference (its CPU ops, extensions/oc_helper_cpu.cpp and
    oc_helper_helper.cpp) on small seeded cases."""
    store = {}
    for name, c in oc_cases().items():
        M, M_not, per = ref_ops.ref_oc_helper_matrices(torch.tensor(c["asso"]), torch.tensor(c["row_splits"]))
        store[name + "/in/asso"] = c["asso"]
        store[name + "/in/row_splits"] = c["row_splits"]
        store[name + "/out/M"] = M.numpy()
        store[name + "/out/M_not"] = M_not.numpy().astype(np.int32)
        store[name + "/out/per_split"] = per.numpy()
    np.savez_compressed(os.path.join(HERE, "oc.npz"), **store)
    print("oc done")


def make_select():
    """The reference's brute-force op select_knn::select_knn (select_knn_cpu.cpp) with and
    without a radius, on small seeded cases."""
    rng = np.random.RandomState(91)
    store = {}
    for name, sizes, d, k, r in (("no_radius", [60, 90], 3, 8, -1.0), ("radius_small", [150], 3, 12, 0.12),
                                 ("radius_mid_d4", [80, 5, 120], 4, 20, 0.35), ("radius_large", [70, 70], 2, 6, 10.0),
                                 ("fewer_points_than_k", [4, 9], 3, 12, 0.5)):
        rs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        c = rng.rand(int(rs[-1]), d).astype(np.float32)
        idx, dist = ref_ops.ref_select_knn(k, torch.tensor(c), torch.tensor(rs), r)
        store[name + "/in/coords"] = c
        store[name + "/in/row_splits"] = rs
        store[name + "/in/K"] = np.asarray(k)
        store[name + "/in/max_radius"] = np.asarray(r)
        store[name + "/out/idx"] = idx.numpy().astype(np.int32)
        store[name + "/out/distsq"] = dist.numpy()
    np.savez_compressed(os.path.join(HERE, "select.npz"), **store)
    print("select done")


def main():
    torch.set_num_threads(1)
    if "select" in sys.argv[1:]:
        make_select()
        return
    if "stacked" in sys.argv[1:]:
        make_stacked()
        return
    if "oc" in sys.argv[1:]:
        make_oc()
        return
    if "pyg" in sys.argv[1:]:
        make_pyg()
        return
    store = {}
    for name, c in cases.knn_cases().items():
        out = run_knn(c)
        for k, v in c.items():
            store[f"{name}/in/{k}"] = np.asarray(v)
        for k, v in out.items():
            store[f"{name}/out/{k}"] = v
        print("knn", name, out["idx"].shape)
    np.savez_compressed(os.path.join(HERE, "knn.npz"), **store)

    store = {}
    for name, c in cases.binning_cases().items():
        kw = {}
        if "bin_width" in c:
            kw["bin_width"] = torch.tensor(c["bin_width"])
        if "n_bins" in c:
            kw["n_bins"] = torch.tensor(c["n_bins"], dtype=torch.int64)
        if c.get("pre_normalized"):
            kw["pre_normalized"] = True
        r = ref_ops.ref_bin_by_coordinates(torch.tensor(c["coords"]),
                                           torch.tensor(c["row_splits"], dtype=torch.int64), **kw)
        for k, v in c.items():
            store[f"{name}/in/{k}"] = np.asarray(v)
        for k, v in zip(("bin_indices", "flat", "n_bins", "bin_width", "n_per_bin"), r):
            store[f"{name}/out/{k}"] = v.numpy()
        print("binning", name)
    # the reference's own fixture (tests/test_bbc_data.npy, detector-like coordinates),
    # binned as its smoke test does (n_bins = 21, one row split)
    fixture = os.path.join(build_ref.default_reference_root(), "tests", "test_bbc_data.npy")
    if os.path.exists(fixture):
        data = np.load(fixture).astype(np.float32)
        r = ref_ops.ref_bin_by_coordinates(torch.tensor(data), torch.tensor([0, data.shape[0]]),
                                           n_bins=torch.tensor(21))
        store["bbc_fixture/in/coords"] = data
        store["bbc_fixture/in/row_splits"] = np.array([0, data.shape[0]])
        store["bbc_fixture/in/n_bins"] = np.array(21)
        for k, v in zip(("bin_indices", "flat", "n_bins", "bin_width", "n_per_bin"), r):
            store[f"bbc_fixture/out/{k}"] = v.numpy()
        print("binning bbc_fixture", data.shape)
    np.savez_compressed(os.path.join(HERE, "binning.npz"), **store)

    store = {}
    for name, c in cases.gravnet_cases().items():
        torch.manual_seed(1)
        m = ref_ops.RefGravNetOp(c["in_channels"], c["out_channels"], c["space"], c["propagate"], c["k"])
        synthetic.init_gravnet_weights(m, seed=3)
        g = torch.Generator().manual_seed(5)
        x = torch.randn((c["n"], c["in_channels"]), generator=g, requires_grad=True)
        rs = torch.tensor(c["row_splits"], dtype=torch.int32)
        out, idx, dsq, space = m(x, rs)
        (out ** 2).sum().backward()
        store[f"{name}/in/x"] = x.detach().numpy()
        store[f"{name}/in/row_splits"] = c["row_splits"]
        for k, v in c.items():
            if k != "row_splits":
                store[f"{name}/in/{k}"] = np.asarray(v)
        for k, v in m.state_dict().items():
            store[f"{name}/weights/{k}"] = v.numpy()
        store[f"{name}/out/out"] = out.detach().numpy()
        store[f"{name}/out/idx"] = idx.numpy().astype(np.int32)
        store[f"{name}/out/distsq"] = dsq.detach().numpy()
        store[f"{name}/out/space"] = space.detach().numpy()
        store[f"{name}/out/grad_x"] = x.grad.numpy()
        for k, p in m.named_parameters():
            store[f"{name}/grad/{k}"] = p.grad.numpy()
        print("gravnet", name)
    np.savez_compressed(os.path.join(HERE, "gravnet.npz"), **store)

    # index_replacer on random data incl. negative and out-of-range entries
    rng = np.random.RandomState(34)
    tbr = rng.randint(-3, 130, size=(40, 7)).astype(np.int64)
    rpl = rng.permutation(280).astype(np.int64)
    rep = ref_ops.ref_index_replacer(torch.tensor(tbr), torch.tensor(rpl)).numpy()
    np.savez_compressed(os.path.join(HERE, "misc.npz"), ir_in=tbr, ir_repl=rpl, ir_out=rep)
    print("misc done")
    make_stacked()
    make_oc()
    make_select()
    make_pyg()


if __name__ == "__main__":
    main()
