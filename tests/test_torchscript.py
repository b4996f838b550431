"""TorchScript compatibility of the drop-in API, after the reference's own tests
(tests/test_binned_select_knn.py:242-311, tests/test_bin_by_coordinates.py:84-109,
tests/test_gnn_ops.py:29-149): modules that call the wrappers can be scripted, traced, saved and
loaded and give the results of the eager call.  Compilation is checked without a GPU; execution
needs one."""
import io
from typing import Optional, Tuple

import pytest
import torch

import fastgraphcompute_b200 as fgc
from fastgraphcompute_b200.extensions.binned_select_knn import binned_select_knn
from fastgraphcompute_b200.extensions.bin_by_coordinates import bin_by_coordinates
from fastgraphcompute_b200.extensions.index_replacer import index_replacer
from fastgraphcompute_b200.gnn_ops import GravNetOp


class BinnedSelectKnnModule(torch.nn.Module):
    def forward(self, K: int, coordinates: torch.Tensor, row_splits: torch.Tensor,
                direction: Optional[torch.Tensor] = None,
                n_bins: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        return binned_select_knn(K, coordinates, row_splits, direction=direction, n_bins=n_bins)


class BinByCoordinatesModule(torch.nn.Module):
    def forward(self, coordinates: torch.Tensor, row_splits: torch.Tensor, bin_width: torch.Tensor,
                nbins: torch.Tensor, return_all: bool
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        return bin_by_coordinates(coordinates, row_splits, bin_width, nbins, return_all)


class IndexReplacerModule(torch.nn.Module):
    def forward(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return index_replacer(a, b)


class SimpleGravNetModel(torch.nn.Module):
    def __init__(self, in_dim: int, prop_dim: int, s: int, k: int):
        super().__init__()
        self.gravnet = GravNetOp(in_channels=in_dim, out_channels=prop_dim, space_dimensions=s,
                                 propagate_dimensions=prop_dim, k=k)

    def forward(self, x: torch.Tensor, row_splits: torch.Tensor) -> torch.Tensor:
        out, idx, dist, space = self.gravnet(x, row_splits)
        return out


def test_everything_compiles_without_a_gpu():
    torch.jit.script(BinnedSelectKnnModule())
    torch.jit.script(BinByCoordinatesModule())
    torch.jit.script(IndexReplacerModule())
    torch.jit.script(SimpleGravNetModel(8, 16, 3, 8))
    torch.jit.script(GravNetOp(8, 16, 3, 16, 8))
    for name in ("knn_forward", "knn_backward", "gravnet_aggregate", "gravnet_aggregate_backward",
                 "index_replacer", "bin_by_coordinates"):
        assert hasattr(torch.ops.fgc_b200, name)


def test_ops_reject_cpu_tensors_through_the_dispatcher():
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        torch.ops.fgc_b200.knn_forward(torch.rand(10, 3), torch.tensor([0, 10]), 4, None, False)


def _roundtrip(scripted):
    buf = io.BytesIO()
    torch.jit.save(scripted, buf)
    buf.seek(0)
    return torch.jit.load(buf)


@pytest.mark.gpu
def test_knn_module_script_save_load():
    dev = "cuda:0"
    K, N, D = 8, 100, 3
    g = torch.Generator().manual_seed(0)
    coords = torch.randn((N, D), generator=g).to(dev)
    rs = torch.tensor([0, 50, N], dtype=torch.int64, device=dev)
    n_bins = torch.tensor(4, dtype=torch.int64, device=dev)
    module = BinnedSelectKnnModule().to(dev)
    scripted = torch.jit.script(module)
    with torch.no_grad():
        i0, d0 = module(K, coords, rs, None, n_bins)
        i1, d1 = scripted(K, coords, rs, None, n_bins)
        i2, d2 = _roundtrip(scripted)(K, coords, rs, None, n_bins)
    assert i0.shape == (N, K) and d0.shape == (N, K)
    assert torch.equal(i0, i1) and torch.equal(d0, d1) and torch.equal(i0, i2) and torch.equal(d0, d2)

    @torch.jit.script
    def wrapper(K: int, coords: torch.Tensor, row_splits: torch.Tensor) -> torch.Tensor:
        idx, dist = binned_select_knn(K, coords, row_splits)
        return torch.cat([idx.float(), dist], dim=1)

    assert wrapper(K, coords, rs).shape == (N, 2 * K)
    # gradients flow through the scripted module as well
    c = coords.clone().requires_grad_(True)
    _, d = scripted(K, c, rs, None, None)
    d.sum().backward()
    c2 = coords.clone().requires_grad_(True)
    _, dd = module(K, c2, rs, None, None)
    dd.sum().backward()
    assert torch.allclose(c.grad, c2.grad, atol=1e-6)


@pytest.mark.gpu
def test_binning_and_index_replacer_modules_script():
    dev = "cuda:0"
    coords = torch.tensor([[0.1, 0.1], [2.5, 2.5], [4.9, 4.9]], device=dev)
    rs = torch.tensor([0, 3], device=dev)
    bw = torch.tensor([0.5], device=dev)
    nb = torch.tensor([10, 10], device=dev)
    m = BinByCoordinatesModule()
    s = torch.jit.script(m)
    for o, t in zip(m(coords, rs, bw, nb, True), _roundtrip(s)(coords, rs, bw, nb, True)):
        assert torch.equal(o, t)
    a = torch.tensor([[3, -1, 0], [2, 1, 7]], device=dev)
    b = torch.tensor([10, 11, 12, 13], device=dev)
    assert torch.equal(torch.jit.script(IndexReplacerModule())(a, b), index_replacer(a, b))


@pytest.mark.gpu
def test_gravnet_model_script_trace_save_load():
    dev = "cuda:0"
    torch.manual_seed(0)
    in_dim, prop_dim, s, k = 8, 16, 3, 8
    model = SimpleGravNetModel(in_dim, prop_dim, s, k).to(dev)
    x = torch.randn(100, in_dim, device=dev)
    rs = torch.tensor([0, 50, 100], dtype=torch.int32, device=dev)
    scripted = torch.jit.script(model)
    traced = torch.jit.trace(model, (x, rs))
    with torch.no_grad():
        ref = model(x, rs)
        assert ref.shape == (100, prop_dim)
        for other in (scripted, _roundtrip(scripted), traced, _roundtrip(traced)):
            assert torch.allclose(ref, other(x, rs), atol=1e-6)
    op = GravNetOp(in_dim, prop_dim, s, prop_dim, k, optimization_arguments={}).to(dev)
    with torch.no_grad():
        a = op(x, rs)[0]
        b = torch.jit.script(op)(x, rs)[0]
    assert torch.allclose(a, b, atol=1e-6)
    # training step through the scripted model
    xs = x.clone().requires_grad_(True)
    (scripted(xs, rs) ** 2).sum().backward()
    xe = x.clone().requires_grad_(True)
    (model(xe, rs) ** 2).sum().backward()
    assert torch.allclose(xs.grad, xe.grad, atol=1e-5)


@pytest.mark.gpu
def test_reference_op_names_in_a_fresh_process():
    """Registering the reference's op names must happen in a process that has not loaded the
    reference's own library (the oracle tests do): run it in a child."""
    import subprocess
    import sys
    import os
    code = '''
import torch, sys
sys.path.insert(0, %r)
import fastgraphcompute_b200 as fgc
from fastgraphcompute_b200 import torch_ops
print(torch_ops.register_reference_op_names())
c = torch.rand(200, 3, device="cuda:0"); rs = torch.tensor([0, 200], device="cuda:0")
i, d = torch.ops.fastgraphcompute_custom_ops.binned_select_knn_autograd(c, rs, 5, None, None, 3, False)
i2, d2 = fgc.binned_select_knn(5, c, rs)
assert torch.equal(i, i2) and torch.equal(d, d2)
g = torch.ops.binned_select_knn_grad.binned_select_knn_grad(torch.ones_like(d), i, d, c)
assert g.shape == c.shape
r = torch.ops.index_replacer.index_replacer(torch.tensor([1, -1, 0], device="cuda:0"), torch.tensor([7, 8], device="cuda:0"))
assert r.tolist() == [8, -1, 7]
b = torch.ops.bin_by_coordinates.bin_by_coordinates(c, rs, None, torch.tensor(4, device="cuda:0"), True, False)
assert int(b[4].sum()) == 200
print("child ok")
''' % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "child ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_torch_compile_fullgraph_of_a_gravnet_layer():
    """torch.compile(fullgraph=True) captures a module that calls the neighbour search and the
    aggregation as ONE graph (the ops have shape inference and autograd registered with the
    dispatcher), and the compiled module gives the eager results, forward and backward.  The
    backend is aot_eager: graph capture, functionalisation and the joint forward/backward graph
    are exercised; code generation for the dense layers is not this library's business."""
    torch.manual_seed(3)
    dev = "cuda:0"
    model = SimpleGravNetModel(8, 16, 3, 8).to(dev)
    x = torch.randn((300, 8), device=dev)
    rs = torch.tensor([0, 120, 300], dtype=torch.int64, device=dev)
    xe = x.clone().requires_grad_(True)
    eager = model(xe, rs)
    (eager ** 2).sum().backward()
    eager_grads = [p.grad.clone() for p in model.parameters()]
    model.zero_grad(set_to_none=True)
    compiled = torch.compile(model, fullgraph=True, backend="aot_eager")
    xc = x.clone().requires_grad_(True)
    out = compiled(xc, rs)
    (out ** 2).sum().backward()
    assert torch.allclose(out, eager, rtol=1e-5, atol=1e-6)
    assert torch.allclose(xc.grad, xe.grad, rtol=1e-4, atol=1e-5)
    for p, g in zip(model.parameters(), eager_grads):
        assert torch.allclose(p.grad, g, rtol=1e-4, atol=1e-5)
