"""RMSNorm forward / backward on the device against the checker (oracle/norm.py)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from helpers import rel_l2
from oracle import norm as ora
from rustingbrain_b200 import InvalidConfig
from rustingbrain_b200.norm import RmsNorm

pytestmark = pytest.mark.gpu


def _case(rows, d, seed):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.standard_normal((rows, d)).astype(np.float32) * 1.7, g.standard_normal((rows, d)).astype(np.float32),
            (1.0 + 0.3 * g.standard_normal(d)).astype(np.float32))


@pytest.mark.parametrize("rows,d", [(2, 8), (70, 16), (33, 512), (257, 4096), (1, 8192)])
@pytest.mark.parametrize("precision,tol", [("f32", 1e-5), ("bf16", 2e-2)])
def test_forward_and_backward_match_the_checker(rows, d, precision, tol):
    x, gy, w = _case(rows, d, seed=rows + d)
    dt = torch.float32 if precision == "f32" else torch.bfloat16
    xd, gyd = torch.from_numpy(x).cuda().to(dt), torch.from_numpy(gy).cuda().to(dt)
    xs, gys = xd.float().cpu().numpy(), gyd.float().cpu().numpy()       # what the device sees
    norm = RmsNorm(d, 1e-6)
    norm.weight.copy_(torch.from_numpy(w))
    y = norm.forward(xd)
    gx = norm.backward(xd, gyd)
    gx_o, gw_o = ora.backward(xs, w, gys, 1e-6)
    assert rel_l2(y.float().cpu().numpy(), ora.forward(xs, w, 1e-6)) <= tol
    assert rel_l2(gx.float().cpu().numpy(), gx_o) <= tol
    assert rel_l2(norm.grad.cpu().numpy(), gw_o) <= 1e-5                 # f32 sums of the values the device saw
    norm.backward(xd, gyd)                                               # the gradient accumulates (norm.rs:113-117)
    assert rel_l2(norm.grad.cpu().numpy(), 2 * gw_o) <= 1e-5


def test_a_frozen_weight_collects_no_gradient_and_shapes_are_checked():  # norm.rs:112
    x, gy, w = _case(40, 64, seed=1)
    norm = RmsNorm(64)
    norm.frozen = True
    gx = norm.backward(torch.from_numpy(x).cuda(), torch.from_numpy(gy).cuda())
    assert float(norm.grad.abs().sum()) == 0.0
    assert rel_l2(gx.cpu().numpy(), ora.backward(x, np.ones(64, np.float32), gy, 1e-6)[0]) <= 1e-5
    with pytest.raises(InvalidConfig):
        RmsNorm(12).forward(torch.zeros(3, 12, device="cuda"))           # d_model must be a multiple of 8


def test_the_reference_known_answers_on_the_device():  # norm.rs:149-170 padded to 8 channels
    norm = RmsNorm(8)
    y = norm.forward(torch.full((1, 8), 5.0, device="cuda"))
    assert float((y - 1.0).abs().max()) < 1e-4
    norm.weight.copy_(torch.tensor([2.0, 0.5] * 4))
    y = norm.forward(torch.ones(1, 8, device="cuda"))
    assert float((y[0, 0] - 2.0).abs()) < 1e-4 and float((y[0, 1] - 0.5).abs()) < 1e-4
