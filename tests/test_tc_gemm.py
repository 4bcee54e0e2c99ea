"""Each tcgen05 grouped-GEMM variant against a torch fp32 product of the same bf16 operands."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from rustingbrain_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 2], ids=["one_sm", "two_sm", "wide"], autouse=True)
def tc_variant(request):
    """Every case runs on the one-SM tiles, on the two-SM (cta_group::2) tiles and on the one-SM 256x256 tiles."""
    _lib.lib().moe_debug_set_tc_pair(request.param)
    yield request.param
    _lib.lib().moe_debug_set_tc_pair(3)   # back to the per-launch choice


def _groups(rows_per_group):
    row0 = np.concatenate([[0], np.cumsum(rows_per_group)]).astype(np.int32)
    assert np.all(row0 % 128 == 0)
    tstart = (row0 // 128).astype(np.int32)
    return torch.from_numpy(row0).cuda(), torch.from_numpy(tstart).cuda(), row0


def _run(variant, a, b, out0, out1, aux, row0, tstart, G, rows, m, n, k, accumulate=0):
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().moe_debug_tc_gemm(variant, a.data_ptr(), b.data_ptr(), out0.data_ptr(),
                                      out1.data_ptr() if out1 is not None else None,
                                      aux.data_ptr() if aux is not None else None, row0.data_ptr(), tstart.data_ptr(),
                                      G, rows, m, n, k, accumulate, flag.data_ptr(),
                                      C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait inside the kernel gave up (code %d)" % int(flag.item())


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _interleave(g, u):
    """[.., F] gate and up -> [.., 2F] in blocks of 32 gate then 32 up."""
    F = g.shape[-1]
    return torch.stack([g.reshape(*g.shape[:-1], F // 32, 32), u.reshape(*u.shape[:-1], F // 32, 32)], dim=-2).reshape(
        *g.shape[:-1], 2 * F)


@pytest.mark.parametrize("rows_per_group,N,K", [([128], 256, 64), ([256, 0, 128], 512, 192), ([384, 128], 320, 2048)])
def test_rows_nt_store(rows_per_group, N, K):
    torch.manual_seed(0)
    row0, tstart, r0 = _groups(rows_per_group)
    G, R = len(rows_per_group), int(r0[-1])
    a = torch.randn(R, K, device="cuda").bfloat16()
    b = (torch.randn(G, N, K, device="cuda") * 0.05).bfloat16()
    out = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    _run(0, a, b, out, None, None, row0, tstart, G, R, 0, N, K)
    ref = torch.cat([a[r0[g]:r0[g + 1]].float() @ b[g].float().T for g in range(G)])
    assert _rel(out, ref) < 1e-2


def test_rows_nt_swiglu():
    torch.manual_seed(1)
    rows_per_group, F, K = [256, 128], 160, 256
    row0, tstart, r0 = _groups(rows_per_group)
    G, R = 2, int(r0[-1])
    a = torch.randn(R, K, device="cuda").bfloat16()
    wg = (torch.randn(G, F, K, device="cuda") * 0.05).bfloat16()
    wu = (torch.randn(G, F, K, device="cuda") * 0.05).bfloat16()
    b = _interleave(wg.transpose(1, 2), wu.transpose(1, 2)).transpose(1, 2).contiguous()  # [G, 2F, K]
    h = torch.zeros(R, F, device="cuda", dtype=torch.bfloat16)
    gu = torch.zeros(R, 2 * F, device="cuda", dtype=torch.bfloat16)
    _run(1, a, b, h, gu, None, row0, tstart, G, R, 0, 2 * F, K)
    g_ref = torch.cat([a[r0[g]:r0[g + 1]].float() @ wg[g].float().T for g in range(G)])
    u_ref = torch.cat([a[r0[g]:r0[g + 1]].float() @ wu[g].float().T for g in range(G)])
    assert _rel(gu, _interleave(g_ref, u_ref)) < 1e-2
    assert _rel(h, torch.nn.functional.silu(g_ref) * u_ref) < 1.5e-2


@pytest.mark.parametrize("rows_per_group,N,K", [([128], 256, 64), ([256, 128], 160, 320)])
def test_rows_nn_store(rows_per_group, N, K):
    torch.manual_seed(2)
    row0, tstart, r0 = _groups(rows_per_group)
    G, R = len(rows_per_group), int(r0[-1])
    a = torch.randn(R, K, device="cuda").bfloat16()
    b = (torch.randn(G, K, N, device="cuda") * 0.05).bfloat16()
    out = torch.zeros(R, N, device="cuda", dtype=torch.bfloat16)
    _run(2, a, b, out, None, None, row0, tstart, G, R, 0, N, K)
    ref = torch.cat([a[r0[g]:r0[g + 1]].float() @ b[g].float() for g in range(G)])
    assert _rel(out, ref) < 1e-2


def test_rows_nn_swiglu_backward():
    torch.manual_seed(3)
    rows_per_group, F, K = [128, 256], 96, 128
    row0, tstart, r0 = _groups(rows_per_group)
    G, R = 2, int(r0[-1])
    dy = torch.randn(R, K, device="cuda").bfloat16()
    wd = (torch.randn(G, K, F, device="cuda") * 0.1).bfloat16()     # [d, F]: dh = dy @ wd
    g = torch.randn(R, F, device="cuda").bfloat16()
    u = torch.randn(R, F, device="cuda").bfloat16()
    gu = _interleave(g, u).contiguous()
    dgu = torch.zeros(R, 2 * F, device="cuda", dtype=torch.bfloat16)
    _run(3, dy, wd, dgu, None, gu, row0, tstart, G, R, 0, F, K)
    dh = torch.cat([dy[r0[i]:r0[i + 1]].float() @ wd[i].float() for i in range(G)])
    s = torch.sigmoid(g.float())
    dg = dh * u.float() * (s * (1 + g.float() * (1 - s)))
    du = dh * (g.float() * s)
    assert _rel(dgu, _interleave(dg, du)) < 1.5e-2


@pytest.mark.parametrize("rows_per_group,M,N", [([128], 128, 256), ([256, 0, 384], 192, 320)])
def test_rows_tn_accumulate(rows_per_group, M, N):
    torch.manual_seed(4)
    row0, tstart, r0 = _groups(rows_per_group)
    G, R = len(rows_per_group), int(r0[-1])
    a = torch.randn(R, M, device="cuda").bfloat16()
    b = torch.randn(R, N, device="cuda").bfloat16()
    out = torch.full((G, M, N), 7.0, device="cuda")
    _run(4, a, b, out, None, None, row0, tstart, G, R, M, N, 0, accumulate=0)
    ref = torch.stack([a[r0[g]:r0[g + 1]].float().T @ b[r0[g]:r0[g + 1]].float() for g in range(G)])
    assert _rel(out, ref) < 1e-3
    assert torch.all(out[1] == 0) if rows_per_group[min(1, G - 1)] == 0 and G > 1 else True
    _run(4, a, b, out, None, None, row0, tstart, G, R, M, N, 0, accumulate=1)
    assert _rel(out, 2 * ref) < 1e-3
