"""GPU tests of the compact joint producer (cwrnnt_joint_forward / cwrnnt_joint_backward) against the numpy oracle:
act(enc[n,t] + pred[n,u]) written as compact rows, and its two reductions back onto the padded encoder / predictor
tensors. Tolerances: float32/float64 results match the double oracle to rounding of the type; half types to one ulp of
the storage type (the sums run in float32)."""
import ctypes

import numpy as np
import pytest
import torch

from compactwarprnntloss_b200 import capi

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _case(seed, B, Tr, Ur, H, pad_t=0, pad_u=0):
    rng = np.random.default_rng(seed)
    lx = rng.integers(Tr[0], Tr[1] + 1, size=B).astype(np.int32)
    ly = rng.integers(Ur[0], Ur[1] + 1, size=B).astype(np.int32)
    t_max, u_max1 = int(lx.max()) + pad_t, int(ly.max()) + 1 + pad_u
    enc = rng.standard_normal((B, t_max, H))
    pred = rng.standard_normal((B, u_max1, H))
    n_rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    return lx, ly, enc, pred, n_rows


EPS = {torch.float32: 2e-6, torch.float64: 1e-12, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}


@pytest.mark.parametrize("activation", ["none", "relu", "tanh"])
@pytest.mark.parametrize("dtype,H", [(torch.float32, 64), (torch.float32, 37), (torch.float16, 640),
                                     (torch.bfloat16, 96), (torch.bfloat16, 50), (torch.float64, 18)])
def test_forward_and_backward_against_oracle(oracle, activation, dtype, H):
    lx, ly, enc, pred, n_rows = _case(H, 5, (1, 30), (0, 12), H, pad_t=2, pad_u=1)
    e = torch.as_tensor(enc).to(dtype).to(DEV)
    q = torch.as_tensor(pred).to(dtype).to(DEV)
    lxd, lyd = torch.as_tensor(lx).to(DEV), torch.as_tensor(ly).to(DEV)
    e64, q64 = e.double().cpu().numpy(), q.double().cpu().numpy()  # the exactly-representable inputs
    out = capi.joint_forward(e, q, lxd, lyd, n_rows, activation)
    want = oracle.joint_compact(e64, q64, lx, ly, activation)
    assert out.shape == want.shape
    eps = EPS[dtype]
    np.testing.assert_allclose(out.double().cpu().numpy(), want, rtol=eps, atol=eps)

    rng = np.random.default_rng(1)
    g = torch.as_tensor(rng.standard_normal(want.shape)).to(dtype).to(DEV)
    genc, gpred = capi.joint_backward(e, q, lxd, lyd, g, activation)
    wenc, wpred = oracle.joint_compact_backward(e64, q64, lx, ly, g.double().cpu().numpy(), activation)
    scale = max(np.abs(wenc).max(), np.abs(wpred).max(), 1.0)
    # a sum of up to 31 products, rounded once to the storage type
    np.testing.assert_allclose(genc.double().cpu().numpy(), wenc, rtol=4 * eps, atol=4 * eps * scale)
    np.testing.assert_allclose(gpred.double().cpu().numpy(), wpred, rtol=4 * eps, atol=4 * eps * scale)
    # the padding of both gradients is zero-filled
    for n in range(len(lx)):
        assert not genc[n, lx[n]:].any() and not gpred[n, ly[n] + 1:].any()


def test_autograd_joint_linear_loss_chain(oracle):
    """enc/pred -> compact_joint -> linear -> fused transducer loss, gradients back to enc and pred: against the same
    chain in double on the CPU (oracle joint, numpy matmul, oracle loss)."""
    from compactwarprnntloss_b200 import compact_joint, transducer_loss
    lx, ly, enc, pred, n_rows = _case(9, 4, (3, 20), (1, 8), 32)
    V = 24
    rng = np.random.default_rng(2)
    W = rng.standard_normal((V, 32)) * 0.3
    y = rng.integers(1, V, size=(4, int(ly.max()))).astype(np.int32)
    e = torch.as_tensor(enc, dtype=torch.float32, device=DEV).requires_grad_(True)
    q = torch.as_tensor(pred, dtype=torch.float32, device=DEV).requires_grad_(True)
    Wt = torch.as_tensor(W, dtype=torch.float32, device=DEV)
    lxd, lyd, yd = torch.as_tensor(lx).to(DEV), torch.as_tensor(ly).to(DEV), torch.as_tensor(y).to(DEV)
    h = compact_joint(e, q, lxd, lyd, "tanh")
    loss = transducer_loss(h @ Wt.t(), lxd, yd, lyd, 0, "mean", fused_log_softmax=True)
    loss.backward()

    e64, q64 = e.detach().double().cpu().numpy(), q.detach().double().cpu().numpy()
    W64 = Wt.double().cpu().numpy()
    h64 = oracle.joint_compact(e64, q64, lx, ly, "tanh")
    costs, dlogits = oracle.fused(h64 @ W64.T, lx, ly, y, 0, weights=np.full(4, 0.25))
    wenc, wpred = oracle.joint_compact_backward(e64, q64, lx, ly, dlogits @ W64, "tanh")
    assert abs(float(loss.detach()) - costs.mean()) <= 1e-5 * abs(costs.mean())
    np.testing.assert_allclose(e.grad.double().cpu().numpy(), wenc, atol=2e-5)
    np.testing.assert_allclose(q.grad.double().cpu().numpy(), wpred, atol=2e-5)


def test_lengths_that_disagree_with_the_row_count_write_nothing():
    lx, ly, enc, pred, n_rows = _case(3, 3, (2, 9), (1, 4), 16)
    e, q = torch.as_tensor(enc, dtype=torch.float32, device=DEV), torch.as_tensor(pred, dtype=torch.float32, device=DEV)
    lxd, lyd = torch.as_tensor(lx).to(DEV), torch.as_tensor(ly).to(DEV)
    g = torch.ones(n_rows + 5, 16, device=DEV)
    genc, gpred = capi.joint_backward(e, q, lxd, lyd, g, "relu")   # 5 rows too many
    assert not genc.any() and not gpred.any()
    out = torch.full((n_rows + 5, 16), 7.0, device=DEV)
    p = capi._joint_problem(e, q, lxd, n_rows + 5)
    scratch = torch.empty(256, dtype=torch.uint8, device=DEV)
    capi.check(capi.lib().cwrnnt_joint_forward(ctypes.byref(p), 1, e.data_ptr(), e.size(1),
                                               q.data_ptr(), q.size(1), lxd.data_ptr(), lyd.data_ptr(),
                                               scratch.data_ptr(), 256, out.data_ptr(), None), "joint")
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    with pytest.raises(capi.CwrnntError):  # an activation code that does not exist
        capi.check(capi.lib().cwrnnt_joint_forward(ctypes.byref(p), 9, e.data_ptr(), e.size(1),
                                                   q.data_ptr(), q.size(1), lxd.data_ptr(), lyd.data_ptr(),
                                                   scratch.data_ptr(), 256, out.data_ptr(), None), "joint")
