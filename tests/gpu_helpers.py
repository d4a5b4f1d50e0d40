"""Runs the CUDA engine through its C ABI (ctypes, raw device pointers) on a numpy test case."""
import numpy as np
import torch

from compactwarprnntloss_b200 import capi


def run_engine(case, dtype=torch.float32, fused=True, reduce=None, average_frames=False, grad_costs=None,
               costs_only=False, want_grad=True, mean_denominator=0, device="cuda:0", max_u=None, keep=False):
    """Returns dict(costs, loss, grad, status, + device tensors when keep=True)."""
    dev = torch.device(device)
    x = torch.as_tensor(case["x"]).to(dtype).to(dev).contiguous()
    lx = torch.as_tensor(case["lx"], dtype=torch.int32).to(dev)
    ly = torch.as_tensor(case["ly"], dtype=torch.int32).to(dev)
    y = torch.as_tensor(case["y"], dtype=torch.int32).to(dev).contiguous()
    flags = 0
    if fused:
        flags |= capi.FUSED_LOG_SOFTMAX
    if costs_only:
        flags |= capi.COSTS_ONLY
    if reduce == "mean":
        flags |= capi.REDUCE_MEAN
    if reduce == "sum":
        flags |= capi.REDUCE_SUM
    if average_frames:
        flags |= capi.AVERAGE_FRAMES
    p = capi.make_problem(x, lx, y, case["blank"], flags, mean_denominator, max_u=max_u)
    ct = capi.cost_dtype(dtype)
    ws = capi.alloc_workspace(p, dev)
    costs = torch.full((p.B,), float("nan"), dtype=ct, device=dev)
    loss = torch.full((), float("nan"), dtype=ct, device=dev)
    capi.forward(p, x, lx, ly, y if y.numel() else None, ws, costs, loss)
    out = dict(costs=costs.double().cpu().numpy(), loss=float(loss.double().cpu()))
    out["status"] = capi.read_status(ws)
    if want_grad and not costs_only:
        gx = torch.full_like(x, float("nan"))
        gc, stride = None, 0
        if grad_costs is not None:
            gc = torch.as_tensor(np.atleast_1d(grad_costs)).to(ct).to(dev)
            stride = 0 if gc.numel() == 1 else 1
        capi.backward(p, x, lx, ly, y if y.numel() else None, ws, gc, stride, gx)
        out["grad"] = gx.double().cpu().numpy()
    if keep:
        out.update(p=p, x=x, lx=lx, ly=ly, y=y, ws=ws)
    torch.cuda.synchronize(dev)
    return out
