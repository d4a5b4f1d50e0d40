"""`GraphedStep`: one training step of the loss (costs, loss, gradient) captured once as a CUDA graph and replayed.

For fixed-shape buckets - a training loop that pads or packs its batches to a few (rows, sequences, label width)
shapes - the whole pipelined step (K0, the gathers, the wavefronts on their side streams, the gradient kernels, every
event) becomes one graph launch, and the workspace and outputs of a bucket are allocated once and reused. The
sequence lengths and labels live on the device, and the kernels work out the lattice geometry and the sequence groups
there, so a graph captured for one batch serves any batch with the same number of rows and sequences and a label
width within the bucket's.

The reference has no counterpart: it allocates five tensors and synchronises with the host six times in every call
(cwarp_cuda_rnnt_kernel.cu:395-404, cwarp_cuda_gather_kernel.cu:85-87), which rules a graph out.
"""
from typing import Optional, Tuple

import torch

from . import capi

__all__ = ["GraphedStep"]


class GraphedStep:
    """Static buffers + captured graph for one shape bucket.

    n_rows, V, B, max_u   the bucket: rows of x, vocabulary, sequences, width of the padded label matrix
    dtype                 element type of x and of the gradient
    flags                 capi flag bits (FUSED_LOG_SOFTMAX, REDUCE_MEAN / REDUCE_SUM, AVERAGE_FRAMES)
    groups                sequence groups of the pipelined step (0 = the library's choice)

    `step(x, lx, ly, y)` copies the inputs into the bucket's buffers on the current stream, replays the graph and
    returns (loss, costs, grad_x): views of the bucket's output buffers, valid until the next `step`.
    """

    def __init__(self, n_rows: int, V: int, B: int, max_u: int, dtype: torch.dtype = torch.float32,
                 device: Optional[torch.device] = None, blank: int = 0,
                 flags: int = capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN, groups: int = 0, mean_denominator: int = 0):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        dev = self.device
        self.x = torch.zeros(n_rows, V, dtype=dtype, device=dev)
        self.lx = torch.ones(B, dtype=torch.int32, device=dev)
        self.ly = torch.zeros(B, dtype=torch.int32, device=dev)
        self.y = torch.zeros(B, max(max_u, 1), dtype=torch.int32, device=dev)
        self.p = capi.Problem(n_rows, V, B, self.y.size(1), max_u, blank, capi.dtype_code(dtype), flags,
                              mean_denominator)
        ct = capi.cost_dtype(dtype)
        self.workspace = capi.alloc_workspace(self.p, dev)
        self.costs = torch.zeros(B, dtype=ct, device=dev)
        self.loss = torch.zeros((), dtype=ct, device=dev)
        self.grad = torch.zeros_like(self.x)
        self.pipe = capi.Pipe(dev)
        self._groups = groups
        self._stream = torch.cuda.Stream(dev)
        # first use outside capture (module load, shared-memory opt-in); the placeholder lengths do not match n_rows,
        # which the kernels report in the status word and otherwise ignore
        with torch.cuda.stream(self._stream):
            self._launch()
            self._stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self._stream):
                self._launch()
        self._stream.synchronize()

    def _launch(self) -> None:
        capi.loss_grad(self.p, self.x, self.lx, self.ly, self.y, self.workspace, self.costs, self.loss, None, 0,
                       self.grad, pipe=self.pipe, groups=self._groups)

    def step(self, x: torch.Tensor, lx: torch.Tensor, ly: torch.Tensor,
             y: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        assert x.shape == self.x.shape and x.dtype == self.x.dtype, "x does not fit this bucket"
        assert lx.numel() == self.lx.numel() and ly.numel() == self.ly.numel()
        assert y.dim() == 2 and y.size(0) == self.y.size(0) and y.size(1) <= self.y.size(1)
        self.x.copy_(x, non_blocking=True)
        self.lx.copy_(lx, non_blocking=True)
        self.ly.copy_(ly, non_blocking=True)
        self.y[:, :y.size(1)].copy_(y, non_blocking=True)
        self.graph.replay()
        return self.loss, self.costs, self.grad

    def status(self):
        """Device status words of the last step (synchronises): [bits, first bad sequence, rows, 0]."""
        return capi.read_status(self.workspace)
