"""B200-native RNN-T (transducer) loss for compact-layout inputs.

Sub-modules:
  loss      `transducer_loss` - the reference project's Python entry point (needs the built CUDA extension)
  capi      ctypes view of the C ABI (include/cwarp_rnnt_b200.h)
  sharding  sequence sharding across GPUs and the cost-vector exchange
  synth     seeded synthetic workloads of the benchmark configurations
  joint     `compact_joint` - the joint network's broadcast-add written directly as compact rows
  graphs    `GraphedStep` - a whole training step of the loss as one replayed CUDA graph per shape bucket
  analysis  `analyse` - best alignment, node posteriors and padded alpha / beta from a forward pass
  build     in-tree build of the native parts

Importing the package itself is light and works on a machine without a GPU; `loss` and `capi.lib()` raise if the
native parts are missing - there is no fallback path.
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("transducer_loss", "TransducerLoss", "compact_from_padded"):
        from . import loss
        return getattr(loss, name)
    if name == "GraphedStep":
        from . import graphs
        return graphs.GraphedStep
    if name in ("analyse", "LatticeAnalysis"):
        from . import analysis
        return getattr(analysis, name)
    if name == "compact_joint":
        from . import joint
        return joint.compact_joint
    raise AttributeError(name)
