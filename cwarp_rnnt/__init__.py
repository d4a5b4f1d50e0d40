"""Drop-in for the reference package name: `import cwarp_rnnt; cwarp_rnnt.transducer_loss(x, lx, y, ly, blank,
reduction)` and `import cwarp_rnnt._C as core` resolve to the B200 engine in compactwarprnntloss_b200."""
from compactwarprnntloss_b200 import __version__  # noqa: F401
from compactwarprnntloss_b200.loss import TransducerLoss, compact_from_padded, transducer_loss  # noqa: F401
