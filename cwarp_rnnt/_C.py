"""`cwarp_rnnt._C`: the reference extension module's three functions (cwarp_cuda.cpp:138-153), served by the B200
engine's torch binding."""
from compactwarprnntloss_b200._C import (_cwarp_rnnt_backward, _cwarp_rnnt_forward, _cwarp_rnnt_loss,  # noqa: F401
                                          _rnnt_backward, _rnnt_forward, _rnnt_status)
