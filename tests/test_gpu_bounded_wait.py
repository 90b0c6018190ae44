"""A device-side wait that nothing satisfies runs out after its time limit, reports through the status word and leaves
the context usable (the failure-detection contract of every flag / peer wait in the extension)."""
import time

import pytest
import torch

from lbi_b200 import ops
from lbi_b200.utils.failure import KernelWaitTimeout, check_kernel_status

pytestmark = pytest.mark.gpu


def test_wait_on_a_flag_nobody_sets_times_out_cleanly():
    dev = "cuda"
    mailbox = torch.arange(64, dtype=torch.float32, device=dev)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    check_kernel_status(mailbox)  # clear anything earlier tests left
    ops.ext().set_peer_wait_limit_ms(1000)
    t0 = time.perf_counter()
    out = ops.ext().wait_state(mailbox, flags, 3, 1)  # flag 3 stays 0 < 1
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.9 < waited < 10.0, f"bounded wait took {waited:.2f} s"
    with pytest.raises(KernelWaitTimeout):
        check_kernel_status(mailbox)
    check_kernel_status(mailbox)  # the word was reset by the read
    # the context still works, and a satisfied wait returns the data
    flags[3] = 1
    out = ops.ext().wait_state(mailbox, flags, 3, 1)
    torch.cuda.synchronize()
    assert torch.equal(out, mailbox)
    check_kernel_status(mailbox)
    ops.ext().set_peer_wait_limit_ms(20000)
    a = torch.randn(256, 256, device=dev)
    assert torch.isfinite(a @ a).all()
