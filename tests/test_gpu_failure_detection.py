"""Failure detection on the device without a fault: every wait inside the kernels is bounded, and a wait that runs
out records a code in the device status word and lets the kernel return.  The self-test entry point makes such a
wait run out on purpose (a barrier nobody arrives at, 50 ms limit); the host must see the code, and the context
must stay usable for the next launch on the same stream."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

import jaxmodules_b200 as jm
from jaxmodules_b200 import _native as nat
from jaxmodules_b200 import attention as A
from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_context_survives():
    lib = nat.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert A.device_status() == 0
    t0 = time.monotonic()
    assert lib.bma_debug_expire_wait(50_000_000, 777, st) == nat.BMA_OK       # 50 ms
    code = C.c_int32()
    assert lib.bma_device_status(st, C.byref(code)) == nat.BMA_ERR_DEVICE_CHECK and code.value == 777
    assert 0.04 < time.monotonic() - t0 < 5.0          # it waited for its limit, and not much longer
    assert lib.bma_device_status(st, C.byref(code)) == nat.BMA_OK and code.value == 0    # reading clears the word

    # the first code wins until it is read
    lib.bma_debug_expire_wait(1_000_000, 11, st)
    lib.bma_debug_expire_wait(1_000_000, 12, st)
    assert A.device_status() == 11 and A.device_status() == 0

    # argument checks: no limit above one second, no zero code
    assert lib.bma_debug_expire_wait(2_000_000_000, 5, st) == nat.BMA_ERR_ARG
    assert lib.bma_debug_expire_wait(1_000_000, 0, st) == nat.BMA_ERR_ARG

    # the same stream and context keep working
    g = np.random.Generator(np.random.PCG64(0))
    Q, K, V = (torch.from_numpy(g.standard_normal((1, 256, 2, 128), dtype=np.float32)).to(torch.bfloat16) for _ in range(3))
    O = jm.masked_attention_via_map(Q.cuda(), K.cuda(), V.cuda(), is_causal=True)
    ref = ao.masked_attention_dense(Q.float().numpy(), K.float().numpy(), V.float().numpy(), is_causal=True)["O"]
    assert np.abs(O.cpu().numpy() - ref).max() <= 2e-2
    assert A.device_status() == 0


def test_status_check_after_every_launch_raises(monkeypatch):
    """BMA_CHECK_STATUS=1 semantics: a non-zero status word turns into an exception at the next checked launch."""
    monkeypatch.setattr(A, "_check_status", True)
    nat.lib().bma_debug_expire_wait(1_000_000, 42, torch.cuda.current_stream().cuda_stream)
    Q = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="device status 42"):
        jm.masked_attention_via_map(Q, Q, Q, is_causal=True)
    assert A.device_status() == 0
