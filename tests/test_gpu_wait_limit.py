"""The exit path of the bounded waits, exercised in the safe form: a diagnostic kernel waits on a
barrier that nothing signals, with a limit of a millisecond.  It has to give up, return normally,
leave its bit in the device status word, and the context has to stay usable.  No real kernel is
starved and nothing faults, traps or spins without bound."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_util import bits, prepare_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_wait_runs_out_status_is_reported_then_cleared(sdk, backend, oracle):
    torch.zeros(1, device=DEV)
    assert backend.device_status() == 0
    limit_ns = 1_000_000
    elapsed = backend.micro_wait_limit(limit_ns)
    assert limit_ns <= elapsed < 200 * limit_ns, elapsed              # gave up after the limit, and soon after it
    lib = backend.library()
    status = ctypes.c_int32(0)
    rc = lib.ss_device_status(None, ctypes.byref(status))
    assert rc == backend.SS_E_DEVICE and status.value == 8
    assert b"wait-limit probe" in lib.ss_last_error()
    assert lib.ss_device_status(None, ctypes.byref(status)) == 0 and status.value == 0      # read-and-clear
    # the raising form
    backend.micro_wait_limit(limit_ns)
    with pytest.raises(RuntimeError, match="bounded wait"):
        backend.check_device()
    backend.check_device()
    # the context is intact: a projection afterwards is still bit-exact
    case = prepare_case(oracle, 100, 256, 96, 6, seed=3)
    op = sdk.PackedLinear.prepare(torch.from_numpy(case["qweight"]), torch.from_numpy(case["scales"]),
                                  torch.from_numpy(case["bias"]), 6).to(DEV)
    assert np.array_equal(bits(op(case["x"].to(DEV))), case["out_bits"])
    assert backend.device_status() == 0
    with pytest.raises(ValueError):
        backend.micro_wait_limit(10 ** 12)                            # limits beyond 100 ms are refused


def test_wait_limit_option_round_trip(backend):
    assert backend.get_option("wait_ns") == 2_000_000_000
    previous = backend.set_option("wait_ns", 5_000_000)
    assert previous == 2_000_000_000 and backend.get_option("wait_ns") == 5_000_000
    backend.set_option("wait_ns", previous)
    with pytest.raises(ValueError):
        backend.set_option("no_such_switch", 1)
