"""Bank slots on the GPU: the kernels read packed / metadata / scales / bias at launch time, so
mode switches and in-place coefficient updates need no new operator, eagerly or under graph replay
(reference callers: sdacc/diffusion_research/banks.py:55-56,121-127, affine.py:59,74)."""
import numpy as np
import pytest
import torch

from gpu_util import bits
from test_banks import make_payloads

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("residency", ["active", "all"])
def test_mode_switching_matches_oracle(sdk, backend, oracle, residency):
    from slidesparse_diffusion_b200 import banks
    k, n, m = 96, 40, 50
    payloads, dense = make_payloads(sdk, oracle, k=k, n=n)
    slot = banks.ResidentBankSlot(payloads, DEV, residency=residency)
    ops = slot.operators(k, n)
    x = oracle.make_activation(m, k, seed=9)
    bias = payloads[4]["bias"].numpy()
    for mode in (6, 4, 8, 4):
        slot.activate(mode)
        y = ops[mode](x.to(DEV))
        qweight, scales = dense[mode]
        assert np.array_equal(bits(y), oracle.projection(x, qweight, scales, bias, mode)["out_bits"]), mode


def test_in_place_coefficients_are_seen_by_a_replayed_graph(sdk, backend, oracle):
    from slidesparse_diffusion_b200 import banks
    k, n, m, mode = 128, 64, 33, 8
    payloads, dense = make_payloads(sdk, oracle, k=k, n=n, modes=(mode,))
    slot = banks.ResidentBankSlot(payloads, DEV, residency="active")
    op = slot.operators(k, n)[mode]
    slot.activate(mode)
    x = oracle.make_activation(m, k, seed=2)
    xd = x.to(DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        op(xd)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = op(xd)
    qweight, scales = dense[mode]
    bias = payloads[mode]["bias"].numpy()
    graph.replay()
    assert np.array_equal(bits(y), oracle.projection(x, qweight, scales, bias, mode)["out_bits"])
    new_scales = (scales * np.float32(1.5)).astype(np.float32)
    new_bias = (bias[::-1] * np.float32(0.25)).copy()
    op.scales.copy_(torch.from_numpy(new_scales))
    op.bias.copy_(torch.from_numpy(new_bias))
    graph.replay()
    assert np.array_equal(bits(y), oracle.projection(x, qweight, new_scales, new_bias, mode)["out_bits"])
