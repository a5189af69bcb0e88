"""Prepared plans and resource queries on the GPU: the path the reference's runtime takes for every
`graph*` / `direct2_*` profile (sdacc/w8a8_slidesparse/csrc/graph_projection.cuh:92-125,153-176 and
`library.prepare_selected`, sdacc/diffusion_research/library.py:31-50), and `configure`
(csrc/dualscale_sm80.cu:282-318).  Every output is compared bit for bit with the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

from gpu_util import bits, expected_bits, prepare_case, ptr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make(sdk, case, mode, frontend):
    bias = None if case["bias"] is None else torch.from_numpy(case["bias"])
    return sdk.PackedLinear.prepare(torch.from_numpy(case["qweight"]), torch.from_numpy(case["scales"]), bias, mode,
                                    frontend=frontend).to(DEV)


@pytest.mark.parametrize("frontend", ["graph_native", "graph1_packed16", "direct2_native"])
def test_prepared_plan_through_the_module(sdk, backend, oracle, oracle_c, frontend):
    m, k, n, mode = 300, 1152, 640, 6
    case = prepare_case(oracle, m, k, n, mode, seed=21)
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"])
    op = make(sdk, case, mode, frontend)
    x = case["x"].to(DEV)
    with pytest.raises(RuntimeError, match="configure_for"):
        op(x)                                            # a plan front-end without a plan for these rows
    handle = op.configure_for(m)
    assert isinstance(handle, int) and handle > 0 and op.configure_for(m) == handle

    # owner stream: the plan's resident scratch; twice, the second call re-uses it
    first, second = op(x), op(x)
    # another stream: independent scratch (the module passes torch-allocated buffers)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        foreign = op(x)
    torch.cuda.current_stream().wait_stream(side)
    # 3-D input, flattened by the module
    batched = op(x.reshape(2, m // 2, k))
    torch.cuda.synchronize()
    for y in (first, second, foreign, batched.reshape(m, n)):
        assert np.array_equal(bits(y), expect)

    # inside an outer CUDA-graph capture the plan must not touch its resident scratch
    static_x = x.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = op(static_x)
    static_x.copy_(torch.flip(x, dims=(0,)))
    graph.replay()
    torch.cuda.synchronize()
    flipped = expected_bits(oracle, oracle_c, torch.flip(case["x"], dims=(0,)), case["qweight"], case["scales"], case["bias"], mode)
    assert np.array_equal(bits(captured), flipped)
    after = op(x)                                        # eager again after the capture: still the owner stream
    assert np.array_equal(bits(after), expect)

    # resources: the reference's five values through the operator, eight through the C ABI
    five = torch.ops.sdacc_prepared_projection_sm80.resources(handle)
    assert len(five) == 5 and five[0] == 352 and 0 < five[1] <= 227 * 1024 and 0 < five[2] <= 255 and five[4] == 1
    eight = (ctypes.c_int64 * 8)()
    assert backend.library().ss_plan_resources(handle, eight, 8) == 0
    assert list(eight[:5]) == list(five) and eight[5] in (128, 192, 224, 240, 256) and eight[6] >= 3 and eight[7] == 512

    # an addend cannot go through a plan (the reference's plans have none): the module falls back
    addend = torch.randn(m, n, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    with_addend = op(x, output_addend=addend.to(DEV))
    expect_addend = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"], bits(addend))
    assert np.array_equal(bits(with_addend), expect_addend)

    # .to() replaces the buffers, so the plans over the old ones are released first
    op.to(DEV)
    assert not op._graphs
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    assert backend.library().ss_plan_run(handle, ptr(x), k, None, None, ptr(out), n, None) == backend.SS_E_HANDLE
    with pytest.raises(RuntimeError):
        torch.ops.sdacc_prepared_projection_sm80.run(x, handle, n)
    assert backend.device_status() == 0


def test_plan_c_abi_scratch_rules(sdk, backend, oracle, oracle_c):
    """ss_plan_run: resident scratch on the owning stream, caller scratch demanded elsewhere."""
    m, k, n, mode = 130, 512, 200, 8
    case = prepare_case(oracle, m, k, n, mode, seed=5)
    op = make(sdk, case, mode, "native")
    lib = backend.library()
    x = case["x"].to(DEV)
    handle = ctypes.c_int64()
    assert lib.ss_plan_create(ptr(op.packed), ptr(op.metadata), ptr(op.scales), ptr(op.bias), k, m, n,
                              op.packed.shape[0], mode, ctypes.byref(handle)) == 0
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert lib.ss_plan_run(handle.value, ptr(x), k, None, None, ptr(out), n, ctypes.c_void_p(main.cuda_stream)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(out), case["out_bits"])
    # a second stream without scratch is refused before anything is launched
    rc = lib.ss_plan_run(handle.value, ptr(x), k, None, None, ptr(out), n, ctypes.c_void_p(side.cuda_stream))
    assert rc == backend.SS_E_ARG and b"caller scratch" in lib.ss_last_error()
    pm, pk = -(-m // 32) * 32, case["pk"]
    q = torch.empty((pm, pk), dtype=torch.int8, device=DEV)
    sa = torch.empty(pm, dtype=torch.float32, device=DEV)
    other = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    side.wait_stream(main)
    assert lib.ss_plan_run(handle.value, ptr(x), k, ptr(q), ptr(sa), ptr(other), n, ctypes.c_void_p(side.cuda_stream)) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(other), case["out_bits"])
    assert np.array_equal(q.cpu().numpy(), case["q"]) and np.array_equal(sa.cpu().numpy(), case["sa"])
    # weights are re-read at every run: scales overwritten in place take effect without a new plan
    op.scales.mul_(2.0)
    assert lib.ss_plan_run(handle.value, ptr(x), k, None, None, ptr(out), n, ctypes.c_void_p(main.cuda_stream)) == 0
    torch.cuda.synchronize()
    doubled = oracle_c.epilogue(case["acc"], case["sa"], 2 * case["scales"], case["bias"])
    assert np.array_equal(bits(out), doubled)
    assert lib.ss_plan_release(handle.value) == 0
    assert lib.ss_plan_run(handle.value, ptr(x), k, None, None, ptr(out), n, None) == backend.SS_E_HANDLE
    assert backend.device_status() == 0


def test_configure_reports_the_kernel_resources(sdk, backend, oracle):
    case = prepare_case(oracle, 64, 1152, 4608, 4, seed=2)
    op = make(sdk, case, 4, "auto")
    listed = torch.ops.sdacc_dualscale_sm80.configure(op.packed, 5, False)
    assert len(listed) == 10 and listed[:5] == listed[5:]
    threads, smem, regs, local, ctas = listed[:5]
    assert threads == 352 and 100 * 1024 < smem <= 227 * 1024 and 64 <= regs <= 255 and local == 0 and ctas == 1
    assert op.configure() == {5: listed}
    assert torch.ops.sdacc_dualscale_sm80.configure(op.packed, 14, True) == listed        # SM80 tile ids select nothing
    with pytest.raises((ValueError, RuntimeError)):
        torch.ops.sdacc_dualscale_sm80.configure(op.packed, 9, False)
    lib = backend.library()
    out = (ctypes.c_int64 * 8)()
    # (m, n, pk) -> token tile / pipeline depth the launcher would use
    for m, n, pk in ((4096, 4608, 1152), (1536, 9216, 4096), (256, 3072, 16384), (16384, 12288, 4608)):
        assert lib.ss_gemm_resources(m, n, pk, out, 8) == 0
        assert out[0] == 352 and out[5] in (128, 192, 224, 240, 256) and 3 <= out[6] <= 8 and out[7] == 512
        assert out[1] <= 227 * 1024 and out[3] == 0
    assert lib.ss_gemm_resources(4096, 4608, 1152, out, 8) == 0 and out[5] in (192, 224)    # the weights-resident form
    assert lib.ss_gemm_resources(0, 1, 128, out, 8) == backend.SS_E_ARG
    assert lib.ss_gemm_resources(1, 1, 100, out, 8) == backend.SS_E_ARG
