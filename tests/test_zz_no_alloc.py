"""ss_projection_static: the projection for callers that may not allocate device memory
(engines that own all of HBM through their own pools, loops where cudaMalloc/cudaFree are off
limits).  Its scratch is a fixed array inside the library, shared by every call, so the test
runs it twice in a row -- a large problem, then a smaller one that leaves stale bytes behind in
the array -- and demands the same bits as ss_projection with caller-provided scratch."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def run_both(backend, oracle, m, k, n, mode, seed):
    lib = backend.library()
    qweight, scales = oracle.make_weight(n, k, mode, seed=seed)
    bias = (0.1 * torch.randn(n, generator=torch.Generator().manual_seed(seed))).float()
    x = oracle.make_activation(m, k, seed=seed + 1).to(DEV)
    lifted = oracle.slide_weight(qweight, mode)
    valid, pk = oracle.lifted_k(k, mode)
    packed_np, raw = oracle.pack(lifted, pk)
    packed = torch.from_numpy(packed_np).to(DEV)
    meta = torch.from_numpy(oracle.meta_to_b200(raw, pk).view(np.int32)).to(DEV)
    sw, b = torch.from_numpy(scales).to(DEV), bias.to(DEV)
    pm, pn = -(-m // 32) * 32, packed.shape[0]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    q = torch.empty((pm, pk), dtype=torch.int8, device=DEV)
    sa = torch.empty(pm, dtype=torch.float32, device=DEV)
    expect = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = lib.ss_projection(ptr(x), x.stride(0), m, k, mode, ptr(packed), ptr(meta), ptr(sw), ptr(b), None, 0,
                           n, pn, ptr(q), ptr(sa), ptr(expect), n, stream)
    assert rc == 0, lib.ss_last_error().decode()

    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = lib.ss_projection_static(ptr(x), x.stride(0), m, k, mode, ptr(packed), ptr(meta), ptr(sw), ptr(b),
                                  n, pn, ptr(got), n, stream)
    assert rc == 0, lib.ss_last_error().decode()
    torch.cuda.synchronize()
    # From the second call on nothing may be allocated: neither through torch's allocator nor
    # behind it (the driver's free-memory figure must not move either).
    again = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    torch_before, (free_before, _) = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()
    rc = lib.ss_projection_static(ptr(x), x.stride(0), m, k, mode, ptr(packed), ptr(meta), ptr(sw), ptr(b),
                                  n, pn, ptr(again), n, stream)
    assert rc == 0, lib.ss_last_error().decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == torch_before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(again.view(torch.int16), got.view(torch.int16))
    a = got.view(torch.int16).cpu().numpy()
    e = expect.view(torch.int16).cpu().numpy()
    assert not np.isnan(got.float().cpu().numpy()).any()
    assert np.array_equal(a, e), f"{int((a != e).sum())} of {a.size} outputs differ from ss_projection"


def test_static_scratch_projection_matches_on_two_calls_in_a_row(backend, oracle):
    run_both(backend, oracle, m=700, k=1152, n=640, mode=8, seed=11)     # fills a large part of the array
    run_both(backend, oracle, m=70, k=264, n=96, mode=6, seed=12)        # smaller: stale bytes must not leak
    assert backend.device_status() == 0


def test_static_scratch_rejects_oversized_problem(backend):
    lib = backend.library()
    fake = ctypes.c_void_p(256)
    rc = lib.ss_projection_static(fake, 12288, 4096, 12288, 8, fake, fake, fake, None, 3072, 3072, fake, 3072, None)
    assert rc == backend.SS_E_LIMIT
    message = lib.ss_last_error().decode()
    assert "scratch" in message and "33554432" in message
