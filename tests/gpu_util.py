"""Helpers shared by the GPU parity tests: raw C-ABI calls on torch-owned device buffers."""
import ctypes

import numpy as np
import torch


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def check(backend, rc):
    assert rc == 0, backend.library().ss_last_error().decode()


def c_quantize_lift(backend, x, mode):
    """ss_quantize_lift on a BF16 CUDA [m,k] tensor (row stride taken from the tensor)."""
    m, k = x.shape
    valid = -(-k // mode) * (mode // 2 - 1) * 4
    pk, pm = -(-valid // 128) * 128, -(-m // 32) * 32
    q = torch.full((pm, pk), 0x5A, dtype=torch.int8, device=x.device)       # poison
    sa = torch.full((pm,), float("nan"), dtype=torch.float32, device=x.device)
    check(backend, backend.library().ss_quantize_lift(ptr(x), x.stride(0), m, k, mode, ptr(q), ptr(sa), stream()))
    return q, sa


def c_gemm_int32(backend, q, packed, meta, m, n):
    pm, pk = q.shape
    acc = torch.full((m, n), -(2 ** 31) + 7, dtype=torch.int32, device=q.device)  # poison
    check(backend, backend.library().ss_gemm_int32(ptr(q), ptr(packed), ptr(meta), ptr(acc), m, n, pm,
                                                   packed.shape[0], pk, stream()))
    return acc


def c_gemm_run(backend, q, packed, meta, sa, sw, bias, m, n, addend=None):
    pm, pk = q.shape
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=q.device)
    check(backend, backend.library().ss_gemm_run(
        ptr(q), ptr(packed), ptr(meta), ptr(sa), ptr(sw), ptr(bias) if bias is not None and bias.numel() else None,
        ptr(addend), addend.stride(0) if addend is not None else 0, ptr(out), n, m, n, pm,
        packed.shape[0], pk, stream()))
    return out


def prepare_case(oracle, m, k, n, mode, seed=0, with_bias=True):
    """Seeded inputs + every oracle intermediate for one projection."""
    qweight, scales = oracle.make_weight(n, k, mode, seed=seed)
    bias = None
    if with_bias:
        bias = (0.1 * torch.randn(n, generator=torch.Generator().manual_seed(seed + 7))).float().numpy()
    x = oracle.make_activation(m, k, seed=seed + 13)
    expect = oracle.projection(x, qweight, scales, bias, mode)
    _, pk = oracle.lifted_k(k, mode)
    expect.update(x=x, qweight=qweight, scales=scales, bias=bias, pk=pk,
                  meta_b200=oracle.meta_to_b200(expect["raw"], pk))
    return expect


def verify_accumulators(oracle, acc_cpu, q_ref, qweight, mode, m, n, rows=48, cols=160, seed=7):
    """Full-size check of INT32 accumulators [m, n] without redoing the contraction on the CPU:
    row and column checksums in int64 (every output element enters one of each) and an exact
    comparison on a random sample of rows x columns."""
    lifted = torch.from_numpy(oracle.slide_weight(qweight, mode)).to(torch.int64)          # [n, valid]
    valid = lifted.shape[1]
    q64 = torch.from_numpy(q_ref[:m, :valid]).to(torch.int64)
    assert torch.equal(acc_cpu.sum(dim=1, dtype=torch.int64), q64 @ lifted.sum(dim=0))
    assert torch.equal(acc_cpu.sum(dim=0, dtype=torch.int64), lifted @ q64.sum(dim=0))
    gen = torch.Generator().manual_seed(seed)
    r = torch.randperm(m, generator=gen)[:rows]
    c = torch.randperm(n, generator=gen)[:cols]
    assert torch.equal(acc_cpu[r][:, c].to(torch.int64), q64[r] @ lifted[c].T)


class option:
    """Context manager: one tuning switch of the native library set for the duration of a block."""

    def __init__(self, backend, name, value):
        self.backend, self.name, self.value = backend, name, value

    def __enter__(self):
        self.previous = self.backend.set_option(self.name, self.value)
        return self

    def __exit__(self, *exc):
        self.backend.set_option(self.name, self.previous)


def expected_bits(oracle, oracle_c, x, qweight, scales, bias, mode, addend_bits=None):
    """BF16 bit patterns of the complete projection: the oracle's quantise / slide / contraction with
    the C oracle's epilogue (a true fmaf, which settles the double-rounding corner cases)."""
    ref = oracle.projection(x, qweight, scales, bias, mode)
    return oracle_c.epilogue(ref["acc"], ref["sa"], scales, bias, addend_bits)
