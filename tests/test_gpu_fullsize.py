"""Parity at the full sizes of the benchmark configurations, through properties that do not need
the CPU to redo the whole contraction:

  * front-end: compared element for element with the oracle (it is element-wise, cheap on a CPU);
  * INT32 accumulators: (a) exact on a random sample of token rows x channels, (b) row and column
    checksums -- sum_n acc[m,n] == q[m] . (sum_n w_n) and sum_m acc[m,n] == (sum_m q[m]) . w_n in
    int64 -- which every single output element enters, (c) the sliding identity
    lift(q) . slide(w)^T == q . w^T on the same sample, from the un-lifted operands;
  * BF16 output of the complete projection: bit for bit against the C oracle's epilogue applied to
    the accumulators verified in (a)-(c).
"""
import numpy as np
import pytest
import torch

from gpu_util import bits, c_gemm_int32

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# (mode, M, K, N): cfg0; FLUX QKV / fc2 at M=1536; FLUX fc1 at the largest M; SD3.5 image fc1 and
# text fc2; Sigma cross-KV
FULL = [(4, 4096, 1152, 4608), (6, 1536, 3072, 9216), (8, 1536, 12288, 3072), (8, 16384, 3072, 12288),
        (6, 2048, 2432, 9728), (6, 666, 9728, 2432), (8, 600, 1152, 2304)]


@pytest.mark.parametrize("mode,m,k,n", FULL)
def test_full_size_projection(sdk, backend, oracle, oracle_c, mode, m, k, n):
    qweight, scales = oracle.make_weight(n, k, mode, seed=m + n)
    bias = (0.1 * torch.randn(n, generator=torch.Generator().manual_seed(k))).float()
    x = oracle.make_activation(m, k, seed=n + 1)
    op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), bias, mode).to(DEV)
    xd = x.to(DEV)

    # front-end, whole tensor
    q, sa = sdk.quantize_lift(xd, mode)
    q_ref, sa_ref = oracle.quantize_lift(x, mode)
    assert np.array_equal(sa.cpu().numpy(), sa_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)

    # accumulators
    acc = c_gemm_int32(backend, q, op.packed, op.metadata, m, n)
    acc_cpu = acc.cpu()
    lifted = torch.from_numpy(oracle.slide_weight(qweight, mode)).to(torch.int64)          # [n, valid]
    valid = lifted.shape[1]
    q64 = torch.from_numpy(q_ref[:m, :valid]).to(torch.int64)
    # (b) checksums
    assert torch.equal(acc_cpu.sum(dim=1, dtype=torch.int64), q64 @ lifted.sum(dim=0))
    assert torch.equal(acc_cpu.sum(dim=0, dtype=torch.int64), lifted @ q64.sum(dim=0))
    # (a) exact sample and (c) sliding identity
    gen = torch.Generator().manual_seed(7)
    rows = torch.randperm(m, generator=gen)[:48]
    cols = torch.randperm(n, generator=gen)[:160]
    sample = acc_cpu[rows][:, cols].to(torch.int64)
    assert torch.equal(sample, q64[rows] @ lifted[cols].T)
    xq, _ = oracle.quantize_lift(x[rows], 4)          # mode 2:4 lifts nothing: plain quantised rows
    base = torch.from_numpy(xq[:len(rows), :k]).to(torch.int64)
    assert torch.equal(sample, base @ torch.from_numpy(qweight[cols.numpy()]).to(torch.int64).T)

    # complete projection
    y = op(xd)
    expect = oracle_c.epilogue(acc_cpu.numpy(), sa_ref, scales, bias.numpy())
    assert np.array_equal(bits(y), expect)
    assert backend.device_status(torch.device(DEV)) == 0
