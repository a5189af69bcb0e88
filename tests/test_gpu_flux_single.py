"""The FLUX single-stream call shapes at full size with the real operator
(sdacc/diffusion_research/models/flux_layers.py:45-55, sdacc/w8a8_slidesparse/composite.py:4-19,
workloads/inventory.json g015-g018): a fused Q|K|V|FFN-in projection of 21504 channels, and the
protected mixed output projection whose sparse operand is the column slice x[..., 3072:] of a
[1536, 15360] tensor, read in place, with the dense attention product as the epilogue addend."""
import numpy as np
import pytest
import torch

from gpu_util import bits, c_gemm_int32, verify_accumulators

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
M, HIDDEN, MLP = 1536, 3072, 12288


@pytest.mark.parametrize("mode", [6, 8])
def test_protected_ffn_output_full_size(sdk, backend, oracle, oracle_c, mode):
    qweight, scales = oracle.make_weight(HIDDEN, MLP, mode, seed=40 + mode)
    bias = (0.1 * torch.randn(HIDDEN, generator=torch.Generator().manual_seed(3))).float()
    ffn = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), bias, mode)
    gen = torch.Generator().manual_seed(9)
    attention_weight = (0.02 * torch.randn(HIDDEN, HIDDEN, generator=gen)).to(torch.bfloat16)
    module = sdk.ProtectedFFNOutput(ffn, attention_weight).to(DEV)
    wide = torch.cat([torch.randn(M, HIDDEN, generator=gen).to(torch.bfloat16),
                      oracle.make_activation(M, MLP, seed=77)], dim=1)            # [1536, 15360]
    xd = wide.to(DEV)
    y = module(xd)
    assert y.shape == (M, HIDDEN)

    # the sparse operand is the slice, read with its row stride of 15360: quantised values first
    rest = xd[:, HIDDEN:]
    assert rest.stride(0) == HIDDEN + MLP and not rest.is_contiguous()
    q, sa = sdk.quantize_lift(rest, mode)
    q_ref, sa_ref = oracle.quantize_lift(wide[:, HIDDEN:].contiguous(), mode)
    assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(sa.cpu().numpy(), sa_ref)
    acc = c_gemm_int32(backend, q, module.ffn.packed, module.ffn.metadata, M, HIDDEN).cpu()
    verify_accumulators(oracle, acc, q_ref, qweight, mode, M, HIDDEN)
    # the protected part is the same BF16 product the reference forms (torch.matmul on the GPU)
    addend = torch.matmul(xd[:, :HIDDEN], module.attention_weight.t())
    expect = oracle_c.epilogue(acc.numpy(), sa_ref, scales, bias.numpy(), bits(addend))
    assert np.array_equal(bits(y), expect)
    # 3-D input [batch, tokens, 15360], as the model block passes it
    y3 = module(xd.reshape(2, M // 2, HIDDEN + MLP))
    assert np.array_equal(bits(y3.reshape(M, HIDDEN)), expect)
    resources = module.configure()
    assert set(resources) == {"ffn", "mixed"}
    assert backend.device_status() == 0


def test_shared_qkv_ffn_projection_full_size(sdk, backend, oracle, oracle_c):
    mode, widths = 6, (HIDDEN, HIDDEN, HIDDEN, MLP)
    n = sum(widths)                                                       # 21504
    qweight, scales = oracle.make_weight(n, HIDDEN, mode, seed=11)
    bias = (0.1 * torch.randn(n, generator=torch.Generator().manual_seed(4))).float()
    packed = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), bias, mode).to(DEV)
    shared = sdk.SharedProjection(packed, widths)
    x = oracle.make_activation(M, HIDDEN, seed=5)
    xd = x.to(DEV)
    members = shared(xd)
    assert [tuple(t.shape) for t in members] == [(M, w) for w in widths]
    q, sa = sdk.quantize_lift(xd, mode)
    q_ref, sa_ref = oracle.quantize_lift(x, mode)
    assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(sa.cpu().numpy(), sa_ref)
    acc = c_gemm_int32(backend, q, packed.packed, packed.metadata, M, n).cpu()
    verify_accumulators(oracle, acc, q_ref, qweight, mode, M, n)
    expect = oracle_c.epilogue(acc.numpy(), sa_ref, scales, bias.numpy())
    start = 0
    for member, width in zip(members, widths):
        assert np.array_equal(bits(member), expect[:, start:start + width])
        start += width
    with pytest.raises(ValueError):
        sdk.SharedProjection(packed, (HIDDEN, HIDDEN))
    assert backend.device_status() == 0
