"""Front-end prologues (LayerNorm + modulation, GELU) against the numpy restatement: the quantised
activations and token scales must be bit-identical, and so must the projection built on them."""
import numpy as np
import pytest
import torch

from gpu_util import bits

pytestmark = pytest.mark.gpu
DEV = "cuda"


def modulation(batch, k, seed, pad=0):
    """shift / scale as views of a wider [batch, 6k + pad] tensor, the way adaLN chunks arrive."""
    g = torch.Generator().manual_seed(seed)
    wide = (0.3 * torch.randn(batch, 6 * k + pad, generator=g)).to(torch.bfloat16)
    return wide, wide[:, k:2 * k], wide[:, 4 * k:5 * k]


@pytest.mark.parametrize("mode,k", [(4, 128), (4, 1152), (6, 1152), (8, 1152), (6, 2432), (8, 4608), (6, 12288), (4, 8)])
def test_gelu_frontend_within_tolerance(backend, oracle, mode, k):
    """GELU uses the hardware tanh approximation (relative error 2^-11): the BF16 activation may
    differ from the fp32 numpy restatement by one unit in the last place.  Tolerance: token scales
    within 2^-7 relative; where the scale is identical, INT8 values differ by at most 1 and in at
    most 5 % of places; everywhere, the dequantised value q * scale within 1.5 quantisation steps."""
    m = 37
    x = (oracle.make_activation(m, k, seed=k + mode).float() * 0.5).to(torch.bfloat16)
    x[3, : min(k, 16)] = 0
    q, sa = backend.quantize_lift_fused(x.to(DEV), mode, backend.Prologue.gelu())
    q_ref, sa_ref = oracle.quantize_lift_fused(x, mode, "gelu")
    q, sa = q.cpu().numpy().astype(np.int32), sa.cpu().numpy()
    assert np.all(np.abs(sa - sa_ref) <= sa_ref * 2.0 ** -7)
    same = sa == sa_ref
    assert same.mean() > 0.5
    diff = np.abs(q - q_ref)
    assert diff[same].max() <= 1 and (diff[same] != 0).mean() <= 5e-2
    assert np.all(np.abs(q * sa[:, None] - q_ref * sa_ref[:, None]) <= 1.5 * sa_ref[:, None])
    # padded rows stay zero with scale one
    assert np.all(q[m:] == 0) and np.all(sa[m:] == 1)


@pytest.mark.parametrize("mode,k,batch,rows", [(4, 1152, 2, 20), (6, 1152, 2, 33), (8, 1152, 3, 7), (6, 2432, 2, 40),
                                               (4, 4608, 1, 9), (8, 3072, 2, 16), (6, 128, 2, 5)])
def test_norm_modulate_frontend_bit_exact(backend, oracle, mode, k, batch, rows):
    x = oracle.make_activation(batch * rows, k, seed=k + rows).reshape(batch, rows, k)
    wide, shift, scale = modulation(batch, k, seed=mode)
    wide_d = wide.to(DEV)
    pro = backend.Prologue.norm_modulate(wide_d[:, k:2 * k], wide_d[:, 4 * k:5 * k], 1e-6)
    q, sa = backend.quantize_lift_fused(x.to(DEV), mode, pro)
    q_ref, sa_ref = oracle.quantize_lift_fused(x.reshape(-1, k), mode, "norm_modulate", shift, scale, rows, 1e-6)
    assert np.array_equal(sa.cpu().numpy(), sa_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    # the separate PyTorch operators give the same BF16 values up to their own rounding steps
    eager = pro.torch_reference(x.to(DEV))
    q2, sa2 = backend.quantize_lift_fused(eager, mode, backend.Prologue("none"))
    assert np.abs(q2.cpu().numpy().astype(np.int32) - q_ref).max() <= 2


def test_projection_fused_matches_oracle(sdk, backend, oracle):
    mode, k, n, batch, rows = 6, 1152, 200, 2, 45
    qweight, scales = oracle.make_weight(n, k, mode, seed=1)
    bias = np.linspace(-0.5, 0.5, n).astype(np.float32)
    op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), torch.from_numpy(bias), mode).to(DEV)
    x = oracle.make_activation(batch * rows, k, seed=5).reshape(batch, rows, k)
    wide, shift, scale = modulation(batch, k, seed=11, pad=8)
    wide_d = wide.to(DEV)
    pro = backend.Prologue.norm_modulate(wide_d[:, k:2 * k], wide_d[:, 4 * k:5 * k], 1e-6)
    y = op.forward_fused(x.to(DEV), pro)
    assert y.shape == (batch, rows, n)
    normed = oracle.prologue_norm_modulate(x.reshape(-1, k), shift, scale, rows, 1e-6, mode)
    expect = oracle.projection(torch.from_numpy(normed).to(torch.bfloat16), qweight, scales, bias, mode)["out_bits"]
    assert np.array_equal(bits(y).reshape(-1, n), expect)
    # GELU prologue: floating point within tolerance (the quantisation step of a token is about
    # max|gelu(x)| / 127; the output may move by a few steps times the weight norm)
    y2 = op.forward_fused(x.to(DEV), backend.Prologue.gelu()).float().cpu().reshape(-1, n)
    act = oracle.prologue_gelu(x.reshape(-1, k))
    expect2 = oracle.projection(torch.from_numpy(act).to(torch.bfloat16), qweight, scales, bias, mode)["out_bits"]
    expect2 = torch.from_numpy(expect2.view(np.int16)).view(torch.bfloat16).float()
    assert float((y2 - expect2).abs().max()) <= 0.02 * float(expect2.abs().max())


def test_prologue_argument_errors(backend):
    x = torch.zeros(2, 4, 64, dtype=torch.bfloat16, device=DEV)
    good = torch.zeros(2, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        backend.Prologue("layernorm")
    with pytest.raises(ValueError):
        backend.quantize_lift_fused(x, 4, backend.Prologue.norm_modulate(good[:, :32], good, 1e-6))
    with pytest.raises(ValueError):
        backend.quantize_lift_fused(x.reshape(8, 64), 4, backend.Prologue.norm_modulate(good, good, 1e-6))
    with pytest.raises(ValueError):
        backend.quantize_lift_fused(torch.zeros(2, 4, 60, dtype=torch.bfloat16, device=DEV), 4, backend.Prologue.gelu())


@pytest.mark.parametrize("name", ["dit-xl-512", "sd35-large-512"])
def test_denoiser_with_fused_neighbours_tracks_unfused(sdk, backend, name):
    from slidesparse_diffusion_b200 import denoiser
    spec = denoiser.tiny(denoiser.SPECS[name], hidden=256, heads=4, mlp=512, grid=8, text_dim=128)
    kwargs = {f: getattr(spec, f) for f in ("blocks", "hidden", "heads", "mlp", "grid", "text_tokens",
                                            "text_dim", "pooled_dim", "classes")}
    model = denoiser.build(name, device=DEV, steps=4, **kwargs)
    mode = model.pack(only_profitable=False)
    model.select(mode)
    loop = denoiser.DenoiseLoop(model)
    cond = loop.conditioning(seed=2)
    side = spec.grid * spec.patch
    latent = torch.randn(2, spec.latent_channels, side, side, device=DEV).to(torch.bfloat16)
    t = torch.full((2,), 500.0, device=DEV)
    with torch.no_grad():
        plain = model(latent, t, cond).float()
        model.fuse_neighbours(True)
        fused = model(latent, t, cond).float()
    err = (plain - fused).abs().max() / plain.abs().max().clamp_min(1e-6)
    assert torch.isfinite(fused).all() and float(err) < 0.05, float(err)


@pytest.mark.parametrize("mode,k,n,batch,rows", [(4, 512, 200, 2, 64), (6, 1152, 1152, 2, 96), (8, 256, 72, 3, 32)])
def test_gated_accumulation_matches_oracle(sdk, backend, oracle, oracle_c, mode, k, n, batch, rows):
    """residual += bf16(gate[b] * y) in the GEMM epilogue (TMA reduction) against the C restatement,
    bit for bit, with the GELU prologue's activation taken from the GPU front-end itself."""
    qweight, scales = oracle.make_weight(n, k, mode, seed=3)
    bias = np.linspace(-0.5, 0.5, n).astype(np.float32)
    op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), torch.from_numpy(bias), mode).to(DEV)
    x = oracle.make_activation(batch * rows, k, seed=8).reshape(batch, rows, k)
    g = torch.Generator().manual_seed(4)
    wide = (0.5 * torch.randn(batch, 6 * n, generator=g)).to(torch.bfloat16)
    gate = wide[:, 2 * n:3 * n]
    residual = torch.randn(batch, rows, n, generator=g).to(torch.bfloat16)
    res_d = residual.to(DEV).clone()
    out = op.forward_fused(x.to(DEV), None, gate=wide.to(DEV)[:, 2 * n:3 * n], residual=res_d)
    assert out.data_ptr() == res_d.data_ptr()
    q, sa = oracle.quantize_lift(x.reshape(-1, k), mode)
    _, pk = oracle.lifted_k(k, mode)
    acc = oracle.gemm_int32(q, oracle.slide_weight(qweight, mode), batch * rows)
    expect = oracle_c.epilogue_gated(acc, sa, scales, bias, gate.contiguous().view(torch.int16).numpy().view(np.uint16),
                                     rows, residual.view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(bits(out).reshape(-1, n), expect)
    # the same through the PyTorch operators, within BF16 rounding of the intermediate
    eager = torch.addcmul(residual.to(DEV), wide.to(DEV)[:, 2 * n:3 * n][:, None], op(x.to(DEV)))
    assert float((eager.float() - out.float()).abs().max()) <= 0.02 * float(eager.float().abs().max())


def test_gated_accumulation_argument_errors(sdk, backend, oracle):
    k, n = 128, 64
    qweight, scales = oracle.make_weight(n, k, 4, seed=1)
    op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), None, 4).to(DEV)
    x = torch.zeros(2, 40, k, dtype=torch.bfloat16, device=DEV)            # 40 rows per batch: not a multiple of 32
    gate = torch.zeros(2, n, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        op.forward_fused(x, None, gate=gate, residual=torch.zeros(2, 40, n, dtype=torch.bfloat16, device=DEV))
    x = torch.zeros(2, 64, k, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        op.forward_fused(x, None, gate=gate, residual=torch.zeros(2, 64, n + 8, dtype=torch.bfloat16, device=DEV)[..., :n])
    with pytest.raises(ValueError):
        op.forward_fused(x, None, gate=gate)
