"""Denoiser harness on the GPU: device-side preparation of routed groups and sparse routed steps."""
import numpy as np
import pytest
import torch

from gpu_util import bits

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def mods(sdk, backend):
    from slidesparse_diffusion_b200 import denoiser, routing
    return denoiser, routing


@pytest.mark.parametrize("mode,widths,k", [(4, (48, 48, 48), 128), (6, (40, 24), 300), (8, (200,), 1152)])
def test_pack_members_matches_host_preparation_and_oracle(mods, sdk, oracle, mode, widths, k):
    """Device prune + grid + pack of fused members == the oracle's grid and packer on the same pruned
    weight, and the routed output == the oracle projection bit for bit."""
    _, routing = mods
    torch.manual_seed(mode)
    members = [torch.nn.Linear(k, w).to(DEV, torch.bfloat16) for w in widths]
    op = routing.pack_members(members, mode)
    weight = torch.cat([m.weight for m in members]).detach().float().cpu().numpy()
    bias = torch.cat([m.bias for m in members]).detach().float().cpu().numpy()
    pruned, _ = oracle.magnitude_prune(weight, mode)
    qweight, scales = oracle.weight_grid(pruned)
    assert np.array_equal(op.scales.cpu().numpy(), scales)
    _, pk = oracle.lifted_k(k, mode)
    packed_ref, raw = oracle.pack(oracle.slide_weight(qweight, mode), pk)
    assert np.array_equal(op.packed.cpu().numpy(), packed_ref)
    assert np.array_equal(op.metadata.cpu().numpy().view(np.uint32), oracle.meta_to_b200(raw, pk))
    x = oracle.make_activation(70, k, seed=mode)
    state = routing.ProjectionState(members, {mode: op})
    state.select(mode)
    with torch.no_grad():
        outs = state.members_output(x.to(DEV))
    expect = oracle.projection(x, qweight, scales, bias, mode)["out_bits"]
    assert np.array_equal(bits(torch.cat(outs, -1)), expect)


@pytest.mark.parametrize("name", ["dit-xl-512", "pixart-sigma-1024", "sd35-large-512"])
def test_sparse_denoise_step_tracks_dense_with_pruned_weights(mods, name):
    """A sparse routed forward stays close to the dense forward of the same model whose routed
    weights were replaced by their pruned + INT8-dequantised values (W8A8 noise only)."""
    denoiser, routing = mods
    spec = denoiser.tiny(denoiser.SPECS[name], hidden=256, heads=4, mlp=512, grid=8, text_dim=128)
    kwargs = {f: getattr(spec, f) for f in ("blocks", "hidden", "heads", "mlp", "grid", "text_tokens",
                                            "text_dim", "pooled_dim", "classes")}
    model = denoiser.build(name, device=DEV, steps=4, **kwargs)
    mode = model.pack(only_profitable=False)
    loop = denoiser.DenoiseLoop(model, graph=True)
    cond = loop.conditioning(seed=2)
    side = spec.grid * spec.patch
    latent = torch.randn(2, spec.latent_channels, side, side, device=DEV).to(torch.bfloat16)
    t = torch.full((2,), 321.0, device=DEV)
    with torch.no_grad():
        model.select(mode)
        sparse = model(latent, t, cond).float()
        model.select(0)
        # overwrite routed dense weights with what the sparse operator actually multiplies by
        for state in model.states:
            op = state.ops[mode]
            raw = op.identity
            assert raw["metadata_layout"] == "b200-v1"
            start = 0
            dense = _dequantised(op)
            for member in state.members:
                member.weight.copy_(dense[start:start + member.out_features].to(member.weight.dtype))
                start += member.out_features
        dense_out = model(latent, t, cond).float()
    err = (sparse - dense_out).abs().max() / dense_out.abs().max().clamp_min(1e-6)
    assert torch.isfinite(sparse).all() and float(err) < 0.08, float(err)
    model.select(mode)
    a = loop.run(seed=1)
    b = loop.run(seed=1)
    assert torch.isfinite(a).all() and torch.equal(a, b)


def _dequantised(op):
    """[n,k] fp32 weight the packed operator represents (values x per-channel scale)."""
    from slidesparse_diffusion_b200 import importer
    from __graft_entry__ import load_oracle
    oracle, _ = load_oracle()
    pk = op.identity["k_physical"]
    raw = importer.b200_metadata_to_raw(op.metadata.cpu(), op.packed.shape[0], pk).numpy().view(np.uint32)
    lifted = oracle.unpack(op.packed.cpu().numpy(), raw)[:op.n]                 # [n, pk] over lifted columns
    src = oracle.lift_indices(op.k, op.mode)                 # every retained weight sits in exactly one window
    dense = np.zeros((op.n, op.k + 1), dtype=np.int32)
    np.add.at(dense, (slice(None), src), lifted[:, :len(src)].astype(np.int32))
    return torch.from_numpy(dense[:, :op.k].astype(np.float32) * op.scales.cpu().numpy()[:, None]).to(op.packed.device)
