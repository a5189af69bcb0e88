"""Projection routing and the denoiser harness on CPU, with exact stand-in operators.

The sparse kernels need a GPU; here each routed group gets an operator that computes the dense
product of the concatenated members, so a routed forward must reproduce the dense forward exactly
up to fp32 summation order.  That checks the fusing of Q|K|V / K|V members, the splits, the text /
image stream wiring and the protected-prefix addend path (reference:
sdacc/diffusion_research/models/projections.py:26-62, sd3.py:52-65, sigma.py:73-86)."""
import pytest
import torch
from torch.nn import functional as F


@pytest.fixture(scope="module")
def mods(sdk):
    from slidesparse_diffusion_b200 import denoiser, routing
    return denoiser, routing


def dense_operator(members, mode, protected_prefix=0):
    weight = torch.cat([m.weight for m in members]).detach()[:, protected_prefix:]
    bias = torch.cat([m.bias for m in members]).detach()

    def run(x, output_addend=None):
        y = F.linear(x, weight, bias)
        return y if output_addend is None else y + output_addend
    return run


@pytest.mark.parametrize("name,per_block", [("dit-xl-512", 3), ("pixart-sigma-1024", 5), ("sd35-large-512", 6)])
def test_routed_forward_equals_dense_forward(mods, name, per_block):
    denoiser, _ = mods
    spec = denoiser.tiny(denoiser.SPECS[name])
    model = denoiser.build(name, device="cpu", dtype=torch.float32, **{f: getattr(spec, f) for f in (
        "blocks", "hidden", "heads", "mlp", "grid", "text_tokens", "text_dim", "pooled_dim", "classes")})
    expected_units = per_block * spec.blocks - (2 if spec.family == "mmdit" else 0)
    assert len(model.units) == len(model.states) == expected_units
    assert [u["unit"] for u in model.units] == list(range(expected_units))
    loop = denoiser.DenoiseLoop(model, dtype=torch.float32)
    cond = loop.conditioning(seed=3)
    side = spec.grid * spec.patch
    latent = torch.randn(2, spec.latent_channels, side, side, generator=torch.Generator().manual_seed(1))
    t = torch.tensor([500.0, 500.0])
    with torch.no_grad():
        dense = model(latent, t, cond)
        mode = model.pack(packer=dense_operator, only_profitable=False)
        assert mode == spec.mode
        model.select(mode)
        routed = model(latent, t, cond)
        model.select(0)
        again = model(latent, t, cond)
    assert dense.shape == (2, spec.out_channels, side, side)
    assert torch.equal(dense, again)
    assert torch.allclose(dense, routed, rtol=1e-4, atol=1e-5)
    # row counts follow the reference inventory: CFG pair x tokens of the stream that feeds the group
    for unit in model.units:
        text_rows = unit["module"].startswith("text.") or unit["module"] == "cross-KV"
        assert unit["m"] == 2 * (spec.text_tokens if text_rows else spec.tokens)


def test_projection_state_contract(mods):
    _, routing = mods
    torch.manual_seed(0)
    q, k, v = (torch.nn.Linear(12, 8) for _ in range(3))
    state = routing.ProjectionState([q, k, v], {6: dense_operator([q, k, v], 6)})
    x = torch.randn(5, 12)
    for bad in (2, 4, 8, True, "6"):
        with pytest.raises(ValueError):
            state.select(bad)
    state.select(6)
    outs = state.members_output(x)
    assert [o.shape[-1] for o in outs] == [8, 8, 8]
    for out, member in zip(outs, (q, k, v)):
        assert torch.allclose(out, member(x), atol=1e-6)
    assert torch.allclose(state.teacher(x), torch.cat(outs, -1), atol=1e-6)
    with pytest.raises(ValueError):
        routing.ProjectionState([q, k], {}, protected_prefix=4)


def test_protected_prefix_goes_through_the_addend(mods):
    _, routing = mods
    torch.manual_seed(1)
    mixed = torch.nn.Linear(20, 6)
    seen = {}

    def op(x, output_addend=None):
        seen["k"], seen["addend"] = x.shape[-1], output_addend
        return F.linear(x, mixed.weight[:, 8:], mixed.bias) + output_addend

    state = routing.ProjectionState([mixed], {8: op}, protected_prefix=8)
    proxy = routing.OrdinaryProxy(state)
    x = torch.randn(3, 20)
    dense = proxy(x)
    state.select(8)
    routed = proxy(x)
    assert seen["k"] == 12 and seen["addend"].shape == (3, 6)
    assert torch.allclose(dense, routed, atol=1e-5)
    assert torch.allclose(state.teacher(x), F.linear(x[:, 8:], mixed.weight[:, 8:], mixed.bias))
    with pytest.raises(ValueError):
        state.members_output(x)


@pytest.mark.parametrize("name", ["dit-xl-512", "pixart-sigma-1024", "sd35-large-512"])
def test_sampling_loop_runs_and_is_deterministic(mods, name):
    denoiser, _ = mods
    spec = denoiser.tiny(denoiser.SPECS[name])
    kwargs = {f: getattr(spec, f) for f in ("blocks", "hidden", "heads", "mlp", "grid", "text_tokens",
                                            "text_dim", "pooled_dim", "classes")}
    model = denoiser.build(name, device="cpu", dtype=torch.float32, steps=6, **kwargs)
    loop = denoiser.DenoiseLoop(model, dtype=torch.float32)
    a = loop.run(seed=4)
    b = loop.run(seed=4)
    c = loop.run(seed=5)
    assert torch.isfinite(a).all() and torch.equal(a, b) and not torch.equal(a, c)


def test_sampler_tables(mods):
    denoiser, _ = mods
    for name, spec in denoiser.SPECS.items():
        ts, coef = denoiser.sampler_table(spec)
        assert ts.shape == (spec.steps,) and coef.shape == (spec.steps, 4)
        assert torch.isfinite(coef).all() and torch.all(ts[:-1] > ts[1:])
    # flow matching integrates sigma from 1 to 0
    _, coef = denoiser.sampler_table(denoiser.SPECS["sd35-large-512"])
    assert abs(float(coef[:, 1].sum()) + 1.0) < 1e-5
    # DDIM with a perfect noise prediction recovers x0 at the last step: x = sqrt(a) x0 + sqrt(1-a) eps
    spec = denoiser.SPECS["dit-xl-512"]
    ts, coef = denoiser.sampler_table(spec)
    ac = denoiser._alphas_cumprod()
    x0, eps = torch.tensor(0.7, dtype=torch.float64), torch.tensor(-1.3, dtype=torch.float64)
    x = ac[int(ts[0])].sqrt() * x0 + (1 - ac[int(ts[0])]).sqrt() * eps
    for a, b, _, _ in coef.double():
        x = a * x + b * eps
    assert abs(float(x - x0)) < 1e-4
    # DPM-Solver++ likewise (x0 constant => multistep correction vanishes)
    spec = denoiser.SPECS["pixart-sigma-1024"]
    ts, coef = denoiser.sampler_table(spec)
    x = ac[int(ts[0])].sqrt() * x0 + (1 - ac[int(ts[0])]).sqrt() * eps
    prev = torch.tensor(0.0, dtype=torch.float64)
    for i, (a, b, c, d) in enumerate(coef.double()):
        alpha = ac[int(ts[i])].sqrt()
        e = (x - alpha * x0) / (1 - ac[int(ts[i])]).sqrt()       # the exact noise at this point
        cur = x * torch.sqrt(1 + d * d) - d * e
        x = a * x + b * e + c * prev
        prev = cur
        assert abs(float(cur - x0)) < 1e-3
    assert abs(float(x - x0)) < 1e-3


def test_images_for_rank(mods):
    denoiser, _ = mods
    for world in (1, 2, 4, 8):
        parts = [denoiser.images_for_rank(64, r, world) for r in range(world)]
        assert sorted(sum(parts, [])) == list(range(64))
        assert {len(p) for p in parts} == {64 // world}


def test_unprofitable_groups_stay_dense(mods, sdk):
    """pack() skips the shapes profile.selectable rejects; select() leaves them on the dense path."""
    denoiser, _ = mods
    from slidesparse_diffusion_b200 import profile
    assert not profile.selectable(8, 600, 1152, 2304)          # PixArt cross-KV: launch-latency sized
    assert not profile.selectable(8, 8192, 1152, 1152)         # cross-attention Q: square, no neighbour to absorb
    assert profile.selectable(4, 2048, 1152, 3456) and profile.selectable(6, 666, 9728, 2432)
    spec = denoiser.tiny(denoiser.SPECS["pixart-sigma-1024"])
    kwargs = {f: getattr(spec, f) for f in ("blocks", "hidden", "heads", "mlp", "grid", "text_tokens",
                                            "text_dim", "pooled_dim", "classes")}
    model = denoiser.build("pixart-sigma-1024", device="cpu", dtype=torch.float32, **kwargs)
    mode = model.pack(packer=dense_operator)                   # tiny shapes: nothing is profitable
    assert model.sparse_units(mode) == 0
    model.select(mode)
    assert all(state.active == 0 for state in model.states)
