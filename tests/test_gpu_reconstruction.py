"""Weight preparation on the GPU: the `compress` kernels through the package against the C oracle
(bit for bit: selected zeros, INT8 weight, compensated fp32 weight, proxy loss), against the
reference's own results on the golden cases, and through to a packed projection."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reconstruction.npz")
CASES = [tuple(int(v) for v in row) for row in GOLDEN["cases"]]


@pytest.fixture(scope="module")
def recon(sdk):
    from slidesparse_diffusion_b200 import reconstruction
    return reconstruction


def _bits(t):
    return t.detach().cpu().contiguous().numpy().view(np.uint32)


@pytest.mark.parametrize("index", range(len(CASES)))
def test_golden_cases_equal_the_reference(recon, index):
    rows, columns, group, blocksize, joint, tail, explicit = CASES[index]
    g = lambda key: GOLDEN[f"{key}{index}"]
    dev = "cuda:0"
    curvature = recon.Curvature(torch.from_numpy(g("upper")).to(dev), torch.from_numpy(g("dead")).to(dev),
                                float(g("damping")))
    seen = []
    result = recon.compress(torch.from_numpy(g("weight")).to(dev), curvature, group,
                            method="joint" if joint else "prune_then_rtn", blocksize=blocksize,
                            scales=torch.from_numpy(g("scales_in")).to(dev) if explicit else None,
                            allow_tail=bool(tail), progress=lambda **kw: seen.append(kw))
    assert np.array_equal(result["zeros"].cpu().numpy(), g("zeros"))
    assert np.array_equal(result["qweight"].cpu().numpy(), g("qweight"))
    assert np.array_equal(_bits(result["scales"]), g("scales").view(np.uint32))
    assert np.array_equal(_bits(result["compensated"]), g("compensated").view(np.uint32))
    assert np.array_equal(_bits(result["proxy_loss"]), g("proxy_loss").view(np.uint32))
    assert seen[-1] == dict(finalized_columns=columns, total_columns=columns)
    assert len(seen) == -(-columns // blocksize)
    assert result["group"] == group and result["blocksize"] == blocksize and not result["activation_error_compensated"]


def _synthetic(rows, columns, seed, dead=()):
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1, size=(2 * columns, columns)).astype(np.float32)
    x[:, rng.permutation(columns)[:max(1, columns // 100)]] *= 10
    x[:, list(dead)] = 0
    hessian = torch.from_numpy(x.T @ x / x.shape[0])
    weight = torch.from_numpy(rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32))
    return weight, (hessian + hessian.T) / 2


@pytest.mark.parametrize("rows,columns,group,blocksize,method,dead", [
    (300, 384, 4, 192, "joint", ()),
    (130, 576, 6, 192, "joint", (5, 200, 201)),
    (257, 512, 8, 192, "prune_then_rtn", ()),
    (64, 1152, 6, 96, "joint", ()),
    (33, 410, 8, 200, "joint", (409,)),          # tail group of 2 columns
    (1000, 224, 4, 224, "joint", ()),            # widest usable block the kernel holds
])
def test_kernels_match_the_oracle(recon, oracle_c, rows, columns, group, blocksize, method, dead):
    assert blocksize <= recon.max_blocksize()
    weight, hessian = _synthetic(rows, columns, seed=rows + columns, dead=dead)
    curvature = recon.factor_hessian(hessian)                       # CPU: both sides get the same factor
    assert int(curvature.dead.sum()) == len(dead)
    scales = recon.channel_scales(weight)
    q, zeros, w, losses = oracle_c.obs_compress(weight.numpy(), curvature.upper.numpy(), curvature.dead.numpy(),
                                                scales.numpy(), group, blocksize, method == "joint")
    dev = "cuda:0"
    on_gpu = recon.Curvature(curvature.upper.to(dev), curvature.dead.to(dev), curvature.damping)
    result = recon.compress(weight.to(dev), on_gpu, group, method=method, blocksize=blocksize,
                            allow_tail=bool(columns % group))
    assert np.array_equal(result["zeros"].cpu().numpy(), zeros)
    assert np.array_equal(result["qweight"].cpu().numpy(), q)
    assert np.array_equal(_bits(result["compensated"]), w.view(np.uint32))
    assert np.array_equal(_bits(result["proxy_loss"]), losses.view(np.uint32))
    again = recon.compress(weight.to(dev), on_gpu, group, method=method, blocksize=blocksize,
                           allow_tail=bool(columns % group))
    assert torch.equal(again["qweight"], result["qweight"]) and torch.equal(again["compensated"], result["compensated"])


def test_compensation_beats_magnitude_pruning_and_feeds_the_packer(sdk, recon, oracle):
    """On correlated inputs the compensated weight has a lower output error than magnitude pruning
    plus rounding, and the result goes through PackedLinear.prepare into the sparse projection."""
    rows, columns, group = 256, 1152, 6
    rng = np.random.default_rng(5)
    mix = (rng.normal(0, 1, size=(columns, columns)) / np.sqrt(columns)).astype(np.float32)
    x = rng.normal(0, 1, size=(4096, columns)).astype(np.float32) @ (np.eye(columns, dtype=np.float32) + 2 * mix)
    hessian = torch.from_numpy(x.T @ x / x.shape[0])
    weight = torch.from_numpy(rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32))
    dev = "cuda:0"
    curvature = recon.factor_hessian(((hessian + hessian.T) / 2).to(dev))
    result = recon.compress(weight.to(dev), curvature, group)
    q, scales = result["qweight"], result["scales"]
    assert int((q.reshape(rows, -1, group) != 0).sum(-1).max()) <= group - 2
    assert torch.equal(q.float() * scales[:, None], result["compensated"])
    # magnitude pruning + rounding on the same grid
    groups = weight.abs().reshape(rows, -1, group)
    keep = torch.ones_like(groups, dtype=torch.bool)
    keep.scatter_(-1, groups.topk(2, dim=-1, largest=False).indices, False)
    plain = (recon.round_signed(weight, scales.cpu()[:, None]) * scales.cpu()[:, None]) * keep.reshape(rows, columns)
    xt = torch.from_numpy(x)
    dense = xt @ weight.T
    err_plain = float((xt @ plain.T - dense).square().mean())
    err_obs = float((xt @ result["compensated"].cpu().T - dense).square().mean())
    assert err_obs < 0.8 * err_plain, (err_obs, err_plain)
    # through the packer into the projection
    op = sdk.PackedLinear.prepare(q.cpu(), scales.cpu(), None, group).to(dev)
    act = oracle.make_activation(64, columns, seed=9)
    y = op(act.to(dev))
    expect = oracle.projection(act, q.cpu().numpy(), scales.cpu().numpy(), None, group)["out_bits"]
    assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), expect)


def test_pack_members_with_a_curvature(sdk, recon, oracle, oracle_c):
    """routing.pack_members(curvature=...) = compress + slide + pack on the device; its projection
    equals the oracle projection of the oracle's compressed weight."""
    from slidesparse_diffusion_b200 import routing
    torch.manual_seed(3)
    dev = "cuda:0"
    q_proj, k_proj = torch.nn.Linear(384, 96), torch.nn.Linear(384, 64)
    _, hessian = _synthetic(1, 384, seed=11)
    on_cpu = recon.factor_hessian(hessian)
    curvature = recon.Curvature(on_cpu.upper.to(dev), on_cpu.dead.to(dev), on_cpu.damping)
    op = routing.pack_members([q_proj.to(dev), k_proj.to(dev)], 8, curvature=curvature)
    weight = torch.cat([q_proj.weight, k_proj.weight]).detach().float().cpu()
    bias = torch.cat([q_proj.bias, k_proj.bias]).detach().float().cpu().numpy()
    scales = recon.channel_scales(weight).numpy()
    q, _, _, _ = oracle_c.obs_compress(weight.numpy(), on_cpu.upper.numpy(), on_cpu.dead.numpy(), scales, 8)
    act = oracle.make_activation(40, 384, seed=2)
    expect = oracle.projection(act, q, scales, bias, 8)["out_bits"]
    y = op(act.to(dev))
    assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), expect)


def test_full_size_weight_sample_rows_equal_the_oracle(recon, oracle_c):
    """FLUX fused-QKV weight (9216 x 3072, 4:6): rows are independent, so 32 rows spread over the
    weight are checked bit for bit against the oracle and every row for the (L-2):L structure and
    the frozen grid."""
    rows, columns, group = 9216, 3072, 6
    dev = "cuda:0"
    gen = torch.Generator(device=dev).manual_seed(77)
    x = torch.randn(2 * columns, columns, device=dev, generator=gen)
    x[:, ::97] *= 8
    hessian = x.T @ x / x.shape[0]
    weight = 0.02 * torch.randn(rows, columns, device=dev, generator=gen)
    curvature = recon.factor_hessian((hessian + hessian.T) / 2)
    result = recon.compress(weight, curvature, group)
    q = result["qweight"]
    assert int((q.reshape(rows, -1, group) != 0).sum(-1).max()) <= group - 2
    assert torch.equal(q.float() * result["scales"][:, None], result["compensated"])
    assert int(result["zeros"].sum()) == rows * columns // group * 2
    pick = torch.arange(0, rows, rows // 32, device=dev)[:32]
    expect_q, expect_zeros, expect_w, expect_loss = oracle_c.obs_compress(
        weight[pick].cpu().numpy(), curvature.upper.cpu().numpy(), curvature.dead.cpu().numpy(),
        result["scales"][pick].cpu().numpy(), group)
    assert np.array_equal(q[pick].cpu().numpy(), expect_q)
    assert np.array_equal(result["zeros"][pick].cpu().numpy(), expect_zeros)
    assert np.array_equal(_bits(result["compensated"][pick]), expect_w.view(np.uint32))
    assert np.array_equal(_bits(result["proxy_loss"][pick]), expect_loss.view(np.uint32))
