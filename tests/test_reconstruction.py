"""Weight preparation on CPU: the C oracle of `compress` against the reference's own results
(tests/golden/reconstruction.npz, written by tests/golden/make_golden.py from
diffusion_research/reconstruction.py run on CPU), `factor_hessian` against the stored factors, and
the argument errors of the package's `compress` (which needs no GPU to refuse bad input)."""
from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reconstruction.npz")
CASES = [tuple(int(v) for v in row) for row in GOLDEN["cases"]]


@pytest.fixture(scope="module")
def recon(sdk):
    from slidesparse_diffusion_b200 import reconstruction
    return reconstruction


@pytest.mark.parametrize("index", range(len(CASES)))
def test_oracle_reproduces_the_reference_bit_for_bit(oracle_c, index):
    rows, columns, group, blocksize, joint, tail, explicit = CASES[index]
    g = lambda key: GOLDEN[f"{key}{index}"]
    q, zeros, w, losses = oracle_c.obs_compress(g("weight"), g("upper"), g("dead"), g("scales"), group, blocksize,
                                                bool(joint))
    assert np.array_equal(zeros, g("zeros"))
    assert np.array_equal(q, g("qweight"))
    assert np.array_equal(w.view(np.uint32), g("compensated").view(np.uint32))
    assert np.array_equal(losses.view(np.uint32), g("proxy_loss").view(np.uint32))
    # the structure the packer relies on
    complete = columns // group * group
    per_group = (q[:, :complete].reshape(rows, -1, group) != 0).sum(-1)
    assert per_group.max() <= group - 2


@pytest.mark.parametrize("index", range(len(CASES)))
def test_factor_hessian_matches_the_reference(recon, index):
    g = lambda key: GOLDEN[f"{key}{index}"]
    curvature = recon.factor_hessian(torch.from_numpy(g("hessian")), damping=.01)
    assert np.array_equal(curvature.dead.numpy(), g("dead"))
    assert abs(curvature.damping - float(g("damping"))) <= 1e-7 * abs(float(g("damping")))
    assert np.allclose(curvature.upper.numpy(), g("upper"), rtol=1e-5, atol=1e-7)
    assert np.array_equal(recon.channel_scales(torch.from_numpy(g("weight"))).numpy(), g("scales")) or len(g("scales_in"))


def test_factor_hessian_refuses_bad_input(recon):
    eye = torch.eye(4)
    with pytest.raises(ValueError):
        recon.factor_hessian(torch.zeros(3, 4))
    with pytest.raises(ValueError):
        recon.factor_hessian(eye, damping=-1.0)
    with pytest.raises(ValueError):
        recon.factor_hessian(eye + torch.triu(torch.ones(4, 4), 1))
    bad = eye.clone()
    bad[0, 0] = 0
    bad[0, 1] = bad[1, 0] = .5
    with pytest.raises(ValueError):
        recon.factor_hessian(bad)
    with pytest.raises(ValueError):
        recon.factor_hessian(eye * float("nan"))


def test_compress_refuses_bad_input_before_touching_the_gpu(recon):
    curvature = recon.factor_hessian(torch.eye(12))
    weight = torch.randn(3, 12)
    for kwargs in (dict(group=5), dict(group=4, method="obc"), dict(group=4, blocksize=6), dict(group=4, blocksize=0)):
        with pytest.raises(ValueError):
            recon.compress(weight, curvature, **kwargs)
    with pytest.raises(ValueError):
        recon.compress(torch.randn(12), curvature, 4)
    with pytest.raises(ValueError):
        recon.compress(weight * float("inf"), curvature, 4)
    with pytest.raises(ValueError):
        recon.compress(torch.randn(3, 10), recon.factor_hessian(torch.eye(10)), 4)          # tail not allowed
    with pytest.raises(ValueError):
        recon.compress(torch.randn(3, 16), curvature, 4)                                    # width mismatch
    with pytest.raises(ValueError):
        recon.compress(weight, curvature, 4, scales=torch.tensor([1., 0., 1.]))
    with pytest.raises(ValueError, match="GPU only"):
        recon.compress(weight, curvature, 4)


def test_widest_block_is_reported_without_a_gpu(recon):
    assert recon.max_blocksize() == 225
    with pytest.raises(ValueError):
        recon.compress(torch.randn(3, 12), recon.factor_hessian(torch.eye(12)), 4, blocksize=228)
