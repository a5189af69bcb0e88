"""Properties of the oracle that the reference guards with run-time invariants, and agreement of
its two restatements (numpy and C) where no reference CPU code exists to run."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st


def bits(x):
    return x.view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("mode,k", [(4, 40), (6, 36), (8, 40), (6, 38), (8, 44), (6, 130), (8, 257)])
def test_slide_plus_lift_is_exact(oracle, mode, k):
    """lift(q) . slide(w)^T == q . w^T in int32: the expansion neither drops nor doubles a term."""
    qw, _ = oracle.make_weight(24, k, mode, seed=k)
    x = oracle.make_activation(17, k, seed=mode)
    q, sa = oracle.quantize_lift(x, mode)
    logical, _ = oracle.quantize_lift(x, 4) if k % 4 == 0 else (None, None)
    lifted = oracle.slide_weight(qw, mode)
    acc = oracle.gemm_int32(q, lifted, 17)
    # un-lifted quantised activations: recompute with the scalar formula
    xf = x.float().numpy()
    inv = (np.float32(1) / sa[:17]).astype(np.float32)
    plain = np.rint(np.clip(xf * inv[:, None], -128, 127)).astype(np.int32)
    assert np.array_equal(acc, plain @ qw.astype(np.int32).T)
    if logical is not None:
        assert np.array_equal(logical[:17, :k].astype(np.int32), plain)


def test_quantize_hand_cases(oracle, oracle_c):
    x = torch.tensor([[0.5, -1.0, 127.0, 63.5], [0.0, 0.0, 0.0, 0.0], [1.5, 2.5, -2.5, 254.0]],
                     dtype=torch.bfloat16)
    q, sa = oracle.quantize_lift(x, 4)
    assert q.shape == (32, 128) and sa.shape == (32,)
    assert sa[0] == np.float32(1.0) and q[0, :4].tolist() == [0, -1, 127, 64]      # 0.5 -> 0 (half-even)
    assert sa[1] == np.float32(1.0) / (np.float32(127.0) * np.float32(512.0))        # scale floor
    assert q[1, :4].tolist() == [0, 0, 0, 0]
    assert sa[2] == np.float32(2.0) and q[2, :4].tolist() == [1, 1, -1, 127]        # 0.75->1, 1.25->1
    assert (sa[3:] == 1.0).all() and not q[3:].any()
    qc, sac = oracle_c.quantize_lift(bits(x), 4)
    assert np.array_equal(q, qc) and np.array_equal(sa, sac)


def test_quantize_nonfinite_conventions(oracle, oracle_c):
    x = torch.tensor([[float("nan"), 1.0, -2.0, 0.5], [float("inf"), 1.0, -1.0, float("-inf")]],
                     dtype=torch.bfloat16)
    q, sa = oracle.quantize_lift(x, 4)
    assert q[0, :4].tolist() == [-128, 64, -127, 32]       # NaN is ignored by absmax, quantises to -128
    assert np.isinf(sa[1]) and q[1, :4].tolist() == [-128, 0, 0, -128]
    qc, sac = oracle_c.quantize_lift(bits(x), 4)
    assert np.array_equal(q, qc) and np.array_equal(sa, sac)


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 40), st.integers(1, 90), st.sampled_from([4, 6, 8]), st.integers(0, 2 ** 31 - 1))
def test_numpy_and_c_quantize_agree(oracle, oracle_c, m, k, mode, seed):
    x = oracle.make_activation(m, k, seed=seed)
    q, sa = oracle.quantize_lift(x, mode)
    qc, sac = oracle_c.quantize_lift(bits(x), mode)
    assert np.array_equal(q, qc) and np.array_equal(sa, sac)


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 50), st.integers(4, 80), st.sampled_from([4, 6, 8]), st.integers(0, 2 ** 31 - 1))
def test_gemm_restatements_agree(oracle, oracle_c, n, k, mode, seed):
    qw, _ = oracle.make_weight(n, k, mode, seed=seed)
    x = oracle.make_activation(9, k, seed=seed + 1)
    q, _ = oracle.quantize_lift(x, mode)
    lifted = oracle.slide_weight(qw, mode)
    _, pk = oracle.lifted_k(k, mode)
    packed, raw = oracle.pack(lifted, pk)
    acc = oracle.gemm_int32(q, lifted, 9)
    assert np.array_equal(acc, oracle_c.gemm_int32(q, lifted, 9))
    assert np.array_equal(acc, oracle_c.gemm_int32_packed(q, packed, raw, 9, n))


def test_epilogue_restatements_agree(oracle, oracle_c):
    rng = np.random.default_rng(0)
    acc = rng.integers(-2 ** 20, 2 ** 20, size=(64, 48)).astype(np.int32)
    sa = rng.uniform(1e-3, 0.2, 64).astype(np.float32)
    sw = rng.uniform(1e-4, 1e-2, 48).astype(np.float32)
    bias = rng.normal(0, 0.1, 48).astype(np.float32)
    add = torch.from_numpy(rng.normal(0, 1, (64, 48)).astype(np.float32)).to(torch.bfloat16)
    for b in (None, bias):
        for a in (None, add):
            py = oracle.epilogue(acc, sa, sw, b, a)
            c = oracle_c.epilogue(acc, sa, sw, b, None if a is None else bits(a))
            assert np.array_equal(py, c)


def test_epilogue_hand_case(oracle):
    acc = np.array([[3, -5]], np.int32)
    out = oracle.epilogue(acc, np.array([0.5], np.float32), np.array([2.0, 0.25], np.float32),
                          np.array([1.0, 0.0], np.float32))
    got = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16).float().tolist()
    assert got == [[4.0, -0.625]]


def test_magnitude_prune_structure(oracle):
    for mode in (4, 6, 8):
        qw, scales = oracle.make_weight(16, 70, mode, seed=mode)
        groups = np.pad(qw, ((0, 0), (0, (-70) % mode))).reshape(16, -1, mode)
        assert (np.count_nonzero(groups, axis=-1) <= mode - 2).all()
        assert (scales > 0).all()
