"""The oracle (numpy and C restatements) against vectors produced by the reference's CPU code."""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def slide_pack():
    return np.load(GOLDEN / "slide_pack.npz")


def cases(data):
    for i, (l, n, k) in enumerate(data["cases"]):
        yield i, int(l), int(n), int(k)


def test_lifted_k_matches_reference(oracle, slide_pack):
    for i, l, n, k in cases(slide_pack):
        assert list(oracle.lifted_k(k, l)) == list(slide_pack[f"dims{i}"])
    # values printed by the reference for the benchmark widths
    table = {1152: (1152, 1536, 1792), 3072: (3072, 4096, 4608), 12288: (12288, 16384, 18432),
             2432: (2432, 3328, 3712), 9728: (9728, 13056, 14592), 4608: (4608, 6144, 6912)}
    for k, expect in table.items():
        assert tuple(oracle.lifted_k(k, l)[1] for l in (4, 6, 8)) == expect


def test_slide_weight_matches_reference(oracle, oracle_c, slide_pack):
    for i, l, n, k in cases(slide_pack):
        w, lifted = slide_pack[f"w{i}"], slide_pack[f"lifted{i}"]
        assert np.array_equal(oracle.slide_weight(w, l), lifted)
        assert np.array_equal(oracle_c.slide_weight(w, l), lifted)
    for name, mode in (("small46", 6), ("small68", 8), ("tail46", 6)):
        assert np.array_equal(oracle.slide_weight(slide_pack[name], mode), slide_pack[name + "_lifted"])
        assert np.array_equal(oracle_c.slide_weight(slide_pack[name], mode), slide_pack[name + "_lifted"])


def test_slide_weight_hand_vectors(oracle):
    got = oracle.slide_weight(np.array([[1, 0, 2, 3, 0, 4]], np.int8), "4:6")
    assert got.tolist() == [[1, 0, 2, 0, 0, 3, 0, 4]]
    got = oracle.slide_weight(np.array([[1, 2, 0, 3, 4, 0, 5, 6]], np.int8), "6:8")
    assert got.tolist() == [[1, 2, 0, 0, 0, 3, 4, 0, 0, 0, 5, 6]]
    assert np.array_equal(oracle.slide_weight(np.array([[0, 3, 0, 4]], np.int8), "2:4"), [[0, 3, 0, 4]])


def test_overfull_group_is_rejected(oracle, oracle_c, slide_pack):
    assert int(slide_pack["overfull_raises"]) == 1
    bad = np.array([[1, 2, 3, 4, 5, 0]], np.int8)
    with pytest.raises(ValueError):
        oracle.slide_weight(bad, "4:6")
    with pytest.raises(ValueError):
        oracle_c.slide_weight(bad, 6)


def test_pack_matches_reference(oracle, oracle_c, slide_pack):
    for i, l, n, k in cases(slide_pack):
        lifted = slide_pack[f"lifted{i}"]
        valid, pk = slide_pack[f"dims{i}"]
        packed, raw = oracle.pack(lifted, int(pk))
        assert np.array_equal(packed, slide_pack[f"packed{i}"])
        packed_c, raw_c = oracle_c.pack(lifted, int(pk))
        assert np.array_equal(packed_c, packed) and np.array_equal(raw_c, raw)
        # the reference publishes its metadata only after the SM80 reorder: undo it
        pn = packed.shape[0]
        assert np.array_equal(oracle.meta_from_sm80(slide_pack[f"meta_sm80_{i}"], pn, int(pk)), raw)
        # metadata + values reconstruct the lifted weight
        assert np.array_equal(oracle.unpack(packed, raw)[:n, :valid], lifted)


def test_pack_hand_vector(oracle, slide_pack):
    packed, raw = oracle.pack(slide_pack["pack_in"], 128)
    assert np.array_equal(packed, slide_pack["pack_in_packed"])
    assert packed[0, :4].tolist() == [1, 2, 3, 4] and packed[1, :4].tolist() == [0, 5, 6, 0]
    assert raw[0, 0] == 0x4444449C and raw[1, 0] == 0x44444448 and raw[2, 0] == 0x44444444
    assert np.array_equal(oracle.meta_from_sm80(slide_pack["pack_in_meta_sm80"], 32, 128), raw)


def test_lift_indices_match_reference(oracle):
    data = np.load(GOLDEN / "lift.npz")
    for i, (l, k) in enumerate(data["pairs"]):
        l, k = int(l), int(k)
        idx = oracle.lift_indices(k, l)
        assert np.array_equal(idx, data[f"idx{i}"])
        if f"a{i}" in data:
            a = data[f"a{i}"]
            padded = np.concatenate([a, np.zeros((a.shape[0], 1), np.int8)], axis=1)
            valid, pk = oracle.lifted_k(k, l)
            mine = np.zeros((32, pk), np.int8)
            mine[:a.shape[0], :valid] = padded[:, idx]
            assert np.array_equal(mine, data[f"lifted{i}"])


def test_weight_grid_matches_reference(oracle):
    data = np.load(GOLDEN / "weight_grid.npz")
    q, scales = oracle.weight_grid(data["w"])
    assert np.array_equal(scales, data["scales"])
    assert np.array_equal(q, data["q"])
    assert scales[3] == 1.0


def test_b200_metadata_round_trip(oracle, slide_pack):
    for i, l, n, k in cases(slide_pack):
        pk = int(slide_pack[f"dims{i}"][1])
        _, raw = oracle.pack(slide_pack[f"lifted{i}"], pk)
        hw = oracle.meta_to_b200(raw, pk)
        assert sorted(oracle.b200_meta_index(raw.shape[0], pk).ravel().tolist()) == list(range(hw.size))
        assert np.array_equal(hw[oracle.b200_meta_index(raw.shape[0], pk)], raw)


# ---- vectors produced by the reference's own GPU kernels (oracle/ref_gpu.py, run on a B200) ----

def ref_gpu_cases():
    import hashlib
    import importlib.util
    spec = importlib.util.spec_from_file_location("ss_ref_gpu", Path(__file__).parent.parent / "oracle" / "ref_gpu.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module, hashlib


def test_quantise_lift_matches_reference_gpu_output(oracle, oracle_c):
    """quantize (and quantize_packed16) of the reference, recompiled and run on a GPU: INT8
    activations and token scales, including rows of zeros, sub-floor values, Inf and NaN."""
    module, hashlib = ref_gpu_cases()
    data = np.load(GOLDEN / "ref_gpu.npz")
    assert [tuple(int(v) for v in row) for row in data["cases"]] == [tuple(int(v) for v in c) for c in module.CASES]
    for index, (mode, m, k, n, config, bias, addend) in enumerate(module.CASES):
        x, *_ = module.case_inputs(oracle, index, mode, m, k, n, bias, addend)
        x_bits = x.view(__import__("torch").int16).numpy().view(np.uint16)
        for impl in (oracle, oracle_c):
            q, sa = impl.quantize_lift(x if impl is oracle else x_bits, mode)
            assert hashlib.sha256(np.ascontiguousarray(sa).tobytes()).hexdigest() == str(data[f"sa_sha{index}"]), (index, impl.__name__)
            assert hashlib.sha256(np.ascontiguousarray(q).tobytes()).hexdigest() == str(data[f"q_sha{index}"]), (index, impl.__name__)
            if f"q{index}" in data:
                assert np.array_equal(q, data[f"q{index}"]) and np.array_equal(sa, data[f"sa{index}"])


def test_projection_matches_reference_gpu_output(oracle, oracle_c):
    """run / projection of the reference (sparse GEMM + dequantising epilogue, with and without bias
    and addend): the BF16 output bit for bit, and its CPU packer's bytes on the way."""
    module, hashlib = ref_gpu_cases()
    data = np.load(GOLDEN / "ref_gpu.npz")
    for index, (mode, m, k, n, config, bias, addend) in enumerate(module.CASES):
        x, qweight, scales, b, a = module.case_inputs(oracle, index, mode, m, k, n, bias, addend)
        _, pk = oracle.lifted_k(k, mode)
        packed, raw = oracle.pack(oracle.slide_weight(qweight, mode), pk)
        pn = packed.shape[0]
        sm80 = np.empty(pn * pk // 32, dtype=np.uint32)
        sm80[oracle.sm80_meta_index(pn, pk).ravel()] = raw.ravel()
        assert hashlib.sha256(packed.tobytes()).hexdigest() == str(data[f"packed_sha{index}"])
        assert hashlib.sha256(sm80.view(np.int32).tobytes()).hexdigest() == str(data[f"meta_sha{index}"])
        q, sa = oracle.quantize_lift(x, mode)
        acc = oracle.gemm_int32(q, oracle.unpack(packed, raw)[:n], m)
        out = oracle_c.epilogue(acc, sa, scales, b if b.size else None,
                                None if a is None else a.view(__import__("torch").int16).numpy().view(np.uint16))
        assert np.array_equal(out, data[f"y{index}"]), index
