"""Parity of the CUDA path with the CPU oracle, called through the C ABI.  Bit-exact for the
INT8 activations, scales, packed weights, metadata and INT32 accumulators; the BF16 output is
compared bit-for-bit as well (the stated tolerance is 1 BF16 ulp = relative 2^-8; mismatches are
counted and must be zero, the ulp bound is asserted as a backstop)."""
import numpy as np
import pytest
import torch

from gpu_util import bits, c_gemm_int32, c_gemm_run, c_quantize_lift, option, prepare_case, ptr, stream, check

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.view(dtype)).to(DEV)


@pytest.mark.parametrize("mode", [4, 6, 8])
@pytest.mark.parametrize("m,k", [(1, 8), (31, 40), (32, 128), (33, 130), (200, 1152), (64, 2432),
                                 (96, 3072), (40, 12288), (7, 4100), (5, 16384)])
def test_frontend_bit_exact(backend, oracle, mode, m, k):
    x = oracle.make_activation(m, k, seed=m * 31 + k)
    q_ref, sa_ref = oracle.quantize_lift(x, mode)
    q, sa = c_quantize_lift(backend, x.to(DEV), mode)
    torch.cuda.synchronize()
    assert np.array_equal(sa.cpu().numpy(), sa_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)


@pytest.mark.parametrize("mode", [4, 6, 8])
def test_frontend_strided_and_unaligned_rows(backend, oracle, mode):
    wide = oracle.make_activation(50, 15360 // 8 + 6, seed=5).to(DEV)
    for lo, hi in ((384, 384 + 1536), (3, 3 + 1001), (0, 77)):
        view = wide[:, lo:hi]
        q_ref, sa_ref = oracle.quantize_lift(view.cpu().contiguous(), mode)
        q, sa = c_quantize_lift(backend, view, mode)
        assert np.array_equal(q.cpu().numpy(), q_ref) and np.array_equal(sa.cpu().numpy(), sa_ref)


def test_frontend_nonfinite(backend, oracle):
    x = oracle.make_activation(4, 256, seed=1)
    x[0, 3] = float("nan")
    x[1, 7] = float("inf")
    x[2, :] = 0
    x[3, 100] = float("-inf")
    for mode in (4, 6, 8):
        q_ref, sa_ref = oracle.quantize_lift(x, mode)
        q, sa = c_quantize_lift(backend, x.to(DEV), mode)
        assert np.array_equal(q.cpu().numpy(), q_ref)
        assert np.array_equal(sa.cpu().numpy(), sa_ref)


SHAPES = [(4, 32, 128, 32), (4, 100, 256, 200), (6, 64, 132, 96), (8, 130, 200, 129), (4, 256, 1152, 512),
          (6, 300, 1152, 384), (8, 257, 1152, 640), (6, 128, 2432, 256), (4, 512, 4608, 1152),
          (8, 192, 3072, 1024), (4, 1, 64, 1), (6, 40, 38, 30)]


@pytest.mark.parametrize("mode,m,k,n", SHAPES)
def test_gemm_int32_accumulators_bit_exact(backend, oracle, mode, m, k, n):
    case = prepare_case(oracle, m, k, n, mode, seed=n)
    q, packed, meta = dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32)
    acc = c_gemm_int32(backend, q, packed, meta, m, n)
    torch.cuda.synchronize()
    assert backend.device_status() == 0
    assert np.array_equal(acc.cpu().numpy(), case["acc"])


@pytest.mark.parametrize("tile", [128, 192, 224, 240, 256])
@pytest.mark.parametrize("store", [1, 0])
def test_every_kernel_variant_is_exact(backend, oracle, oracle_c, tile, store):
    """Every token tile of the kernel (240 ends in a half chunk of 16 tokens), with the TMA-store
    and the direct-store epilogue, ragged edges in M, N and K; BF16 output and INT32 dump."""
    case = prepare_case(oracle, 700, 640, 300, 6, seed=tile)
    with option(backend, "token_tile", tile), option(backend, "store", store):
        wide = torch.full((700, 304), float("nan"), dtype=torch.bfloat16, device=DEV)   # 16-byte row pitch
        lib = backend.library()
        q, packed, meta = dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32)
        sa, sw, bias = dev(case["sa"]), dev(case["scales"]), dev(case["bias"])
        check(backend, lib.ss_gemm_run(ptr(q), ptr(packed), ptr(meta), ptr(sa), ptr(sw), ptr(bias), None, 0, ptr(wide), 304,
                                       700, 300, q.shape[0], packed.shape[0], q.shape[1], stream()))
        out = c_gemm_run(backend, q, packed, meta, sa, sw, bias, 700, 300)              # row pitch 300: direct stores
        acc = c_gemm_int32(backend, q, packed, meta, 700, 300)
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"])
    assert np.array_equal(bits(wide[:, :300]), expect)
    assert torch.isnan(wide[:, 300:].float()).all()                # nothing written beyond the last channel
    assert np.array_equal(bits(out), expect)
    assert np.array_equal(acc.cpu().numpy(), case["acc"])
    assert backend.device_status() == 0


@pytest.mark.parametrize("mode,m,k,n", [(6, 1800, 256, 9216), (8, 3700, 384, 4500), (4, 4096, 1152, 4608), (4, 7300, 1280, 2304)])
@pytest.mark.parametrize("resident", [0, 1])
def test_weights_resident_form_is_exact(backend, oracle, oracle_c, mode, m, k, n, resident):
    """Shapes on which the weights-resident form of the kernel applies (short K, at least four
    token tiles per cluster), with it switched off and on: same bits either way, ragged M and N."""
    case = prepare_case(oracle, m, k, n, mode, seed=m + n)
    with option(backend, "resident", resident):
        out = c_gemm_run(backend, dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32),
                         dev(case["sa"]), dev(case["scales"]), dev(case["bias"]), m, n)
    assert np.array_equal(bits(out), oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"]))
    assert backend.device_status() == 0


@pytest.mark.parametrize("meta_warp,wide_cp", [(0, 1), (0, 0), (1, 0)])
def test_metadata_copy_variants_are_exact(backend, oracle, oracle_c, meta_warp, wide_cp):
    """The switches that decide who copies a stage's metadata into TMEM (the metadata warp or the
    MMA thread) and how (one 128x256b copy or two 128x128b): same bits in every combination, odd and
    even numbers of 128-column blocks."""
    for k in (640, 1536):                                   # 6:8 -> 1024 (8 blocks) / 2304 lifted columns (18 blocks); 4:6 of 640 -> 7 blocks
        for mode in (8, 6):
            case = prepare_case(oracle, 1000, k, 520, mode, seed=k + mode)
            with option(backend, "meta_warp", meta_warp), option(backend, "wide_cp", wide_cp), option(backend, "resident", 0):
                out = c_gemm_run(backend, dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32),
                                 dev(case["sa"]), dev(case["scales"]), dev(case["bias"]), 1000, 520)
            assert np.array_equal(bits(out), oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"]))
    assert backend.device_status() == 0


@pytest.mark.parametrize("tile", [224, 240, 256])
def test_large_token_tiles_full_height(backend, oracle, oracle_c, tile):
    """Several complete token tiles per cluster (so both accumulators and the half chunk of the
    240-token tile are used repeatedly), aligned output."""
    m, k, n, mode = 2 * 240 * 7 + 17, 512, 4096, 8
    case = prepare_case(oracle, m, k, n, mode, seed=tile + 1)
    with option(backend, "token_tile", tile), option(backend, "resident", 0):
        out = c_gemm_run(backend, dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32),
                         dev(case["sa"]), dev(case["scales"]), dev(case["bias"]), m, n)
    assert np.array_equal(bits(out), oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"]))
    assert backend.device_status() == 0


_CAPTURE_STREAM = []


def _capture_stream():
    # one stream for all captures of this module: the library hands its split-schedule areas to at
    # most four streams per device
    if not _CAPTURE_STREAM:
        _CAPTURE_STREAM.append(torch.cuda.Stream())
    return _CAPTURE_STREAM[0]


@pytest.mark.parametrize("tile", [0, 128, 192, 224, 240, 256])
@pytest.mark.parametrize("mode,m,k,n", [(6, 666, 2432, 2304), (8, 256, 3072, 1024), (4, 700, 1152, 5000), (6, 100, 9728, 304),
                                        (4, 1, 1152, 8), (8, 33, 512, 264)])
def test_split_schedule_is_exact(backend, oracle, oracle_c, tile, mode, m, k, n):
    """The split schedule forced on (every cluster takes an equal share of the tiles x stages, shared
    tiles are summed through global memory by whichever piece arrives last): the same bits as the
    whole-tile schedule's oracle, launch after launch (the sums must be left zero), with tiles
    shared by two and by many clusters, ragged M, N and K, and under CUDA-graph replay."""
    case = prepare_case(oracle, m, k, n, mode, seed=tile + n)
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"])
    q, packed, meta = dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32)
    sa, sw, bias = dev(case["sa"]), dev(case["scales"]), dev(case["bias"])
    pitch = -(-n // 8) * 8
    lib = backend.library()
    with option(backend, "split", 1), option(backend, "token_tile", tile), option(backend, "resident", 0):
        launches = backend.get_option("split_launches")
        for _ in range(3):
            wide = torch.full((m, pitch + 8), float("nan"), dtype=torch.bfloat16, device=DEV)
            check(backend, lib.ss_gemm_run(ptr(q), ptr(packed), ptr(meta), ptr(sa), ptr(sw), ptr(bias), None, 0, ptr(wide),
                                           pitch + 8, m, n, q.shape[0], packed.shape[0], q.shape[1], stream()))
            if n % 8 == 0:
                assert np.array_equal(bits(wide[:, :n]), expect)
                assert torch.isnan(wide[:, n:].float()).all()
            else:
                assert np.array_equal(bits(wide[:, :n]), expect)       # unaligned n: the direct-store form ran
        assert backend.get_option("split_launches") == launches + (3 if n % 8 == 0 else 0)
        if n % 8 == 0:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
            side = _capture_stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                # one launch outside the capture: a stream's split area is made by its first such launch
                check(backend, lib.ss_gemm_run(ptr(q), ptr(packed), ptr(meta), ptr(sa), ptr(sw), ptr(bias), None, 0, ptr(out),
                                               n, m, n, q.shape[0], packed.shape[0], q.shape[1], stream()))
                before = backend.get_option("split_launches")
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    check(backend, lib.ss_gemm_run(ptr(q), ptr(packed), ptr(meta), ptr(sa), ptr(sw), ptr(bias), None, 0, ptr(out),
                                                   n, m, n, q.shape[0], packed.shape[0], q.shape[1], stream()))
            assert backend.get_option("split_launches") == before + 1      # the captured launch is a split one
            torch.cuda.current_stream().wait_stream(side)
            for _ in range(3):
                out.fill_(float("nan"))
                graph.replay()
                torch.cuda.synchronize()
                assert np.array_equal(bits(out), expect)
    assert backend.device_status() == 0


def test_split_schedule_chosen_by_the_cost_model(backend, oracle, oracle_c):
    """A launch whose tiles fill a round and a fraction of the next (87 tiles of 224 tokens on 74
    clusters): the library's own choice, against the split schedule switched off."""
    m, k, n, mode = 666, 2432, 7296, 6
    case = prepare_case(oracle, m, k, n, mode, seed=5)
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"])
    args = (dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32), dev(case["sa"]), dev(case["scales"]),
            dev(case["bias"]), m, n)
    assert np.array_equal(bits(c_gemm_run(backend, *args)), expect)
    # a launch the cost model gives the split schedule (100 tiles of 76 stages on 74 clusters), at a
    # size the CPU oracle would take minutes for: seeded random operands, and the bits must equal
    # those of the whole-tile schedule, whose results the other tests pin to the oracle
    m2, n2, pk2 = 2048, 2432, 13056
    gen = torch.Generator(device=DEV).manual_seed(11)
    q2 = torch.randint(-127, 128, (m2, pk2), dtype=torch.int8, device=DEV, generator=gen)
    packed2 = torch.randint(-127, 128, (n2, pk2 // 2), dtype=torch.int8, device=DEV, generator=gen)
    meta2 = torch.full((n2 * pk2 // 32,), 0x44444444, dtype=torch.int32, device=DEV)       # positions 0 and 1 of every group of four
    sa2 = torch.rand(m2, device=DEV, generator=gen) + 0.5
    sw2 = torch.rand(n2, device=DEV, generator=gen) * 1e-3 + 1e-4
    bias2 = torch.randn(n2, device=DEV, generator=gen)
    launches = backend.get_option("split_launches")
    auto = c_gemm_run(backend, q2, packed2, meta2, sa2, sw2, bias2, m2, n2)
    assert backend.get_option("split_launches") == launches + 1
    with option(backend, "split", 0):
        whole = c_gemm_run(backend, q2, packed2, meta2, sa2, sw2, bias2, m2, n2)
    assert backend.get_option("split_launches") == launches + 1
    assert np.array_equal(bits(auto), bits(whole))
    with option(backend, "split", 0):
        assert np.array_equal(bits(c_gemm_run(backend, *args)), expect)
    assert backend.device_status() == 0


@pytest.mark.parametrize("mode,m,k,n", SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_gemm_bf16_output(backend, oracle, oracle_c, mode, m, k, n, with_bias):
    case = prepare_case(oracle, m, k, n, mode, seed=n + 1, with_bias=with_bias)
    q, packed, meta = dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32)
    sa, sw = dev(case["sa"]), dev(case["scales"])
    bias = dev(case["bias"]) if with_bias else None
    out = c_gemm_run(backend, q, packed, meta, sa, sw, bias, m, n)
    got = bits(out)
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"])
    assert np.array_equal(expect, case["out_bits"])        # both oracle restatements agree
    assert int((got != expect).sum()) == 0
    ref = torch.from_numpy(expect.view(np.int16)).view(torch.bfloat16).float()
    assert torch.all((out.cpu().float() - ref).abs() <= ref.abs() * 2.0 ** -8)


def test_gemm_addend(backend, oracle, oracle_c):
    m, k, n, mode = 150, 512, 200, 8
    case = prepare_case(oracle, m, k, n, mode, seed=3)
    wide = (torch.randn(m, n + 24, generator=torch.Generator().manual_seed(9))).to(torch.bfloat16)
    addend = wide[:, 8:8 + n]                      # row stride != n
    out = c_gemm_run(backend, dev(case["q"]), dev(case["packed"]), dev(case["meta_b200"], torch.int32),
                     dev(case["sa"]), dev(case["scales"]), dev(case["bias"]), m, n,
                     addend=wide.to(DEV)[:, 8:8 + n])
    expect = oracle_c.epilogue(case["acc"], case["sa"], case["scales"], case["bias"], bits(addend))
    assert np.array_equal(bits(out), expect)


@pytest.mark.parametrize("mode,n,k", [(4, 40, 128), (6, 96, 300), (8, 70, 200), (6, 33, 1153), (8, 64, 2432)])
def test_device_packer_bit_exact(backend, oracle, mode, n, k):
    qweight, _ = oracle.make_weight(n, k, mode, seed=k)
    _, pk = oracle.lifted_k(k, mode)
    packed_ref, raw = oracle.pack(oracle.slide_weight(qweight, mode), pk)
    pn = packed_ref.shape[0]
    packed = torch.full((pn, pk // 2), 0x33, dtype=torch.int8, device=DEV)
    meta = torch.zeros(pn * pk // 32, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    check(backend, backend.library().ss_pack_device(ptr(dev(qweight)), n, k, mode, ptr(packed), ptr(meta),
                                                    ptr(status), stream()))
    assert int(status.item()) == 0
    assert np.array_equal(packed.cpu().numpy(), packed_ref)
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), oracle.meta_to_b200(raw, pk))


def test_device_packer_flags_bad_structure(backend):
    qweight = torch.tensor([[1, 2, 3, 4, 5, 0] * 4], dtype=torch.int8, device=DEV)
    packed = torch.zeros((32, 128), dtype=torch.int8, device=DEV)
    meta = torch.zeros(32 * 8, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    check(backend, backend.library().ss_pack_device(ptr(qweight), 1, 24, 6, ptr(packed), ptr(meta), ptr(status), stream()))
    assert int(status.item()) == 1


def test_device_weight_grid(backend, oracle):
    w = (torch.randn(37, 301, generator=torch.Generator().manual_seed(4)) * 0.02)
    w[5] = 0
    q_ref, s_ref = oracle.weight_grid(w.numpy())
    q = torch.empty((37, 301), dtype=torch.int8, device=DEV)
    s = torch.empty(37, dtype=torch.float32, device=DEV)
    check(backend, backend.library().ss_weight_grid_device(ptr(w.to(DEV)), 37, 301, ptr(q), ptr(s), stream()))
    assert np.array_equal(s.cpu().numpy(), s_ref) and np.array_equal(q.cpu().numpy(), q_ref)


def test_kernels_match_reference_gpu_golden(sdk, backend, oracle):
    """The B200 kernels against outputs of the reference's own GPU operators (recompiled for
    sm_100 and run on a B200 by oracle/ref_gpu.py; tests/golden/ref_gpu.npz): INT8 activations,
    token scales and the BF16 projection output, bit for bit."""
    import importlib.util
    from pathlib import Path
    root = Path(__file__).resolve().parent
    spec = importlib.util.spec_from_file_location("ss_ref_gpu", root.parent / "oracle" / "ref_gpu.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    data = np.load(root / "golden" / "ref_gpu.npz")
    for index, (mode, m, k, n, config, has_bias, has_addend) in enumerate(ref.CASES):
        x, qweight, scales, b, a = ref.case_inputs(oracle, index, mode, m, k, n, has_bias, has_addend)
        q, sa = sdk.quantize_lift(x.to(DEV), mode)
        if f"q{index}" in data:
            assert np.array_equal(q.cpu().numpy(), data[f"q{index}"]) and np.array_equal(sa.cpu().numpy(), data[f"sa{index}"])
        op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales),
                                      torch.from_numpy(b) if b.size else None, mode).to(DEV)
        y = op(x.to(DEV), output_addend=None if a is None else a.to(DEV))
        assert np.array_equal(bits(y), data[f"y{index}"]), index
