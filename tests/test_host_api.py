"""Host-side mirror of the reference operator API: names, defaults, validation, payloads."""
import inspect

import numpy as np
import pytest
import torch


def make_op(sdk, oracle, n=48, k=72, mode="4:6", bias=True, **kwargs):
    qweight, scales = oracle.make_weight(n, k, mode, seed=n + k)
    b = torch.linspace(-1, 1, n) if bias else None
    return sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), b, mode, **kwargs), qweight, scales


def test_public_names(sdk):
    for name in ("PackedLinear", "quantize_lift", "slide_weight", "lifted_k", "build_native", "load_native",
                 "compile_projection"):
        assert hasattr(sdk, name)
    sig = inspect.signature(sdk.PackedLinear.prepare)
    assert list(sig.parameters) == ["qweight", "scales", "bias", "mode", "config", "strategy", "frontend"]
    assert sig.parameters["mode"].default == "2:4" and sig.parameters["config"].default == "auto"
    sig = inspect.signature(sdk.PackedLinear.__init__)
    assert list(sig.parameters)[1:] == ["packed", "metadata", "scales", "bias", "k", "n", "mode", "config",
                                        "strategy", "identity", "frontend"]
    sig = inspect.signature(sdk.quantize_lift)
    assert list(sig.parameters) == ["x", "mode", "strategy"]
    assert list(inspect.signature(sdk.PackedLinear.forward).parameters) == ["self", "x", "output_addend"]


def test_group_size_and_lifted_k(sdk):
    assert [sdk.group_size(m) for m in ("2:4", "4:6", "6:8", 4, 6, 8)] == [4, 6, 8, 4, 6, 8]
    for bad in ("1:2", 5, None, True):
        with pytest.raises(ValueError):
            sdk.group_size(bad)
    assert sdk.lifted_k(1152, "6:8") == (1728, 1792)
    assert sdk.lifted_k(2432, 6) == (3248, 3328)
    assert sdk.lifted_k(7, "4:6", alignment=4) == (16, 16)
    for args in ((0, 4), (8, 4, 0), (8, 4, 6)):
        with pytest.raises(ValueError):
            sdk.lifted_k(*args)


def test_slide_weight_contract(sdk, oracle):
    qweight, _ = oracle.make_weight(20, 50, 6, seed=1)
    got = sdk.slide_weight(torch.from_numpy(qweight), "4:6")
    assert got.dtype == torch.int8 and got.is_contiguous()
    assert np.array_equal(got.numpy(), oracle.slide_weight(qweight, 6))
    with pytest.raises(TypeError):
        sdk.slide_weight(torch.zeros(4, 8), "2:4")
    with pytest.raises(TypeError):
        sdk.slide_weight(torch.zeros(8, dtype=torch.int8), "2:4")
    with pytest.raises(ValueError):
        sdk.slide_weight(torch.zeros((0, 8), dtype=torch.int8), "2:4")
    with pytest.raises(ValueError):
        sdk.slide_weight(torch.tensor([[1, 2, 3, 4, 5, 0]], dtype=torch.int8), "4:6")


def test_prepare_produces_reference_buffers(sdk, oracle):
    op, qweight, scales = make_op(sdk, oracle)
    assert (op.k, op.n, op.mode, op.in_features, op.out_features) == (72, 48, 6, 72, 48)
    valid, pk = oracle.lifted_k(72, 6)
    packed_ref, raw = oracle.pack(oracle.slide_weight(qweight, 6), pk)
    assert op.packed.shape == (64, pk // 2) and op.packed.dtype == torch.int8
    assert np.array_equal(op.packed.numpy(), packed_ref)
    assert op.metadata.dtype == torch.int32 and op.metadata.numel() == 64 * pk // 32
    assert np.array_equal(op.metadata.numpy().view(np.uint32), oracle.meta_to_b200(raw, pk))
    assert np.array_equal(op.scales.numpy(), scales) and op.bias.shape == (48,)
    assert op.identity["k_physical"] == pk and op.identity["k_lifted"] == valid
    assert set(dict(op.named_buffers())) == {"packed", "metadata", "scales", "bias"}
    no_bias, _, _ = make_op(sdk, oracle, bias=False)
    assert no_bias.bias.numel() == 0 and no_bias.bias.dtype == torch.float32


def test_prepare_validation(sdk, oracle):
    qweight, scales = oracle.make_weight(16, 24, 4, seed=0)
    q, s = torch.from_numpy(qweight), torch.from_numpy(scales)
    for kwargs in (dict(config=7), dict(strategy="other"), dict(frontend="cutlass")):
        with pytest.raises(ValueError):
            sdk.PackedLinear.prepare(q, s, **kwargs)
    for config in (0, 5, 6, 11, 17, "auto"):
        for frontend in ("triton", "native", "scalar", "packed16", "graph_native", "direct2_packed16", "auto"):
            sdk.PackedLinear.prepare(q, s, config=config, frontend=frontend)
    bad = s.clone()
    bad[3] = 0
    with pytest.raises(ValueError):
        sdk.PackedLinear.prepare(q, bad)
    bad[3] = float("nan")
    with pytest.raises(ValueError):
        sdk.PackedLinear.prepare(q, bad)
    with pytest.raises(ValueError):
        sdk.PackedLinear.prepare(q, s[:-1])
    with pytest.raises(ValueError):
        sdk.PackedLinear.prepare(q, s, bias=torch.full((16,), float("inf")))


def test_forward_rejects_non_cuda_or_wrong_width(sdk, oracle):
    op, _, _ = make_op(sdk, oracle)
    with pytest.raises(ValueError):
        op(torch.zeros(4, 72, dtype=torch.bfloat16))              # CPU tensor
    with pytest.raises(ValueError):
        op(torch.zeros(4, 72))                                    # not BF16


def test_configuration_for(sdk, oracle):
    op, _, _ = make_op(sdk, oracle)
    config, frontend = op.configuration_for(512)
    assert isinstance(config, int) and isinstance(frontend, str)
    fixed, _, _ = make_op(sdk, oracle, config=11, frontend="graph_packed16")
    assert fixed.configuration_for(99) == (11, "graph_packed16")


def test_save_load_round_trip(sdk, oracle, tmp_path):
    op, _, _ = make_op(sdk, oracle, config=5, frontend="triton")
    path = tmp_path / "op.pt"
    op.save(path)
    blob = torch.load(path, weights_only=True)
    assert blob["version"] == 1
    assert set(blob) == {"version", "k", "n", "mode", "config", "strategy", "identity", "frontend", "packed",
                         "metadata", "scales", "bias"}
    back = sdk.PackedLinear.load(path)
    assert (back.config, back.frontend) == ("auto", "auto")
    assert back.identity["loaded_execution_original"] == dict(config=5, frontend="triton")
    for name in ("packed", "metadata", "scales", "bias"):
        assert torch.equal(getattr(back, name), getattr(op, name))
    exact = sdk.PackedLinear.load(path, optimized=False)
    assert (exact.config, exact.frontend) == (5, "triton")
    blob["version"] = 2
    torch.save(blob, path)
    with pytest.raises(ValueError):
        sdk.PackedLinear.load(path)


def test_load_converts_reference_payload(sdk, oracle, tmp_path):
    """A payload with metadata in the reference's SM80 order (golden vector from its pack_cpu)."""
    from pathlib import Path
    data = np.load(Path(__file__).parent / "golden/slide_pack.npz")
    i = 4                                                       # (6, 96, 300)
    l, n, k = (int(v) for v in data["cases"][i])
    pk = int(data[f"dims{i}"][1])
    blob = dict(version=1, k=k, n=n, mode=l, config=5, strategy="register", frontend="triton",
                identity=dict(kernel_source_sha="2787082a7feed4f7d9287578f7b7cac80857770dc4d8d704cdf888dca4a625a4"),
                packed=torch.from_numpy(data[f"packed{i}"]), metadata=torch.from_numpy(data[f"meta_sm80_{i}"]),
                scales=torch.ones(n), bias=torch.empty(0))
    path = tmp_path / "ref.pt"
    torch.save(blob, path)
    op = sdk.PackedLinear.load(path)
    _, raw = oracle.pack(data[f"lifted{i}"], pk)
    assert np.array_equal(op.metadata.numpy().view(np.uint32), oracle.meta_to_b200(raw, pk))
    assert op.identity["metadata_layout"] == "b200-v1"


def test_importer_bank(sdk, oracle):
    from pathlib import Path
    from slidesparse_diffusion_b200 import importer
    data = np.load(Path(__file__).parent / "golden/slide_pack.npz")
    i = 7
    l, n, k = (int(v) for v in data["cases"][i])
    pk = int(data[f"dims{i}"][1])
    op = importer.import_reference_bank(torch.from_numpy(data[f"packed{i}"]), torch.from_numpy(data[f"meta_sm80_{i}"]),
                                        torch.ones(n), None, k, n, l)
    _, raw = oracle.pack(data[f"lifted{i}"], pk)
    assert np.array_equal(importer.b200_metadata_to_raw(op.metadata, op.packed.shape[0], pk).numpy().view(np.uint32), raw)


class FakePacked(torch.nn.Module):
    """Exact stand-in operator: same call contract as PackedLinear, dense arithmetic."""

    def __init__(self, weight, bias=None):
        super().__init__()
        self.weight, self.b = weight, bias
        self.n, self.k = weight.shape

    def configure(self, has_addend=False):
        return [has_addend]

    def forward(self, x, output_addend=None):
        y = torch.nn.functional.linear(x, self.weight, self.b)
        return y if output_addend is None else y + output_addend


def test_shared_projection_splits_members(sdk):
    w = torch.randn(12, 5)
    shared = sdk.SharedProjection(FakePacked(w), (3, 4, 5))
    x = torch.randn(2, 7, 5)
    a, b, c = shared(x)
    full = x @ w.T
    assert torch.equal(a, full[..., :3]) and torch.equal(b, full[..., 3:7]) and torch.equal(c, full[..., 7:])
    with pytest.raises(ValueError):
        sdk.SharedProjection(FakePacked(w), (3, 4))


def test_protected_ffn_output_matches_dense(sdk):
    torch.manual_seed(0)
    w = torch.randn(6, 10).to(torch.bfloat16)
    mixed = sdk.ProtectedFFNOutput(FakePacked(w[:, 2:].contiguous()), w[:, :2].contiguous())
    x = torch.randn(3, 4, 10).to(torch.bfloat16)
    expect = torch.nn.functional.linear(x[..., :2], w[:, :2]) + torch.nn.functional.linear(x[..., 2:], w[:, 2:])
    assert torch.allclose(mixed(x).float(), expect.float(), atol=1e-1)
    assert mixed.configure() == dict(ffn=[False], mixed=[True])
    with pytest.raises(ValueError):
        mixed(x[..., :9])
    with pytest.raises(ValueError):
        sdk.ProtectedFFNOutput(FakePacked(w[:, 2:]), w[:, :2].float())


def test_workload_inventory(sdk, oracle):
    from slidesparse_diffusion_b200 import workloads
    flux = workloads.shapes("flux512")
    assert (flux["single.QKV+FFN-in"]["n"], flux["single.QKV+FFN-in"]["members"]) == (21504, [3072, 3072, 3072, 12288])
    assert flux["single.mixed-FFN-out"]["recipe"] == "protected_ffn" and flux["single.mixed-FFN-out"]["slice_start"] == 3072
    assert workloads.shapes("sd35_large512")["text.FFN-out"]["m"] == 666
    assert workloads.shapes("pixart_sigma512")["text.cross-KV"] == dict(
        m=600, k=1152, n=2304, members=[1152, 1152], recipe="ordinary", row_stride=1152, slice_start=0)
    assert len({(w, m) for w in workloads.MODELS for m in workloads.shapes(w)}) >= 55
    qweight, scales = oracle.make_weight(3456, 1152, 6, seed=0)
    op = workloads.prepare_for("pixart_sigma512", "image.QKV", torch.from_numpy(qweight), torch.from_numpy(scales), mode="4:6")
    assert isinstance(op, sdk.SharedProjection) and op.widths == (1152, 1152, 1152)
    with pytest.raises(ValueError):
        workloads.prepare_for("pixart_sigma512", "image.FFN-in", torch.from_numpy(qweight), torch.from_numpy(scales))
    from slidesparse_diffusion_b200.workloads import pixart_sigma512
    assert pixart_sigma512.WORKLOAD == "pixart_sigma512"


def test_missing_library_fails_loudly(sdk, tmp_path):
    import slidesparse_diffusion_b200.backend as backend
    with pytest.raises(FileNotFoundError):
        backend.load_native(tmp_path)
    (tmp_path / "receipt.json").write_text('{"complete": true, "arch": "sm_80"}')
    (tmp_path / backend.LIBRARY_NAME).write_bytes(b"")
    with pytest.raises(ValueError):
        backend.load_native(tmp_path)


def test_load_refuses_payloads_of_unknown_origin(sdk, oracle, tmp_path):
    """An untagged payload is only converted if the reference's packer wrote it; an unknown layout
    tag is refused (the reference's load checks the hash too, runtime.py:236-238 there)."""
    op, _, _ = make_op(sdk, oracle)
    path = tmp_path / "op.pt"
    op.save(path)
    blob = torch.load(path, weights_only=True)
    for identity in (dict(kernel_source_sha="0" * 64), dict(), dict(metadata_layout="b200-v0", kernel_source_sha="x"),
                     dict(metadata_layout="b200-v1")):
        torch.save(dict(blob, identity=identity), path)
        with pytest.raises(ValueError):
            sdk.PackedLinear.load(path)


def test_prepare_for_keeps_unprofitable_groups_dense(sdk, oracle):
    """workloads.prepare_for refuses a group the profile would not select, as the reference does for
    groups that failed its acceleration gate (workloads/__init__.py:17 there)."""
    from slidesparse_diffusion_b200 import workloads, profile
    assert not profile.selectable(8, 600, 1152, 2304) and profile.selectable(4, 2048, 1152, 4608)
    qweight, scales = oracle.make_weight(2304, 1152, 8, seed=0)
    with pytest.raises(ValueError, match="keep Dense"):
        workloads.prepare_for("pixart_sigma512", "text.cross-KV", torch.from_numpy(qweight), torch.from_numpy(scales), mode="6:8")
    qweight, scales = oracle.make_weight(4608, 1152, 4, seed=0)
    op = workloads.prepare_for("pixart_sigma512", "image.FFN-in", torch.from_numpy(qweight), torch.from_numpy(scales))
    assert isinstance(op, sdk.PackedLinear) and (op.k, op.n) == (1152, 4608)
