"""Bank slots: storage, mode switching and the coefficient arena (reference:
sdacc/diffusion_research/banks.py:30-67,106-127)."""
import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def banks(sdk):
    from slidesparse_diffusion_b200 import banks
    return banks


def make_payloads(sdk, oracle, k=96, n=40, modes=(4, 6, 8), seed=0):
    payloads, dense = {}, {}
    for mode in modes:
        qweight, scales = oracle.make_weight(n, k, mode, seed=seed + mode)
        op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales),
                                      torch.linspace(-1, 1, n), mode)
        payloads[mode] = {key: getattr(op, key).clone().contiguous() for key in ("packed", "metadata", "scales", "bias")}
        dense[mode] = (qweight, scales)
    return payloads, dense


def test_slot_validation(banks, sdk, oracle):
    payloads, _ = make_payloads(sdk, oracle)
    with pytest.raises(ValueError):
        banks.ResidentBankSlot({}, "cpu")
    with pytest.raises(ValueError):
        banks.ResidentBankSlot({5: payloads[4]}, "cpu")
    with pytest.raises(ValueError):
        banks.ResidentBankSlot({4: {k: v for k, v in payloads[4].items() if k != "bias"}}, "cpu")
    bad = dict(payloads[4], scales=payloads[4]["scales"].double())
    with pytest.raises(ValueError):
        banks.ResidentBankSlot({4: bad}, "cpu")
    bad = dict(payloads[4], bias=torch.full_like(payloads[4]["bias"], float("nan")))
    with pytest.raises(ValueError):
        banks.ResidentBankSlot({4: bad}, "cpu")
    with pytest.raises(ValueError):
        banks.ResidentBankSlot(payloads, "cpu", residency="some")


@pytest.mark.parametrize("residency", ["active", "all"])
def test_activate_and_views(banks, sdk, oracle, residency):
    payloads, _ = make_payloads(sdk, oracle)
    slot = banks.ResidentBankSlot(payloads, "cpu", residency=residency)
    ops = slot.operators(96, 40)
    assert set(ops) == {4, 6, 8}
    for mode in (4, 8, 6, 6):
        moved = slot.activate(mode)
        for key in banks.KEYS:
            assert torch.equal(getattr(ops[mode], key), payloads[mode][key])
            assert getattr(ops[mode], key).data_ptr() == slot.views[mode][key].data_ptr()
        if residency == "all":
            assert moved == 0
    if residency == "active":
        assert slot.transfers == 3 and slot.transfer_bytes > 0
        largest = sum(max(row[k].numel() * row[k].element_size() for row in payloads.values()) for k in banks.KEYS)
        assert slot.identity["device_bytes"] == slot.device_bytes == largest
        # the three modes alias one buffer per tensor kind
        assert len({ops[m].packed.data_ptr() for m in ops}) == 1
        weights_only = slot.activate(4, include_parameters=False)
        assert weights_only == sum(payloads[4][k].numel() * payloads[4][k].element_size() for k in ("packed", "metadata"))
    else:
        assert slot.transfers == 0 and len({ops[m].packed.data_ptr() for m in ops}) == 3
    with pytest.raises(ValueError):
        slot.activate(2)


def test_coefficient_arena_rebinds_operator_buffers(banks, sdk, oracle):
    slots, ops, widths = {}, {}, {}
    for uid, n in enumerate((40, 24)):
        payloads, _ = make_payloads(sdk, oracle, n=n, seed=10 * uid)
        slots[uid] = banks.ResidentBankSlot(payloads, "cpu", residency="active")
        ops[uid] = slots[uid].operators(96, n)
        widths[uid] = n
    arena = banks.CoefficientArena(slots, ops, widths)
    assert arena.arena.numel() == 2 * (40 + 24)
    moved = arena.fill(slots, {0: 6, 1: 8})
    assert moved == arena.arena.numel() * 4
    assert torch.equal(ops[0][6].scales, slots[0].host[6]["scales"])
    assert torch.equal(ops[1][8].bias, slots[1].host[8]["bias"])
    base = arena.arena.data_ptr()
    assert ops[0][4].scales.data_ptr() == base and ops[1][4].scales.data_ptr() == base + 4 * 80
    with pytest.raises(ValueError):
        banks.CoefficientArena({0: banks.ResidentBankSlot(make_payloads(sdk, oracle)[0], "cpu", residency="all")},
                               {0: {}}, {0: 40})


def test_payload_from_reference_blob(banks, sdk, oracle):
    """A blob in the reference's bank format (metadata in SM80 order) becomes a slot payload whose
    metadata is this library's order of the same raw words."""
    k, n, mode = 300, 70, 6
    qweight, scales = oracle.make_weight(n, k, mode, seed=3)
    _, pk = oracle.lifted_k(k, mode)
    packed, raw = oracle.pack(oracle.slide_weight(qweight, mode), pk)
    pn = packed.shape[0]
    sm80 = np.empty(pn * pk // 32, dtype=np.uint32)
    sm80[oracle.sm80_meta_index(pn, pk).ravel()] = raw.ravel()
    blob = dict(unit=0, group=mode, compact=torch.from_numpy(packed), scales=torch.from_numpy(scales),
                metadata=torch.from_numpy(sm80.view(np.int32)), q_sha="x")
    got_mode, payload = banks.payload_from_reference(blob, k, n)
    assert got_mode == mode
    assert np.array_equal(payload["metadata"].numpy().view(np.uint32), oracle.meta_to_b200(raw, pk))
    assert torch.equal(payload["packed"], torch.from_numpy(packed)) and payload["bias"].shape == (n,)
    with pytest.raises(ValueError):
        banks.payload_from_reference(dict(blob, group=4), k, n)
