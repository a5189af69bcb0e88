"""The C-ABI library loads without a GPU and exports every symbol the header declares; host
entry points (packer, format helpers, argument validation) behave as documented."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "slidesparse_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ss_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(backend):
    lib = backend.library()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_header_cites_reference_for_each_entry():
    text = HEADER.read_text()
    blocks = re.findall(r"/\*((?:(?!\*/).)*)\*/\s*(?:const char\*|int)\s+(ss_[a-z0-9_]+)\s*\(", text, flags=re.S)
    assert len(blocks) >= 18
    for comment, name in blocks:
        if name in ("ss_last_error", "ss_meta_convert", "ss_device_status"):
            continue            # library plumbing without a reference counterpart
        if "No counterpart in the reference" in " ".join(comment.split()):
            continue            # additions that say so themselves
        assert re.search(r"\.(py|cu|cuh):\d+", comment), f"{name} lacks a reference file:line citation"


def test_load_does_not_initialise_cuda(sdk):
    assert not torch.cuda.is_initialized()


def test_query_without_device(backend):
    out = (ctypes.c_int64 * 8)()
    assert backend.library().ss_query(-1, out, 8) == 0
    assert out[0] == 1 and out[1] == 100 and out[6] == 512


def test_lifted_k_entry(backend):
    valid, pk = ctypes.c_int64(), ctypes.c_int64()
    lib = backend.library()
    for k, mode, expect in ((1152, 6, (1536, 1536)), (2432, 6, (3248, 3328)), (12288, 8, (18432, 18432)), (7, 6, (16, 128))):
        assert lib.ss_lifted_k(k, mode, ctypes.byref(valid), ctypes.byref(pk)) == 0
        assert (valid.value, pk.value) == expect
    assert lib.ss_lifted_k(0, 4, None, None) == backend.SS_E_ARG
    assert lib.ss_lifted_k(8, 5, None, None) == backend.SS_E_ARG
    assert b"group" in lib.ss_last_error()


def test_host_packer_matches_oracle(backend, oracle):
    lib = backend.library()
    for mode, n, k in ((4, 40, 128), (6, 33, 130), (8, 70, 200), (6, 96, 1152), (8, 64, 2432)):
        qweight, _ = oracle.make_weight(n, k, mode, seed=n)
        lifted_ref = oracle.slide_weight(qweight, mode)
        valid, pk = oracle.lifted_k(k, mode)
        lifted = np.zeros((n, valid), np.int8)
        assert lib.ss_slide_weight_cpu(qweight.ctypes.data, n, k, mode, lifted.ctypes.data) == 0
        assert np.array_equal(lifted, lifted_ref)
        pn = -(-n // 32) * 32
        packed = np.zeros((pn, pk // 2), np.int8)
        raw = np.zeros((pn, pk // 32), np.uint32)
        hw = np.zeros(pn * pk // 32, np.uint32)
        assert lib.ss_pack_cpu(lifted.ctypes.data, n, valid, pk, packed.ctypes.data, raw.ctypes.data, hw.ctypes.data) == 0
        packed_ref, raw_ref = oracle.pack(lifted_ref, pk)
        assert np.array_equal(packed, packed_ref) and np.array_equal(raw, raw_ref)
        assert np.array_equal(hw, oracle.meta_to_b200(raw_ref, pk))
        back = np.zeros_like(raw)
        assert lib.ss_meta_convert(hw.ctypes.data, back.ctypes.data, pn, pk, 0) == 0
        assert np.array_equal(back, raw_ref)


def test_host_packer_matches_reference_golden(backend):
    data = np.load(ROOT / "tests/golden/slide_pack.npz")
    lib = backend.library()
    for i, (l, n, k) in enumerate(data["cases"]):
        l, n, k = int(l), int(n), int(k)
        valid, pk = (int(v) for v in data[f"dims{i}"])
        w = np.ascontiguousarray(data[f"w{i}"])
        lifted = np.zeros((n, valid), np.int8)
        assert lib.ss_slide_weight_cpu(w.ctypes.data, n, k, l, lifted.ctypes.data) == 0
        assert np.array_equal(lifted, data[f"lifted{i}"])
        pn = -(-n // 32) * 32
        packed = np.zeros((pn, pk // 2), np.int8)
        assert lib.ss_pack_cpu(lifted.ctypes.data, n, valid, pk, packed.ctypes.data, None, None) == 0
        assert np.array_equal(packed, data[f"packed{i}"])


def test_format_violations_are_reported(backend):
    lib = backend.library()
    bad = np.array([[1, 2, 3, 4, 5, 0]], np.int8)
    out = np.zeros((1, 8), np.int8)
    assert lib.ss_slide_weight_cpu(bad.ctypes.data, 1, 6, 6, out.ctypes.data) == backend.SS_E_FORMAT
    assert b"(L-2):L" in lib.ss_last_error()
    three = np.array([[1, 2, 3, 0]], np.int8)
    packed = np.zeros((32, 64), np.int8)
    assert lib.ss_pack_cpu(three.ctypes.data, 1, 4, 128, packed.ctypes.data, None, None) == backend.SS_E_FORMAT
    assert lib.ss_pack_cpu(three.ctypes.data, 1, 4, 100, packed.ctypes.data, None, None) == backend.SS_E_ARG


def test_launch_entries_validate_before_touching_the_gpu(backend):
    lib = backend.library()
    dummy = ctypes.c_void_p(256)
    assert lib.ss_quantize_lift(None, 8, 1, 8, 4, dummy, dummy, None) == backend.SS_E_ARG
    assert lib.ss_quantize_lift(dummy, 8, 1, 8, 5, dummy, dummy, None) == backend.SS_E_ARG
    assert lib.ss_quantize_lift(dummy, 4, 1, 8, 4, dummy, dummy, None) == backend.SS_E_ARG          # stride < k
    assert lib.ss_gemm_int32(dummy, dummy, dummy, dummy, 1, 1, 32, 32, 100, None) == backend.SS_E_ARG   # pk % 128
    assert lib.ss_gemm_int32(dummy, dummy, dummy, dummy, 1, 1, 32, 32, 131072, None) == backend.SS_E_ARG  # int32 bound
    assert lib.ss_gemm_int32(dummy, dummy, dummy, dummy, 40, 1, 32, 32, 128, None) == backend.SS_E_ARG    # m > pm
    assert lib.ss_plan_run(12345, dummy, 8, None, None, dummy, 8, None) == backend.SS_E_HANDLE
    assert lib.ss_plan_release(12345) == 0


def test_tuning_switches_round_trip_on_the_host(backend):
    """ss_set_option / ss_get_option need no GPU: the switches live in host memory."""
    assert backend.get_option("token_tile") == 0 and backend.get_option("resident") == 1
    assert backend.get_option("wait_ns") == 2_000_000_000
    for name, value in (("token_tile", 240), ("store", 0), ("meta_warp", 1), ("wait_ns", 7_000_000)):
        previous = backend.set_option(name, value)
        assert backend.get_option(name) == value
        backend.set_option(name, previous)
        assert backend.get_option(name) == previous
    lib = backend.library()
    assert lib.ss_set_option(b"no_such_switch", 1) == backend.SS_E_ARG and b"no_such_switch" in lib.ss_last_error()
    assert lib.ss_set_option(b"wait_ns", 0) == backend.SS_E_ARG
    assert lib.ss_get_option(b"pdl", None) == backend.SS_E_ARG


def test_diagnostic_entries_validate_before_touching_the_gpu(backend):
    lib = backend.library()
    elapsed = ctypes.c_int64()
    assert lib.ss_micro_wait_limit(0, ctypes.byref(elapsed)) == backend.SS_E_ARG
    assert lib.ss_micro_wait_limit(10 ** 12, ctypes.byref(elapsed)) == backend.SS_E_ARG          # beyond 100 ms
    assert lib.ss_micro_wait_limit(1000, None) == backend.SS_E_ARG
    cycles, stages = ctypes.c_double(), ctypes.c_int64()
    assert lib.ss_micro_pair_rate(256, 256, 100, 0, 0, ctypes.byref(cycles), ctypes.byref(stages)) == backend.SS_E_ARG
    assert lib.ss_micro_pair_rate(256, 256, 256, 0, 16, ctypes.byref(cycles), ctypes.byref(stages)) == backend.SS_E_ARG
    assert lib.ss_gemm_resources(4096, 4608, 1152, None, 8) == backend.SS_E_ARG
