"""This library against the reference's own GPU operators at the full sizes of the benchmark
configurations, on the same GPU: the reference (its `projection_sm80.cu`, recompiled unmodified for
sm_100 by oracle/ref_gpu.py) runs in a child process, because both libraries register the same
torch operator namespaces, and reports SHA-256 digests of its INT8 activations, token scales,
packed weights and BF16 outputs; the digests of this library's results on the same seeded inputs
must be identical."""
import hashlib
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REFERENCE_LIBRARY = ROOT / "oracle" / "_ref" / "projection_sm100.so"


def _sha(t):
    return hashlib.sha256(t.contiguous().cpu().numpy().tobytes()).hexdigest()


@pytest.mark.skipif(not REFERENCE_LIBRARY.exists(), reason="the reference's GPU library has not been built (oracle/ref_gpu.py build)")
def test_full_size_outputs_equal_the_reference_gpu_kernels(sdk, oracle, tmp_path):
    spec = importlib.util.spec_from_file_location("ss_ref_gpu", ROOT / "oracle" / "ref_gpu.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = tmp_path / "digest.json"
    child = subprocess.run([sys.executable, str(ROOT / "oracle" / "ref_gpu.py"), "digest", "--out", str(out)],
                           capture_output=True, text=True, timeout=900)
    assert child.returncode == 0, child.stderr[-2000:]
    rows = json.loads(out.read_text())["rows"]
    assert len(rows) == len(ref.FULL_CASES)
    for index, ((mode, m, k, n, config), row) in enumerate(zip(ref.FULL_CASES, rows)):
        assert row["case"] == [mode, m, k, n, config]
        x, qweight, scales, bias = ref.full_case_inputs(oracle, index, mode, m, k, n)
        op = sdk.PackedLinear.prepare(torch.from_numpy(qweight), torch.from_numpy(scales), torch.from_numpy(bias), mode)
        assert _sha(op.packed) == row["packed"], (index, "packed weights")
        op = op.to("cuda:0")
        q, sa = sdk.quantize_lift(x.to("cuda:0"), mode)
        assert _sha(sa) == row["sa"], (index, "token scales")
        assert _sha(q) == row["q"], (index, "INT8 activations")
        y = op(x.to("cuda:0"))
        assert _sha(y.view(torch.int16)) == row["y"], (index, "BF16 output")
