"""Build recipe and ctypes wrappers for the C oracle (oracle/ss_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__ (build + smoke) and bench.py's
CPU-baseline / reference legs, never by the product package.
"""
import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libss_oracle.so"
_lib = None


def build(force=False):
    src = HERE / "ss_oracle.c"
    if LIB.exists() and not force and LIB.stat().st_mtime >= src.stat().st_mtime:
        return LIB
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
           str(src), "-o", str(LIB), "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


def load():
    global _lib
    if _lib is None:
        if not LIB.exists():
            build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.sso_slide_weight.restype = ctypes.c_int64
        _lib.sso_pack.restype = ctypes.c_int64
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return ctypes.c_int64(int(v))


def slide_weight(qweight, l):
    w = np.ascontiguousarray(qweight, dtype=np.int8)
    n, k = w.shape
    valid = -(-k // l) * (l // 2 - 1) * 4
    out = np.zeros((n, valid), dtype=np.int8)
    rc = load().sso_slide_weight(_p(w), _i64(n), _i64(k), ctypes.c_int(l), _p(out))
    if rc:
        raise ValueError(f"weight violates the frozen (L-2):L structure (row {rc - 1})")
    return out


def pack(lifted, pk):
    w = np.ascontiguousarray(lifted, dtype=np.int8)
    n, kl = w.shape
    pn = -(-n // 32) * 32
    packed = np.zeros((pn, pk // 2), dtype=np.int8)
    raw = np.zeros((pn, pk // 32), dtype=np.uint32)
    rc = load().sso_pack(_p(w), _i64(n), _i64(kl), _i64(pk), _p(packed), _p(raw))
    if rc:
        raise ValueError(f"more than 2 nonzeros in a frozen 2:4 group (row {rc - 1})")
    return packed, raw


def quantize_lift(x_bits, l, row_stride=None):
    """x_bits: uint16 BF16 bit patterns [m,k] (or a strided view given row_stride)."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    m, k = x.shape
    sx = k if row_stride is None else row_stride
    valid = -(-k // l) * (l // 2 - 1) * 4
    pk, pm = -(-valid // 128) * 128, -(-m // 32) * 32
    q = np.empty((pm, pk), dtype=np.int8)
    sa = np.empty(pm, dtype=np.float32)
    load().sso_quantize_lift(_p(x), _i64(sx), _i64(m), _i64(k), ctypes.c_int(l), _p(q), _p(sa))
    return q, sa


def gemm_int32(q, lifted, m):
    q = np.ascontiguousarray(q, dtype=np.int8)
    w = np.ascontiguousarray(lifted, dtype=np.int8)
    n, kl = w.shape
    acc = np.empty((m, n), dtype=np.int32)
    load().sso_gemm_int32(_p(q), _i64(q.shape[1]), _p(w), _i64(kl), _i64(m), _i64(n), _p(acc))
    return acc


def gemm_int32_packed(q, packed, raw, m, n):
    q = np.ascontiguousarray(q, dtype=np.int8)
    packed = np.ascontiguousarray(packed, dtype=np.int8)
    raw = np.ascontiguousarray(raw, dtype=np.uint32)
    acc = np.empty((m, n), dtype=np.int32)
    load().sso_gemm_int32_packed(_p(q), _i64(q.shape[1]), _p(packed), _p(raw), _i64(m), _i64(n), _p(acc))
    return acc


def epilogue(acc, sa, sw, bias=None, addend_bits=None):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    sa = np.ascontiguousarray(sa, dtype=np.float32)
    sw = np.ascontiguousarray(sw, dtype=np.float32)
    out = np.empty((m, n), dtype=np.uint16)
    b = None if bias is None or np.size(bias) == 0 else np.ascontiguousarray(bias, dtype=np.float32)
    a = None if addend_bits is None else np.ascontiguousarray(addend_bits, dtype=np.uint16)
    load().sso_epilogue(_p(acc), _p(sa), _p(sw), _p(b) if b is not None else None,
                        _p(a) if a is not None else None, _i64(n), _i64(m), _i64(n), _p(out))
    return out


if __name__ == "__main__":
    print(build(force=True))


def epilogue_gated(acc, sa, sw, bias, gate_bits, rows_per_batch, residual_bits):
    """BF16 bits of residual + bf16(gate[row // rows_per_batch] * fma(float(acc), sa*sw, bias))."""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    sa = np.ascontiguousarray(sa, dtype=np.float32)
    sw = np.ascontiguousarray(sw, dtype=np.float32)
    b = None if bias is None or np.size(bias) == 0 else np.ascontiguousarray(bias, dtype=np.float32)
    gate = np.ascontiguousarray(gate_bits, dtype=np.uint16)
    residual = np.ascontiguousarray(residual_bits, dtype=np.uint16).reshape(m, n)
    out = np.empty((m, n), dtype=np.uint16)
    load().sso_epilogue_gated(_p(acc), _p(sa), _p(sw), _p(b) if b is not None else None, _p(gate), _i64(gate.shape[1]),
                              _i64(rows_per_batch), _p(residual), _i64(m), _i64(n), _p(out))
    return out


def obs_compress(weight, upper, dead, scales, group, blocksize=192, joint=True):
    """compress (diffusion_research/reconstruction.py:55-133) on fp32 numpy arrays.  Returns
    qweight int8, zeros bool, compensated fp32, proxy_loss fp32."""
    w = np.array(weight, dtype=np.float32, order="C", copy=True)
    dead = np.asarray(dead, dtype=bool)
    w[:, dead] = 0
    rows, columns = w.shape
    u = np.ascontiguousarray(upper, dtype=np.float32)
    s = np.ascontiguousarray(scales, dtype=np.float32)
    zeros = np.zeros((rows, columns), dtype=np.uint8)
    losses = np.zeros(rows, dtype=np.float32)
    load().sso_obs_compress(_p(w), _i64(rows), _i64(columns), _p(u), _p(s), ctypes.c_int(group),
                            ctypes.c_int(blocksize), ctypes.c_int(1 if joint else 0), _p(zeros), _p(losses))
    zeros = zeros.astype(bool)
    zeros[:, dead] = True
    q = np.clip(np.rint(w / s[:, None]), -128, 127).astype(np.int8)
    q[zeros] = 0
    return q, zeros, w, losses
