"""CPU oracle for the sparse W8A8 projection path -- TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may import
this module; it is the checker, never the thing that ships.  The product path never routes
through it.

Every function restates, in numpy / CPU torch, one step of the reference implementation and
names the reference file:line it follows (paths inside the SlideSparse-Diffusion tree):

  group_size, lifted_k   sdacc/w8a8_slidesparse/packing.py:8-20
  slide_weight           sdacc/w8a8_slidesparse/packing.py:23-52
  pack                   sdacc/w8a8_slidesparse/csrc/dualscale_sm80.cu:254-274 (values, raw words)
  sm80_meta_index        observed permutation of dualscale_sm80.cu:275-278 (cutlass reorder_meta)
  lift_indices           sdacc/w8a8_slidesparse/runtime.py:24-28 and
                         diffusion_research/integrations/cachequant/native_sparse.py:11-23
  quantize_lift          sdacc/w8a8_slidesparse/csrc/projection_sm80.cu:8-88
  gemm_int32             dualscale_sm80.cu:189-204 (int8 x int8 -> int32, never saturates :352)
  epilogue               dualscale_sm80.cu:72-78,123-135 (fma(float(acc), sa*sw, bias) [+addend])
  weight_grid            diffusion_research/reconstruction.py:41-53

Pinning: the reference's tests hold no golden vector for this path; the oracle is pinned
against outputs of the reference's own CPU code run where the reference is mounted
(slide_weight, pack_cpu, activation_indices/lift_integer, channel_scales/round_signed), stored
in tests/golden/ by tests/golden/make_golden.py.  quantize_lift, the contraction and the
epilogue are pinned against outputs of the reference's own GPU operators (quantize, run,
projection), recompiled unmodified for sm_100 and run on a B200 by oracle/ref_gpu.py, stored in
tests/golden/ref_gpu.npz.
"""
import numpy as np
import torch

FORMATS = {"2:4": 4, "4:6": 6, "6:8": 8}


def group_size(mode):
    if isinstance(mode, str):
        if mode in FORMATS:
            return FORMATS[mode]
    elif mode in (4, 6, 8):
        return int(mode)
    raise ValueError("format must be 2:4, 4:6, or 6:8")


def lifted_k(k, mode, alignment=128):
    if k <= 0 or alignment <= 0 or alignment % 4:
        raise ValueError("positive K and a multiple-of-four alignment required")
    l = group_size(mode)
    valid = -(-k // l) * (l // 2 - 1) * 4
    return valid, -(-valid // alignment) * alignment


def slide_weight(qweight, mode):
    """int8 [n,k] -> int8 [n,valid].  Window w of a group sees lanes [2w,2w+4) and keeps the first
    two nonzero lanes no earlier window has taken."""
    w = np.asarray(qweight, dtype=np.int8)
    if w.ndim != 2 or w.size == 0:
        raise ValueError("non-empty [out_features, in_features] int8 weight required")
    n, k = w.shape
    l = group_size(mode)
    groups = np.pad(w, ((0, 0), (0, (-k) % l))).reshape(n, -1, l)
    if (np.count_nonzero(groups, axis=-1) > l - 2).any():
        raise ValueError("weight violates the frozen (L-2):L structure")
    windows = l // 2 - 1
    taken = np.zeros(groups.shape, dtype=bool)
    out = np.zeros((n, groups.shape[1], windows, 4), dtype=np.int8)
    for win in range(windows):
        lo = 2 * win
        vals = groups[..., lo:lo + 4]
        pending = (vals != 0) & ~taken[..., lo:lo + 4]
        keep = pending & (np.cumsum(pending, axis=-1) <= 2)
        out[:, :, win, :] = np.where(keep, vals, 0)
        taken[..., lo:lo + 4] |= keep
    if ((groups != 0) & ~taken).any():
        raise RuntimeError("slide failed to allocate a retained weight")
    return out.reshape(n, -1)


def pack(lifted, pk):
    """int8 [n,kl] -> (packed int8 [pn,pk/2], raw metadata uint32 [pn,pk/32]).

    Per quartet: kept lanes = the nonzero lanes, filled up with the lowest-index zero lanes,
    sorted; nibble = i0 | i1 << 2 at bit 4*(g%8) of word g//8."""
    w = np.asarray(lifted, dtype=np.int8)
    n, kl = w.shape
    if not (n > 0 and kl > 0 and pk >= kl and pk % 128 == 0):
        raise ValueError("invalid 128-K padding")
    pn = -(-n // 32) * 32
    full = np.zeros((pn, pk), dtype=np.int8)
    full[:n, :kl] = w
    quartets = full.reshape(pn, pk // 4, 4)
    nz = quartets != 0
    if (nz.sum(-1) > 2).any():
        raise ValueError("more than 2 nonzeros in a frozen 2:4 group")
    # rank lanes: nonzero lanes first (by index), then zero lanes (by index); keep two, sort
    order = np.argsort(np.where(nz, 0, 4) + np.arange(4), axis=-1, kind="stable")[..., :2]
    order.sort(axis=-1)
    kept = np.take_along_axis(quartets, order, axis=-1)
    packed = kept.reshape(pn, pk // 2)
    nibble = (order[..., 0] | (order[..., 1] << 2)).astype(np.uint32)
    shifts = (4 * (np.arange(pk // 4) % 8)).astype(np.uint32)
    raw = (nibble << shifts).reshape(pn, pk // 32, 8).sum(-1, dtype=np.uint64).astype(np.uint32)
    return packed, raw


def unpack(packed, raw, pk=None):
    """Inverse of pack: dense int8 [pn,pk] from compressed values and raw metadata."""
    packed = np.asarray(packed, dtype=np.int8)
    raw = np.asarray(raw).view(np.uint32).reshape(packed.shape[0], -1)
    pn, half = packed.shape
    pk = 2 * half if pk is None else pk
    nib = (raw[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15
    nib = nib.reshape(pn, pk // 4)
    i0, i1 = nib & 3, nib >> 2
    dense = np.zeros((pn, pk // 4, 4), dtype=np.int8)
    vals = packed.reshape(pn, pk // 4, 2)
    np.put_along_axis(dense, i1[..., None].astype(np.int64), vals[..., 1:2], axis=-1)
    np.put_along_axis(dense, i0[..., None].astype(np.int64), vals[..., 0:1], axis=-1)
    return dense.reshape(pn, pk)


def b200_meta_index(pn, pk):
    """Flat index of raw word (row r, column c) in the layout the B200 GEMM reads: blocks of
    32 rows x 4 words (=128 lifted columns) are contiguous."""
    r = np.arange(pn)[:, None]
    c = np.arange(pk // 32)[None, :]
    return ((r // 32) * (pk // 128) + c // 4) * 128 + (r % 32) * 4 + c % 4


def meta_to_b200(raw, pk):
    raw = np.asarray(raw).view(np.uint32)
    pn = raw.shape[0]
    out = np.empty(pn * pk // 32, dtype=np.uint32)
    out[b200_meta_index(pn, pk).ravel()] = raw.ravel()
    return out


def sm80_meta_index(pn, pk):
    """Flat index of raw word (r,c) after the reference's CUTLASS reorder (SM80 layout)."""
    r = np.arange(pn)[:, None]
    c = np.arange(pk // 32)[None, :]
    return ((c // 2) * (2 * pn) + (r // 32) * 64 + ((r % 32) // 16) * 32 + (r % 8) * 4
            + (c % 2) * 2 + ((r % 16) // 8))


def meta_from_sm80(metadata, pn, pk):
    """Reference-format metadata (flat int32, SM80 order) -> raw uint32 [pn, pk/32]."""
    flat = np.asarray(metadata).view(np.uint32).ravel()
    return flat[sm80_meta_index(pn, pk)]


def lift_indices(k, mode):
    """Source column of every lifted column (k = sentinel for tail lanes, reads as zero)."""
    l = group_size(mode)
    valid, _ = lifted_k(k, l)
    c = np.arange(valid)
    windows = l // 2 - 1
    src = (c // (4 * windows)) * l + 2 * ((c // 4) % windows) + c % 4
    return np.minimum(src, k)


def _bf16_to_f32(x):
    if isinstance(x, torch.Tensor):
        if x.dtype != torch.bfloat16:
            raise TypeError("BF16 input required")
        return x.detach().cpu().float().numpy()
    return np.asarray(x, dtype=np.float32)


def quantize_lift(x, mode):
    """BF16 [m,k] -> (q int8 [pm,pk], sa fp32 [pm]).

    absmax with fmaxf (NaN operands ignored, start 0); scale = max(max(a,1e-12)/127, 1/(127*512));
    inv = 1/scale; b = rint(clamp(x*inv, -128, 127)) with NaN -> -128; rows m..pm-1: q=0, sa=1."""
    xf = _bf16_to_f32(x)
    m, k = xf.shape
    l = group_size(mode)
    valid, pk = lifted_k(k, l)
    pm = -(-m // 32) * 32
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        a = np.abs(xf)
        a = np.where(np.isnan(a), np.float32(0), a).max(axis=1).astype(np.float32)
        floor = np.float32(1.0) / (np.float32(127.0) * np.float32(512.0))
        scale = np.maximum(np.maximum(a, np.float32(1e-12)) / np.float32(127.0), floor).astype(np.float32)
        inv = (np.float32(1.0) / scale).astype(np.float32)
        y = (xf * inv[:, None]).astype(np.float32)
        y = np.where(np.isnan(y), np.float32(-128.0), np.clip(y, np.float32(-128.0), np.float32(127.0)))
        b = np.rint(y).astype(np.int8)                        # round-half-even
    src = lift_indices(k, l)
    padded = np.concatenate([b, np.zeros((m, 1), np.int8)], axis=1)
    q = np.zeros((pm, pk), dtype=np.int8)
    q[:m, :valid] = padded[:, src]
    sa = np.ones(pm, dtype=np.float32)
    sa[:m] = scale
    return q, sa


# ---- fused front-end prologues (an extension of this build; the reference has no counterpart) ----
# LayerNorm + modulation: the GPU kernel uses separately rounded fp32 operations in a fixed order,
# restated here operation for operation (numpy float32 arithmetic is IEEE round-to-nearest like the
# device's __fadd_rn / __fmul_rn / __fdiv_rn / __fsqrt_rn), so parity is bit-exact.  GELU: see below.

def _f32(v):
    return np.float32(v)


def _bf16_round_f32(y):
    """fp32 -> nearest-even BF16, returned as fp32 values."""
    return torch.from_numpy(np.ascontiguousarray(y, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def prologue_gelu(x):
    """BF16 [m,k] -> gelu_tanh(x) = x * sigmoid(2 sqrt(2/pi) (x + 0.044715 x^3)) in fp32, rounded to
    BF16 (fp32 values).  The GPU uses the hardware tanh approximation (relative error 2^-11), so
    parity of this prologue is within floating-point tolerance: |error| <= 2.5e-4 |x| before the
    BF16 rounding."""
    xf = _bf16_to_f32(x)
    with np.errstate(invalid="ignore", over="ignore"):
        x2 = (xf * xf).astype(np.float32)
        u2 = (xf * (_f32(1.5957691216057308) + _f32(0.07135481627260025) * x2).astype(np.float32)).astype(np.float32)
        sig = (_f32(1.0) / (_f32(1.0) + np.exp(-u2, dtype=np.float32)).astype(np.float32)).astype(np.float32)
        y = (xf * sig).astype(np.float32)
    return _bf16_round_f32(y)


def frontend_threads(k, mode):
    """(threads per row, 16-byte vectors per chunk, chunks per thread) of the front-end kernel."""
    l = group_size(mode)
    cv = {4: 2, 6: 3, 8: 4}[l]
    ow = {4: 4, 6: 8, 8: 12}[l]
    per_thread = 8 // cv
    _, pk = lifted_k(k, l)
    nvec = -(-k // 8)
    chunks = max(-(-nvec // cv), -(-(pk // 4) // ow))
    threads = -(-(-(-chunks // per_thread)) // 32) * 32       # a multiple of 32 that covers the chunks
    return threads, cv, per_thread


def _block_sum(values, valid, threads, cv, per_thread):
    """Row sums in the kernel's order: each thread adds its elements sequentially (chunk i, vector c,
    element 0..7 at vector index (t + i*threads)*cv + c), lanes combine by xor butterfly 16..1, then
    the warp totals combine the same way.  values: fp32 [m, nvec*8]; valid: element mask or None."""
    m, width = values.shape
    nvec = width // 8
    part = np.zeros((m, threads), dtype=np.float32)
    t = np.arange(threads)
    for i in range(per_thread):
        for c in range(cv):
            idx = (t + i * threads) * cv + c
            ok = idx < nvec
            cols = np.where(ok, idx, 0) * 8
            for e in range(8):
                add = np.where(ok[None, :], values[:, cols + e], _f32(0.0)).astype(np.float32)
                if valid is not None:
                    add = np.where(valid[cols + e][None, :], add, _f32(0.0))
                part = (part + add).astype(np.float32)
    warps = threads // 32
    lanes = part.reshape(m, warps, 32)
    lane = np.arange(32)
    for d in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[:, :, lane ^ d]).astype(np.float32)
    totals = np.zeros((m, 32), dtype=np.float32)
    totals[:, :warps] = lanes[:, :, 0]
    for d in (16, 8, 4, 2, 1):
        totals = (totals + totals[:, lane ^ d]).astype(np.float32)
    return totals[:, 0]


def prologue_norm_modulate(x, shift, scale, rows_per_batch, eps, mode):
    """BF16 [m,k] -> ((x - mean) * rstd) * (1 + scale[b]) + shift[b], b = row // rows_per_batch,
    rounded to BF16 (fp32 values).  mean and biased variance are block sums in the kernel's order
    (which depends on the mode through the thread layout); rstd = 1 / sqrt(var + eps)."""
    xf = _bf16_to_f32(x)
    m, k = xf.shape
    if k % 8:
        raise ValueError("k % 8 == 0 required")
    sh, sc = _bf16_to_f32(shift), _bf16_to_f32(scale)
    threads, cv, per_thread = frontend_threads(k, mode)
    kf = _f32(k)
    mean = (_block_sum(xf, None, threads, cv, per_thread) / kf).astype(np.float32)
    dev = (xf - mean[:, None]).astype(np.float32)
    var = (_block_sum((dev * dev).astype(np.float32), None, threads, cv, per_thread) / kf).astype(np.float32)
    rstd = (_f32(1.0) / np.sqrt((var + _f32(eps)).astype(np.float32)).astype(np.float32)).astype(np.float32)
    b = np.arange(m) // rows_per_batch
    y = (dev * rstd[:, None]).astype(np.float32)
    y = (y * (_f32(1.0) + sc[b]).astype(np.float32)).astype(np.float32)
    y = (y + sh[b]).astype(np.float32)
    return _bf16_round_f32(y)


def quantize_lift_fused(x, mode, prologue, shift=None, scale=None, rows_per_batch=1, eps=1e-6):
    """The fused front-end: prologue ('gelu' | 'norm_modulate' | None), then quantize_lift."""
    if prologue == "gelu":
        y = prologue_gelu(x)
    elif prologue == "norm_modulate":
        y = prologue_norm_modulate(x, shift, scale, rows_per_batch, eps, mode)
    else:
        return quantize_lift(x, mode)
    return quantize_lift(torch.from_numpy(y).to(torch.bfloat16), mode)


def gemm_int32(q, lifted, m=None):
    """acc[m,n] = q[:m] . lifted^T in exact int32 (lifted: [n,kl], kl <= pk)."""
    q = np.asarray(q, dtype=np.int8)
    w = np.asarray(lifted, dtype=np.int8)
    m = q.shape[0] if m is None else m
    qt = torch.from_numpy(np.ascontiguousarray(q[:m, :w.shape[1]])).to(torch.int32)
    wt = torch.from_numpy(np.ascontiguousarray(w)).to(torch.int32)
    return (qt @ wt.T).numpy()


def round_bf16(x32):
    """fp32 -> BF16 bit patterns (uint16), round-to-nearest-even (cvt.rn.bf16.f32)."""
    return torch.from_numpy(np.ascontiguousarray(x32, dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def epilogue(acc, sa, sw, bias=None, addend=None):
    """BF16 bit patterns of fma(float(acc), sa[m]*sw[n], bias[n]) (+ float(addend)).

    The fused multiply-add is evaluated in float64: float(acc) and sa*sw are fp32, so their
    product is exact in float64; adding the bias and rounding once to fp32 differs from a true
    fp32 FMA only in double-rounding corner cases, which the C oracle (fmaf) settles."""
    acc = np.asarray(acc)
    m, n = acc.shape
    scale = (np.asarray(sa, np.float32)[:m, None] * np.asarray(sw, np.float32)[None, :n]).astype(np.float32)
    prod = acc.astype(np.float32).astype(np.float64) * scale.astype(np.float64)
    if bias is not None and np.size(bias):
        prod = prod + np.asarray(bias, np.float32)[None, :n].astype(np.float64)
    y = prod.astype(np.float32)
    if addend is not None:
        y = (y + _bf16_to_f32(addend)[:m, :n]).astype(np.float32)
    return round_bf16(y)


def channel_scales(weight):
    """scale = 2*rowabsmax/255, 1 for an all-zero row (reconstruction.py:41-49)."""
    mx = np.abs(np.asarray(weight, dtype=np.float32)).max(axis=1)
    return np.where(mx > 0, (np.float32(2.0) * mx / np.float32(255.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)


def weight_grid(weight):
    """fp32 [n,k] -> (int8 [n,k], fp32 scales [n]): scale = 2*rowabsmax/255 (1 if zero)."""
    w = np.asarray(weight, dtype=np.float32)
    scales = channel_scales(w)
    q = np.clip(np.rint((w / scales[:, None]).astype(np.float32)), -128, 127).astype(np.int8)
    return q, scales


def magnitude_prune(weight, mode):
    """Zero the 2 smallest-|w| lanes of every aligned group of l (ties -> lowest index); lanes
    missing from a tail group count as already zero.  Synthetic stand-in for the reference's
    OBS pruner; its tail rule is diffusion_research/reconstruction.py:96-101."""
    w = np.array(weight, dtype=np.float32, copy=True)
    n, k = w.shape
    l = group_size(mode)
    pad = (-k) % l
    g = np.pad(np.abs(w), ((0, 0), (0, pad)), constant_values=-1.0).reshape(n, -1, l)
    mask = np.zeros(g.shape, dtype=bool)
    for _ in range(2):                      # argmin returns the lowest index among ties
        first = np.argmin(g, axis=-1)[..., None]
        np.put_along_axis(mask, first, True, axis=-1)
        np.put_along_axis(g, first, np.float32(np.inf), axis=-1)
    mask = mask.reshape(n, -1)[:, :k]
    w[mask] = 0
    return w, mask


def make_weight(n, k, mode, seed=0, std=0.02):
    """Seeded synthetic weight: N(0,std) BF16 values, magnitude-pruned, per-channel INT8.
    Returns (qweight int8 [n,k], scales fp32 [n])."""
    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=gen) * std).to(torch.bfloat16).float().numpy()
    scales = channel_scales(w)
    pruned, mask = magnitude_prune(w, mode)
    q = np.clip(np.rint((pruned / scales[:, None]).astype(np.float32)), -128, 127).astype(np.int8)
    q[mask] = 0
    return q, scales


def make_activation(m, k, seed=0, outlier_fraction=0.01, outlier_gain=20.0):
    """Seeded synthetic activation: N(0,1) with round(fraction*k) channels scaled, BF16."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen)
    count = int(round(outlier_fraction * k))
    if count:
        cols = torch.randperm(k, generator=gen)[:count]
        x[:, cols] *= outlier_gain
    return x.to(torch.bfloat16)


def projection(x, qweight, scales, bias, mode, addend=None):
    """Full path on the CPU: returns dict(q, sa, lifted, packed, raw, acc, out_bits)."""
    l = group_size(mode)
    k = qweight.shape[1]
    _, pk = lifted_k(k, l)
    lifted = slide_weight(qweight, l)
    packed, raw = pack(lifted, pk)
    q, sa = quantize_lift(x, l)
    m = x.shape[0]
    acc = gemm_int32(q, lifted, m)
    out = epilogue(acc, sa, scales, bias, addend)
    return dict(q=q, sa=sa, lifted=lifted, packed=packed, raw=raw, acc=acc, out_bits=out)
