"""Shape dispatch interface of the reference (`sdacc/w8a8_slidesparse/profile.py:5-10`).

The reference maps (mode, M, K, N) to one of its SM80 tile configurations and front-ends from a
frozen table measured on A100.  Neither notion exists on sm_100a: there is one front-end and the
GEMM picks its own token tile from the problem size.  The two functions keep their signatures and
the reference's default answer so callers that unpack `(config, frontend)` keep working.
"""
DEFAULT = (5, "native")


def execution_profile(mode, m, k, n):
    """(config, frontend) for a shape; the same single backend for every shape."""
    return DEFAULT


def known_configurations(mode, k, n):
    return [DEFAULT[0]]


def selectable(mode, m, k, n):
    """Whether the sparse operator is worth using for this shape on a B200.

    The reference marks shapes it keeps dense in its inventory (`workloads/__init__.py:17`,
    "keep Dense"); here the rule comes from the per-shape measurements against BF16 `F.linear`
    (bench.py --workload shapes): projections of less than about 8 GOP are launch-latency sized
    (PixArt cross-KV at 600 text rows: 10.5 us sparse, 6.6 us dense), and square hidden-sized
    projections with no element-wise neighbour to absorb (cross-attention Q, 1152 -> 1152) pay
    more for the quantising front-end than the sparse GEMM saves."""
    if 2.0 * m * n * k < 8e9:
        return False
    if k <= 1536 and n <= 1536:
        return False
    return True
