"""Host-side restatement of the arithmetic of the GEMM's split schedule (`Walk<true>` and the epilogue
of `slidesparse-diffusion_b200/csrc/ss_gemm_pair.cuh`): the launch's tiles x stages are cut into one
contiguous range per cluster, and a piece of a shared tile names the tile's first cluster (`owner`)
and the number of clusters that share it (`pieces`) with closed forms instead of a search.  The
device code cannot run here; what can be checked on the CPU is that those closed forms say what the
ranges say, for every size the launcher may produce."""
import random


def ranges(total, clusters):
    return [(c * total // clusters, (c + 1) * total // clusters) for c in range(clusters)]


def pieces_of(lo, hi, num_st):
    """The (tile, s0, s1) pieces of the range [lo, hi), in order (Walk<true>::decode / advance)."""
    out, pos = [], lo
    while pos < hi:
        tile = pos // num_st
        s0 = pos - tile * num_st
        s1 = min(num_st, s0 + (hi - pos))
        out.append((tile, s0, s1))
        pos += s1 - s0
    return out


def owner_and_pieces(tile, num_st, total, clusters):
    first = tile * num_st
    owner = ((first + 1) * clusters + total - 1) // total - 1
    pieces = ((first + num_st) * clusters + total - 1) // total - owner
    return owner, pieces


def check(num_tiles, num_st, clusters):
    total = num_tiles * num_st
    clusters = min(clusters, total)              # the launcher never starts more clusters than stages
    sharers = {}
    covered = 0
    for c, (lo, hi) in enumerate(ranges(total, clusters)):
        assert hi > lo, "every cluster has work"
        heads = tails = 0
        for i, (tile, s0, s1) in enumerate(pieces_of(lo, hi, num_st)):
            covered += s1 - s0
            whole = s0 == 0 and s1 == num_st
            if not whole:
                sharers.setdefault(tile, []).append(c)
                if s0 == 0:
                    heads += 1
                    assert (tile, s0, s1) == pieces_of(lo, hi, num_st)[-1], "a piece that starts a tile ends the range"
                else:
                    tails += 1
                    assert i == 0, "a piece that does not start its tile starts the range"
        assert heads <= 1 and tails <= 1, "two slabs per cluster are enough"
    assert covered == total
    for tile, who in sharers.items():
        owner, pieces = owner_and_pieces(tile, num_st, total, clusters)
        assert who == list(range(owner, owner + pieces)), (tile, who, owner, pieces)
        assert pieces >= 2


def test_closed_forms_match_the_ranges_exhaustive_small():
    for num_tiles in range(1, 40):
        for num_st in range(2, 12):
            for clusters in (1, 2, 3, 7, 16, 74):
                check(num_tiles, num_st, clusters)


def test_closed_forms_match_the_ranges_benchmark_sizes():
    rng = random.Random(5)
    sizes = [(100, 51, 74), (87, 13, 74), (12, 64, 74), (3312, 18, 74), (648, 16, 74), (342, 5, 74)]
    sizes += [(rng.randrange(1, 5000), rng.randrange(2, 130), 74) for _ in range(200)]
    for num_tiles, num_st, clusters in sizes:
        check(num_tiles, num_st, clusters)
