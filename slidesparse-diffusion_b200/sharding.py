"""Multi-GPU use of the projection: output-channel column shards, one process per GPU.

The reference is single-GPU (it refuses anything else, `sdacc/diffusion_research/runner.py:13-18`).
The projection shards naturally along output channels: rank g packs and keeps only rows
[start_g, end_g) of the quantised weight (with the matching scales and bias), every rank
quantises the full activation itself, and no data moves between GPUs.  Where a caller needs the
full [M, N] output on every rank (tensor-parallel use inside a model) the shards are gathered
with one NCCL all-gather over NVLink.
"""
import torch
import torch.distributed as dist

from .packing import group_size
from .runtime import PackedLinear


def shard_columns(n, world, members=None, align=32):
    """[(start, end)] per rank: contiguous channel ranges with `align`-aligned starts that never
    overlap and together cover [0, n).  Trailing ranks may be empty when n is small.  `members`
    (widths of a fused projection such as Q|K|V) is only checked for consistency: a fused output
    is split by widths after the gather, so member boundaries need not coincide with ranks."""
    if world <= 0 or n <= 0:
        raise ValueError("positive channel count and world size required")
    if members is not None and sum(members) != n:
        raise ValueError("member widths must add up to n")
    units = -(-n // align)
    base, extra = divmod(units, world)
    bounds, start = [], 0
    for rank in range(world):
        width = (base + (1 if rank < extra else 0)) * align
        end = min(n, start + width)
        bounds.append((start, end))
        start = end
    return bounds


def prepare_shard(qweight, scales, bias, mode, rank, world, members=None, **kwargs):
    """PackedLinear for this rank's channel range of a full CPU int8 weight; also returns the range."""
    n = qweight.shape[0]
    start, end = shard_columns(n, world, members)[rank]
    if end <= start:
        raise ValueError(f"rank {rank} of {world} owns no channels of a {n}-channel projection")
    shard_bias = None if bias is None or bias.numel() == 0 else bias[start:end]
    op = PackedLinear.prepare(qweight[start:end].contiguous(), scales[start:end], shard_bias,
                              group_size(mode), **kwargs)
    return op, (start, end)


def gather_shards(local, bounds, group=None):
    """One all-gather of this rank's [..., n_rank] shard: returns `[world, ..., widest]`, rank r's
    shard in slot r (columns beyond its width are padding when the shards are ragged).  With equal
    widths the collective reads the projection's output and writes the result tensor directly: no
    staging copy on either side."""
    world = dist.get_world_size(group)
    if len(bounds) != world:
        raise ValueError("one channel range per rank required")
    widest = max(end - start for start, end in bounds)
    send = local
    if local.shape[-1] != widest:
        send = local.new_zeros((*local.shape[:-1], widest))
        send[..., :local.shape[-1]] = local
    send = send.contiguous()
    if dist.get_backend(group) == "nccl":
        gathered = local.new_empty((world, *send.shape))
        dist.all_gather_into_tensor(gathered, send, group=group)
        return gathered
    parts = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(parts, send, group=group)
    return torch.stack(parts)


def all_gather_columns(local, bounds, group=None):
    """Gather [..., n_rank] shards into one row-major [..., n] tensor on every rank: the all-gather
    of `gather_shards` plus ONE re-ordering copy (shard-major -> row-major)."""
    gathered = gather_shards(local, bounds, group)
    widths = [end - start for start, end in bounds]
    world, widest = gathered.shape[0], gathered.shape[-1]
    if all(w == widest for w in widths):
        return gathered.movedim(0, -2).reshape(*gathered.shape[1:-1], world * widest)
    return torch.cat([gathered[r][..., :widths[r]] for r in range(world)], dim=-1)


class TensorParallelProjection(torch.nn.Module):
    """N-split tensor-parallel projection: local column shard + one NCCL all-gather of the BF16 outputs.

    `layout="rows"` (default) returns the row-major [..., N] tensor a dense layer would (one extra
    copy after the collective).  `layout="shards"` returns the collective's own result
    [world, ..., N / world] without that copy: the natural form for a consumer that splits the
    channels anyway (attention heads: shard r holds heads r * H / world ...), and what the N-split
    variant costs at its best with NCCL."""

    def __init__(self, shard, bounds, group=None):
        super().__init__()
        self.shard, self.bounds, self.group = shard, list(bounds), group
        self.n = self.bounds[-1][1]

    def forward(self, x, output_addend=None, layout="rows"):
        if layout not in ("rows", "shards"):
            raise ValueError("layout is 'rows' or 'shards'")
        rank = dist.get_rank(self.group)
        start, end = self.bounds[rank]
        addend = None if output_addend is None else output_addend[..., start:end]
        local = self.shard(x) if addend is None else self.shard(x, output_addend=addend)
        if layout == "shards":
            return gather_shards(local, self.bounds, self.group)
        return all_gather_columns(local, self.bounds, self.group)


class FusedTensorParallelProjection(torch.nn.Module):
    """N-split tensor-parallel projection whose all-gather happens inside the GEMM epilogue.

    Every rank's gathered [m, N] output lives in symmetric memory (mapped into every process of
    the group); a rank's kernel stores each tile of its column shard into all of them with plain TMA
    stores over NVLink while the remaining tiles are still being computed, instead of running a
    collective afterwards.  Two cross-GPU barriers frame the launch: before it nobody may still be
    reading the buffers of the previous call, after it every shard has landed everywhere."""

    def __init__(self, shard, bounds, group=None):
        super().__init__()
        self.shard, self.bounds = shard, list(bounds)
        self.group = dist.group.WORLD if group is None else group
        self.n = self.bounds[-1][1]
        if self.n % 8:
            raise ValueError("the gathered width must be a multiple of 8 (16-byte row pitch)")
        self._buffers = {}

    def _buffer(self, rows, device):
        import torch.distributed._symmetric_memory as symm_mem
        if rows not in self._buffers:
            out = symm_mem.empty((rows, self.n), dtype=torch.bfloat16, device=device)
            self._buffers[rows] = (out, symm_mem.rendezvous(out, self.group))
        return self._buffers[rows]

    def forward(self, x):
        from . import backend
        if x.ndim != 2:
            raise ValueError("[m, k] input required")
        rank = dist.get_rank(self.group)
        start, end = self.bounds[rank]
        out, handle = self._buffer(x.shape[0], x.device)
        destinations = [int(p) + 2 * start for p in handle.buffer_ptrs]
        handle.barrier()
        backend.projection_peers(x, self.shard.packed, self.shard.metadata, self.shard.scales, self.shard.bias,
                                 self.shard.mode, end - start, destinations, self.n)
        handle.barrier()
        return out
