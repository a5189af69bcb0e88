"""Column-sharded and tensor-parallel use of the projection on two CPU ranks (gloo).

The kernels need a GPU, so each rank stands in for its shard's operator with the CPU oracle fed
from the shard's own packed buffers (values + metadata as the GPU would read them); the test
checks the sharding arithmetic, the packing of shards, and the gather."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from __graft_entry__ import load_oracle, load_package
        sdk = load_package()
        sdk.load_native()
        oracle, _ = load_oracle()
        from slidesparse_diffusion_b200 import importer, sharding

        m, k, n, mode = 40, 132, 200, 6
        qweight, scales = oracle.make_weight(n, k, mode, seed=5)
        bias = np.linspace(-1, 1, n).astype(np.float32)
        x = oracle.make_activation(m, k, seed=6)
        full = oracle.projection(x, qweight, scales, bias, mode)

        shard, (start, end) = sharding.prepare_shard(torch.from_numpy(qweight), torch.from_numpy(scales),
                                                     torch.from_numpy(bias), mode, rank, world)
        bounds = sharding.shard_columns(n, world)
        assert bounds[rank] == (start, end) and shard.n == end - start

        class OracleShard(torch.nn.Module):
            """Same call contract as PackedLinear.forward, arithmetic from the shard's buffers."""
            def forward(self, inp, output_addend=None):
                _, pk = oracle.lifted_k(k, mode)
                raw = importer.b200_metadata_to_raw(shard.metadata, shard.packed.shape[0], pk).numpy().view(np.uint32)
                dense = oracle.unpack(shard.packed.numpy(), raw)[:shard.n]
                q, sa = oracle.quantize_lift(inp, mode)
                acc = oracle.gemm_int32(q, dense, m)
                add = None if output_addend is None else output_addend
                bits = oracle.epilogue(acc, sa, shard.scales.numpy(), shard.bias.numpy(), add)
                return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)

        tp = sharding.TensorParallelProjection(OracleShard(), bounds)
        y = tp(x)
        assert y.shape == (m, n)
        got = y.view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got, full["out_bits"]), "gathered shards differ from the unsharded projection"

        # the collective's own layout: [world, m, widest], rank r's columns in slot r
        shards = tp(x, layout="shards")
        widest = max(e - b for b, e in bounds)
        assert shards.shape == (world, m, widest)
        for r, (b, e) in enumerate(bounds):
            assert np.array_equal(shards[r][:, :e - b].contiguous().view(torch.int16).numpy().view(np.uint16),
                                  full["out_bits"][:, b:e])

        addend = (torch.arange(m * n, dtype=torch.float32).reshape(m, n) / 997).to(torch.bfloat16)
        y2 = tp(x, output_addend=addend)
        expect = oracle.epilogue(full["acc"], full["sa"], scales, bias, addend)
        assert np.array_equal(y2.view(torch.int16).numpy().view(np.uint16), expect)
        results[rank] = "ok"
    except Exception as e:            # noqa: BLE001 - reported to the parent
        results[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_two_rank_column_shards_match_unsharded(sdk, oracle):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_shard_columns_properties(sdk):
    from slidesparse_diffusion_b200 import sharding
    for n, world in ((9216, 8), (3456, 4), (200, 2), (96, 8), (33, 2), (12288, 3)):
        bounds = sharding.shard_columns(n, world)
        assert len(bounds) == world and bounds[0][0] == 0 and bounds[-1][1] == n
        for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
            assert a1 == b0 and a0 <= a1
        assert all(start % 32 == 0 for start, _ in bounds)
        widths = [e - s for s, e in bounds]
        assert max(widths) <= (-(-(-(-n // 32)) // world)) * 32          # no rank above ceil(units/world)
    with pytest.raises(ValueError):
        sharding.shard_columns(0, 2)
    with pytest.raises(ValueError):
        sharding.shard_columns(96, 2, members=[32, 32])
