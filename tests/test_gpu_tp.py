"""N-split tensor-parallel projection on two or more GPUs: the NCCL all-gather variant and the
variant whose gather is done by the GEMM epilogue's stores into every rank's output buffer."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from __graft_entry__ import load_oracle, load_package
        sdk = load_package()
        sdk.load_native()
        oracle, _ = load_oracle()
        from slidesparse_diffusion_b200 import sharding
        m, k, n, mode = 700, 640, 1504, 6
        qweight, scales = oracle.make_weight(n, k, mode, seed=5)
        bias = np.linspace(-1, 1, n).astype(np.float32)
        x = oracle.make_activation(m, k, seed=6)
        expect = oracle.projection(x, qweight, scales, bias, mode)["out_bits"]
        shard, _ = sharding.prepare_shard(torch.from_numpy(qweight), torch.from_numpy(scales),
                                          torch.from_numpy(bias), mode, rank, world)
        bounds = sharding.shard_columns(n, world)
        shard = shard.to(device)
        xd = x.to(device)
        gathered = sharding.TensorParallelProjection(shard, bounds)(xd)
        fused_op = sharding.FusedTensorParallelProjection(shard, bounds)
        fused = fused_op(xd).clone()
        again = fused_op(xd).clone()                      # the buffers are re-used between calls
        torch.cuda.synchronize()
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(bits(gathered), expect), "NCCL all-gather variant differs from the oracle"
        assert np.array_equal(bits(fused), expect), "fused store variant differs from the oracle"
        assert np.array_equal(bits(again), expect)
        import slidesparse_diffusion_b200.backend as backend
        assert backend.device_status(device) == 0
        results[rank] = "ok"
    except Exception as e:            # noqa: BLE001 - reported to the parent
        results[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_variants_match_the_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    manager = mp.Manager()
    results = manager.dict()
    port = 29600 + os.getpid() % 1000
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {rank: "ok" for rank in range(world)}
