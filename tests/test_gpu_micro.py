"""The MMA-rate micro-benchmark runs and shows the bound it exists to show."""
import pytest

pytestmark = pytest.mark.gpu


def test_sparse_mma_is_operand_bound_dense_is_not(backend):
    import torch
    torch.zeros(1, device="cuda")
    dense = backend.micro_mma_rate(256, sparse=False)
    sparse = backend.micro_mma_rate(256, sparse=True)
    # tensor-pipe time of either instruction is 128 cycles; the sparse one reads 20 KB of operands
    assert 120 <= dense <= 150, dense
    assert sparse >= 1.15 * dense, (sparse, dense)
    assert (128 * 32 + 256 * 64) / sparse <= 135.0            # bytes per cycle: the shared-memory read limit
    with pytest.raises(ValueError):
        backend.micro_mma_rate(100)
    assert backend.device_status(torch.device("cuda", 0)) == 0
