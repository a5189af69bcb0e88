"""Importer for operator payloads written by the reference implementation.

The reference stores `metadata` in the order its SM80 kernel reads (CUTLASS `reorder_meta`,
csrc/dualscale_sm80.cu:275-278).  `packed`, `scales` and `bias` are layout-free and carry over
unchanged; only the metadata words are permuted into the order the sm_100a GEMM reads.
"""
import torch


def sm80_flat_index(pn, pk):
    """Flat position, in the reference's metadata tensor, of raw word (row r, column c)."""
    r = torch.arange(pn, dtype=torch.int64)[:, None]
    c = torch.arange(pk // 32, dtype=torch.int64)[None, :]
    return ((c // 2) * (2 * pn) + (r // 32) * 64 + ((r % 32) // 16) * 32 + (r % 8) * 4
            + (c % 2) * 2 + ((r % 16) // 8))


def b200_flat_index(pn, pk):
    """Flat position, in this library's metadata tensor, of raw word (row r, column c)."""
    r = torch.arange(pn, dtype=torch.int64)[:, None]
    c = torch.arange(pk // 32, dtype=torch.int64)[None, :]
    return ((r // 32) * (pk // 128) + c // 4) * 128 + (r % 32) * 4 + c % 4


def sm80_metadata_to_raw(metadata, pn, pk):
    flat = metadata.detach().cpu().contiguous().view(torch.int32).reshape(-1)
    if pn % 32 or pk % 128 or flat.numel() != pn * pk // 32:
        raise ValueError("metadata size does not match [pn, pk/32]")
    return flat[sm80_flat_index(pn, pk)]


def raw_metadata_to_b200(raw, pk):
    raw = raw.detach().cpu().contiguous().view(torch.int32)
    pn = raw.shape[0]
    out = torch.empty(pn * pk // 32, dtype=torch.int32)
    out[b200_flat_index(pn, pk).reshape(-1)] = raw.reshape(-1)
    return out


def b200_metadata_to_raw(metadata, pn, pk):
    flat = metadata.detach().cpu().contiguous().view(torch.int32).reshape(-1)
    return flat[b200_flat_index(pn, pk)]


def sm80_metadata_to_b200(metadata, pn, pk):
    return raw_metadata_to_b200(sm80_metadata_to_raw(metadata, pn, pk), pk)


def import_reference_bank(compact, metadata, scales, bias, k, n, mode, **kwargs):
    """Build a PackedLinear from a reference bank triple (`compact`, `metadata`, `scales`)."""
    from .packing import lifted_k
    from .runtime import PackedLinear, LAYOUT, kernel_source_sha
    _, pk = lifted_k(k, mode)
    pn = compact.shape[0]
    if compact.shape[1] * 2 != pk:
        raise ValueError("compact width does not match the lifted K of this mode")
    meta = sm80_metadata_to_b200(metadata, pn, pk)
    identity = dict(k_physical=pk, kernel_source_sha=kernel_source_sha(), metadata_layout=LAYOUT,
                    imported_from="reference-bank")
    bias = torch.empty(0, dtype=torch.float32) if bias is None else bias.detach().float().contiguous()
    return PackedLinear(compact.detach().contiguous(), meta, scales.detach().float().contiguous(), bias,
                        k, n, mode, identity=identity, **kwargs)
