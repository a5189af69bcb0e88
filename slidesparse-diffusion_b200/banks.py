"""Per-unit storage of the packed modes a denoiser switches between from step to step.

Counterpart of the reference's bank slots (`sdacc/diffusion_research/banks.py`: `ResidentBankSlot`
:30-67, `coalesce_parameters` :106-127); its memory-budget helpers for 40-80 GB parts (:69-81) have
no use on a 180 GB GPU and are not carried.
A unit (one routed projection group) has up to three prepared payloads, one per sparsity mode, each
a dict of `packed`, `metadata`, `scales`, `bias`.  The operators are built over VIEWS of the slot's
device buffers, and the kernels read those pointers at launch time, so a mode switch or an in-place
update of scales/bias needs no new operator.

Two residency policies:
  "active"  one device buffer per tensor kind, sized for the largest mode; `activate(mode)` copies
            that mode's payload from pinned host memory into it (the reference's behaviour, made
            for 40-80 GB parts; the copy belongs inside the timed selection).
  "all"     every mode has its own device buffers and `activate` moves no bytes.  With 180 GB of
            HBM per GPU all three modes of every configuration in this repository fit
            (FLUX: about 22 GB for 4:6 + 6:8 + 2:4 together), so this is the default.
"""
import torch

KEYS = ("packed", "metadata", "scales", "bias")
_DTYPES = {"packed": torch.int8, "metadata": torch.int32, "scales": torch.float32, "bias": torch.float32}


def _check_payloads(payloads):
    """A slot takes {4|6|8: {packed, metadata, scales, bias}} of contiguous CPU tensors."""
    if not payloads:
        raise ValueError("a bank slot needs at least one mode")
    for mode, values in payloads.items():
        if type(mode) is not int or mode not in (4, 6, 8):
            raise ValueError(f"bank modes are the group sizes 4, 6 and 8, not {mode!r}")
        missing, extra = set(KEYS) - set(values), set(values) - set(KEYS)
        if missing or extra:
            raise ValueError(f"mode {mode}: payload must hold exactly {KEYS} (missing {sorted(missing)}, extra {sorted(extra)})")
        for key in KEYS:
            value = values[key]
            if value.device.type != "cpu" or not value.is_contiguous():
                raise ValueError(f"mode {mode}: {key} must be a contiguous CPU tensor (payloads are staged from the host)")
            if value.dtype != _DTYPES[key]:
                raise ValueError(f"mode {mode}: {key} must be {_DTYPES[key]}, got {value.dtype}")
        for key in ("scales", "bias"):
            if not bool(torch.isfinite(values[key]).all()):
                raise ValueError(f"mode {mode}: {key} holds a non-finite value")


class ResidentBankSlot:
    """Device storage + pinned host copies of one unit's packed modes."""

    def __init__(self, payloads, device, residency="all"):
        if residency not in ("all", "active"):
            raise ValueError("residency is 'all' or 'active'")
        _check_payloads(payloads)
        self.device = torch.device(device)
        self.residency = residency
        self.current_mode = None
        self.transfer_bytes = 0
        self.transfers = 0
        pin = self.device.type == "cuda"
        self.host = {mode: {key: (value.pin_memory() if pin and not value.is_pinned() else value)
                            for key, value in values.items()} for mode, values in payloads.items()}
        self.buffers, self.views = {}, {}
        if residency == "active":
            for key in KEYS:
                size = max(row[key].numel() for row in self.host.values())
                self.buffers[key] = torch.empty(size, dtype=_DTYPES[key], device=self.device)
            for mode, values in self.host.items():
                self.views[mode] = {key: self.buffers[key][:value.numel()].view(value.shape)
                                    for key, value in values.items()}
        else:
            for mode, values in self.host.items():
                self.views[mode] = {key: value.to(self.device, non_blocking=pin) for key, value in values.items()}
                for key, value in self.views[mode].items():
                    self.buffers[(mode, key)] = value
        self.identity = dict(
            payload_shapes={str(m): {k: list(v.shape) for k, v in row.items()} for m, row in self.host.items()},
            device_bytes=self.device_bytes, pinned_host=pin, residency=residency,
            copies_on_activate=residency == "active")

    @property
    def device_bytes(self):
        """Bytes this slot keeps on the device: every mode ("all"), or per tensor kind the largest
        mode ("active")."""
        return sum(v.numel() * v.element_size() for v in self.buffers.values())

    def activate(self, mode, include_parameters=True):
        """Make `mode` the one whose operator may run; returns the bytes copied to the device."""
        if type(mode) is not int or mode not in self.host:
            raise ValueError(f"this slot holds modes {sorted(self.host)}, not {mode!r}")
        if mode == self.current_mode:
            return 0
        copied = 0
        if self.residency == "active":
            for key in (KEYS if include_parameters else ("packed", "metadata")):
                source = self.host[mode][key]
                self.views[mode][key].copy_(source, non_blocking=self.device.type == "cuda")
                copied += source.numel() * source.element_size()
            self.transfer_bytes += copied
            self.transfers += 1
        self.current_mode = mode
        return copied

    def operators(self, k, n, **kwargs):
        """{mode: PackedLinear} over this slot's views (no copies; `activate` decides which is valid)."""
        from .runtime import PackedLinear
        return {mode: PackedLinear(view["packed"], view["metadata"], view["scales"], view["bias"], k, n, mode, **kwargs)
                for mode, view in self.views.items()}


class CoefficientArena:
    """One FP32 device tensor holding scales|bias of many units back to back.

    A per-step selector fills the whole arena with one copy; the operators keep reading the same
    views.  Requires residency "active" slots whose modes all have n-element scales and bias."""

    def __init__(self, slots, ops, widths):
        self.ranges, size = {}, 0
        for uid, slot in slots.items():
            n = widths[uid]
            if slot.residency != "active":
                raise ValueError("a coefficient arena makes the modes of a unit share one buffer: 'active' slots only")
            if any(row[key].numel() != n for row in slot.host.values() for key in ("scales", "bias")):
                raise ValueError(f"unit {uid}: every mode needs {n} scales and {n} bias values")
            self.ranges[uid] = (size, n)
            size += 2 * n
        device = next(iter(slots.values())).device
        self.arena = torch.empty(size, dtype=torch.float32, device=device)
        for uid, slot in slots.items():
            offset, n = self.ranges[uid]
            for key, start in (("scales", offset), ("bias", offset + n)):
                slot.buffers[key] = self.arena[start:start + n]
                for mode, row in slot.host.items():
                    view = slot.buffers[key].view(row[key].shape)
                    slot.views[mode][key] = view
                    setattr(ops[uid][mode], key, view)

    def fill(self, slots, modes):
        """Stage the scales|bias of each unit's chosen mode on the host and copy them in one go."""
        staged = torch.empty(self.arena.numel(), dtype=torch.float32,
                             pin_memory=self.arena.device.type == "cuda")
        for uid, (offset, n) in self.ranges.items():
            row = slots[uid].host[modes[uid]]
            staged[offset:offset + n] = row["scales"]
            staged[offset + n:offset + 2 * n] = row["bias"]
        self.arena.copy_(staged, non_blocking=self.arena.device.type == "cuda")
        return staged.numel() * 4


def payload_from_reference(blob, k, n, bias=None):
    """A reference bank blob (`compact`, `metadata` in SM80 order, `scales`, `group`) as a slot payload."""
    from .importer import sm80_metadata_to_b200
    from .packing import lifted_k
    mode = int(blob["group"])
    _, pk = lifted_k(k, mode)
    compact = blob["compact"].detach().cpu().contiguous()
    if compact.dtype != torch.int8 or compact.shape[1] * 2 != pk or compact.shape[0] < n:
        raise ValueError("compact payload does not match this unit")
    bias = torch.zeros(n, dtype=torch.float32) if bias is None else bias.detach().cpu().float().contiguous()
    return mode, dict(packed=compact, metadata=sm80_metadata_to_b200(blob["metadata"], compact.shape[0], pk),
                      scales=blob["scales"].detach().cpu().float().contiguous(), bias=bias)
