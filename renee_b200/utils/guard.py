"""Guard-band allocation: a debugging mode that catches out-of-bounds WRITES by any kernel.

With ``RENEE_B200_GUARD=1`` (or inside ``guard.enabled_for_test()``) every long-lived buffer the
framework allocates — flat parameter / gradient / moment buffers, encoder activations, classifier
weights, momentum and scratch, the step's staging buffers and the symmetric peer-memory allocations —
is carved out of a larger allocation with a 4 KiB band of a fixed byte pattern on each side.
``check()`` compares every band with the pattern in one device reduction and names the buffers whose
bands changed, with the side and the first damaged byte; ``XCTrainer.check_device_status`` calls it
after each epoch and ``assert_clean()`` is what tests call after a few steps.

Why this instead of a sanitizer run: the kernels receive raw pointers, not extents, so an index guard
inside a kernel can only repeat the predicate the kernel already uses; a band next to the buffer sees
what was actually written, whoever wrote it (our kernels, a library GEMM, a peer GPU's store through
NVLink).  It does not see out-of-bounds reads.  Off by default: the bands cost nothing when disabled
(the functions return plain ``torch.empty`` / ``torch.zeros`` tensors).  In guard mode the registry keeps
every guarded allocation alive until ``reset()``.

The reference has no counterpart (it has no tests or debug modes at all).
"""
from __future__ import annotations

import contextlib
import os
from typing import Callable, List, Optional

import torch

BAND_BYTES = 4096
CANARY = 0xA5

_enabled = os.environ.get("RENEE_B200_GUARD", "") == "1"
_registry: List["_Entry"] = []


class GuardError(RuntimeError):
    pass


class _Entry:
    """One guarded allocation.  The registry holds it (and so the memory) until ``reset()``: callers keep
    slices and reshaped views of the payload, so the payload tensor's own lifetime says nothing."""
    __slots__ = ("name", "raw", "lo", "hi")

    def __init__(self, name: str, raw: torch.Tensor, lo: int, hi: int):
        self.name = name
        self.raw = raw            # uint8 view of the whole allocation
        self.lo = lo              # first payload byte
        self.hi = hi              # one past the last payload byte


def enabled() -> bool:
    return _enabled


def enable(flag: bool) -> None:
    global _enabled
    _enabled = bool(flag)


@contextlib.contextmanager
def enabled_for_test():
    """Guard mode for the duration of a ``with`` block; the registry is emptied on both sides."""
    prev = _enabled
    enable(True)
    _registry.clear()
    try:
        yield
    finally:
        enable(prev)
        _registry.clear()


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _shape(shape):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        return tuple(int(s) for s in shape[0])
    return tuple(int(s) for s in shape)


def _register(name: Optional[str], raw: torch.Tensor, nbytes: int, dtype, shape, zero: bool) -> torch.Tensor:
    raw[:BAND_BYTES].fill_(CANARY)
    raw[BAND_BYTES + nbytes:].fill_(CANARY)
    payload = raw[BAND_BYTES:BAND_BYTES + nbytes]
    if zero:
        payload.zero_()
    view = payload.view(dtype).view(shape)
    _registry.append(_Entry(name or f"buffer{len(_registry)}", raw, BAND_BYTES, BAND_BYTES + nbytes))
    return view


def empty(*shape, dtype=torch.float32, device=None, name: Optional[str] = None) -> torch.Tensor:
    shape = _shape(shape)
    if not _enabled:
        return torch.empty(shape, dtype=dtype, device=device)
    nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
    tail = -nbytes % 256          # keeps the trailing band (and the next allocation) 256-byte aligned
    raw = torch.empty(BAND_BYTES + nbytes + tail + BAND_BYTES, dtype=torch.uint8, device=device)
    return _register(name, raw, nbytes, dtype, shape, zero=False)


def zeros(*shape, dtype=torch.float32, device=None, name: Optional[str] = None) -> torch.Tensor:
    shape = _shape(shape)
    if not _enabled:
        return torch.zeros(shape, dtype=dtype, device=device)
    t = empty(shape, dtype=dtype, device=device, name=name)
    t.zero_()
    return t


def from_allocator(alloc: Callable[[int, torch.dtype], torch.Tensor], numel: int, dtype,
                   name: Optional[str] = None) -> torch.Tensor:
    """``alloc(numel, dtype)`` with bands, for memory that must come from a particular allocator
    (symmetric peer memory).  The returned tensor has ``numel`` elements and starts ``BAND_BYTES`` into
    the allocation on every rank alike, so peer pointers derived from it stay consistent."""
    if not _enabled:
        return alloc(numel, dtype)
    esz = torch.empty((), dtype=dtype).element_size()
    band_elems = BAND_BYTES // esz
    nbytes = numel * esz
    tail_elems = (-nbytes % 256) // esz
    whole = alloc(numel + 2 * band_elems + tail_elems, dtype)
    raw = whole.view(torch.uint8)
    return _register(name, raw, nbytes, dtype, (numel,), zero=False)


def payload_offset_bytes() -> int:
    """Byte offset of a ``from_allocator`` tensor inside its allocation (0 when guard mode is off)."""
    return BAND_BYTES if _enabled else 0


def reset() -> None:
    """Forgets every guarded allocation (their memory is freed once the callers' views are gone)."""
    _registry.clear()


def check() -> List[str]:
    """Names (with side and first damaged byte offset relative to the payload) of buffers whose bands changed."""
    if not _registry:
        return []
    by_dev = {}
    for e in _registry:
        by_dev.setdefault(e.raw.device, []).append(e)
    bad: List[str] = []
    for dev, entries in by_dev.items():
        counts = torch.stack([(e.raw[:e.lo] != CANARY).sum() + (e.raw[e.hi:] != CANARY).sum() for e in entries])
        if int(counts.sum().item()) == 0:      # one synchronisation per device on the clean path
            continue
        for e, c in zip(entries, counts.tolist()):
            if c == 0:
                continue
            front = (e.raw[:e.lo] != CANARY).nonzero()
            back = (e.raw[e.hi:] != CANARY).nonzero()
            if front.numel():
                bad.append(f"{e.name}: {front.numel()} byte(s) before the buffer, nearest at offset "
                           f"{int(front.max().item()) - e.lo}")
            if back.numel():
                bad.append(f"{e.name}: {back.numel()} byte(s) after the buffer, nearest at offset "
                           f"{e.hi - e.lo + int(back.min().item())} (buffer is {e.hi - e.lo} bytes)")
    return bad


def assert_clean() -> None:
    bad = check()
    if bad:
        raise GuardError("out-of-bounds writes detected:\n  " + "\n  ".join(bad))


def registered() -> int:
    return len(_registry)
