"""The allocation-free dedup entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they need the
dedup: a server whose memory pool is frozen once its tables are placed, or a
plain-C / ctypes caller without torch's allocator.  For them the library keeps
the scratch in a static device array.  This test drives that entry point the
way such a caller would (ctypes on the shared object, raw pointers, a stream
handle) and checks it against the regular launcher, twice in a row so that the
second call runs on the leftovers of the first.  The file name sorts last on
purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

from kraken_b200 import _build
from kraken_b200._native import C

pytestmark = pytest.mark.gpu
MAX_IDS = 65536


def _entry():
    lib = ctypes.CDLL(_build.SO_PATH)
    fn = lib.kraken_dedup_bucketize_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _regular(ids, world, salt):
    """The existing entry point, with scratch that the caller allocates."""
    dev, n = ids.device, ids.numel()
    hbits = max(4, (2 * max(n, 1) - 1).bit_length())
    hkeys = torch.zeros((1 << hbits, 2), dtype=torch.int64, device=dev)
    hkeys[:, 0] = -1
    slot_of = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    cnt = torch.zeros(world, dtype=torch.int32, device=dev)
    off = torch.zeros(world + 1, dtype=torch.int32, device=dev)
    uniq = torch.zeros(max(n, 1), dtype=torch.int64, device=dev)
    inv = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    C.dedup_bucketize(ids, world, salt, hkeys, slot_of, hbits, cnt, off, uniq, inv, status)
    return off, uniq, inv


def _no_alloc(fn, ids, world, salt):
    dev, n = ids.device, ids.numel()
    off = torch.full((world + 1,), -7, dtype=torch.int32, device=dev)
    uniq = torch.zeros(max(n, 1), dtype=torch.int64, device=dev)
    inv = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    msg = ctypes.create_string_buffer(256)
    rc = fn(ids.data_ptr(), n, world, salt, off.data_ptr(), uniq.data_ptr(), inv.data_ptr(), status.data_ptr(),
            torch.cuda.current_stream().cuda_stream, msg, len(msg))
    assert rc == 0, msg.value
    return off, uniq, inv, status


def _same_result(ids, a, b, world):
    off_a, uniq_a, inv_a = a[0].cpu(), a[1].cpu(), a[2].cpu()
    off_b, uniq_b, inv_b = b[0].cpu(), b[1].cpu(), b[2].cpu()
    assert torch.equal(off_a, off_b)  # same number of unique ids for every owner
    n = ids.numel()
    host = ids.cpu()
    # both maps reproduce the input
    assert torch.equal(uniq_a[inv_a[:n].long()], host) and torch.equal(uniq_b[inv_b[:n].long()], host)
    # inside an owner's segment the order is whatever the atomics gave: compare as sets
    for o in range(world):
        lo, hi = int(off_a[o]), int(off_a[o + 1])
        assert torch.equal(uniq_a[lo:hi].sort().values, uniq_b[lo:hi].sort().values)


def test_no_alloc_entry_matches_regular_entry_twice():
    fn = _entry()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(0)
    first = torch.randint(0, 9000, (50000,), generator=g).to(dev)
    second = torch.randint(-50, 300, (777,), generator=g)           # smaller: runs on the first call's leftovers
    second = torch.where(second == -1, torch.full_like(second, 5), second).to(dev)  # -1 is the reserved id
    for ids, world, salt in [(first, 8, 0), (second, 3, 12345), (first, 1, 7)]:
        got = _no_alloc(fn, ids, world, salt)
        torch.cuda.synchronize()
        assert got[3].item() == 0
        _same_result(ids, got, _regular(ids, world, salt), world)
    # the claim in the name: with its outputs already allocated, a call takes no device memory at all
    # (the first call above has loaded the module and resolved the scratch address)
    n = first.numel()
    off = torch.zeros(9, dtype=torch.int32, device=dev)
    uniq = torch.zeros(n, dtype=torch.int64, device=dev)
    inv = torch.zeros(n, dtype=torch.int32, device=dev)
    msg = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        assert fn(first.data_ptr(), n, 8, 0, off.data_ptr(), uniq.data_ptr(), inv.data_ptr(), None, stream, msg,
                  len(msg)) == 0, msg.value
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)


def test_no_alloc_entry_refuses_what_it_cannot_hold():
    fn = _entry()
    dev = torch.device("cuda", torch.cuda.current_device())
    ids = torch.zeros(MAX_IDS + 1, dtype=torch.int64, device=dev)
    out = torch.zeros(MAX_IDS + 1, dtype=torch.int64, device=dev)
    inv = torch.zeros(MAX_IDS + 1, dtype=torch.int32, device=dev)
    off = torch.zeros(17, dtype=torch.int32, device=dev)
    msg = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(ids.data_ptr(), MAX_IDS + 1, 2, 0, off.data_ptr(), out.data_ptr(), inv.data_ptr(), None, stream, msg,
              len(msg)) == -1
    assert b"too many ids" in msg.value and str(MAX_IDS).encode() in msg.value
    assert fn(ids.data_ptr(), 16, 17, 0, off.data_ptr(), out.data_ptr(), inv.data_ptr(), None, stream, msg,
              len(msg)) == -2
    assert fn(ids.data_ptr(), 16, 2, 0, None, out.data_ptr(), inv.data_ptr(), None, stream, msg, len(msg)) == -3
    # an empty batch is fine and yields empty segments
    assert fn(None, 0, 4, 0, off.data_ptr(), None, None, None, stream, msg, len(msg)) == 0
    torch.cuda.synchronize()
    assert off[:5].tolist() == [0, 0, 0, 0, 0]
