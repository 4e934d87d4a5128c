"""The allocation-free routing-plan entry point, called the way an embedder would call it.

Some users of this library cannot let it allocate: they run inside a process whose device memory
is already handed out, or on a stream where an allocation's implicit synchronisation is not
allowed.  For them the shared object exports one plain C symbol, ``mts_moe_plan_noalloc``, which
takes caller-owned buffers only and keeps its scratch in a fixed array inside the library.

This test loads the built shared object with ``ctypes``, calls that symbol with raw device
pointers on the current stream, and checks every output against the regular (allocating)
``moe_plan`` binding, twice in a row, because consecutive calls share the scratch array.
The file name sorts last so that a run that stops at the first failure has already run all
other tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load_symbol():
    from mini_train_sys_b200.ops.build import EXT_PATH, load_extension

    load_extension()   # resolves the library's torch dependencies before ctypes opens the same file
    lib = ctypes.CDLL(str(EXT_PATH))
    fn = lib.mts_moe_plan_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 6
    return fn


def _call(fn, idx: torch.Tensor, experts: int, capacity: int):
    tokens, top_k = idx.shape
    dev = idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    out = {
        "row_token": torch.empty(capacity, **i32),
        "token_rows": torch.empty(tokens * top_k, **i32),
        "tile_group": torch.empty(capacity // 128, **i32),
        "group_rows": torch.empty(experts + 1, **i32),
        "meta": torch.zeros(4, **i32),
    }
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = fn(idx.data_ptr(), tokens, top_k, experts, capacity, out["row_token"].data_ptr(), out["token_rows"].data_ptr(),
            out["tile_group"].data_ptr(), out["group_rows"].data_ptr(), out["meta"].data_ptr(), stream)
    return rc, out


def test_noalloc_plan_matches_allocating_entry_point():
    from mini_train_sys_b200.ops.native_backend import ext

    fn = _load_symbol()
    torch.manual_seed(21)
    for tokens, top_k, experts in ((3000, 2, 8), (777, 2, 4)):   # two calls in a row share the scratch
        idx = torch.rand(tokens, experts, device="cuda").topk(top_k, -1).indices.to(torch.int32).contiguous()
        want = dict(zip(("row_token", "token_rows", "tile_group", "group_rows", "meta"), ext().moe_plan(idx, experts)))
        capacity = int(ext().moe_capacity_rows(tokens, top_k, experts))
        rc, got = _call(fn, idx, experts, capacity)
        torch.cuda.synchronize()
        assert rc == 0
        live_tiles = int(want["meta"][0])
        for name in ("row_token", "token_rows", "group_rows"):
            assert torch.equal(got[name], want[name]), name
        assert torch.equal(got["tile_group"][:live_tiles], want["tile_group"][:live_tiles])
        assert torch.equal(got["meta"][:3], want["meta"][:3])


def test_noalloc_plan_rejects_oversized_requests():
    fn = _load_symbol()
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    assert fn(p, 1 << 20, 2, 8, 128, p, p, p, p, p, 0) == -1        # 2M routes > 1,048,576
    assert fn(p, 16, 2, 65, 128, p, p, p, p, p, 0) == -1            # more than 64 experts
    assert fn(p, 16, 2, 8, 100, p, p, p, p, p, 0) == -2             # capacity not a multiple of 128
    assert fn(None, 16, 2, 8, 128, p, p, p, p, p, 0) == -2


def test_noalloc_plan_flags_an_undersized_capacity_and_stays_inside_it():
    """A capacity below the padded row count raises the overflow word; nothing is written past the caller's buffers."""

    fn = _load_symbol()
    torch.manual_seed(3)
    tokens, top_k, experts = 2000, 2, 8
    idx = torch.rand(tokens, experts, device="cuda").topk(top_k, -1).indices.to(torch.int32).contiguous()
    capacity = 1024                                       # 4000 routes cannot fit
    guard = 256
    i32 = dict(dtype=torch.int32, device="cuda")
    row_token = torch.full((capacity + guard,), -7, **i32)
    tile_group = torch.full((capacity // 128 + guard,), -7, **i32)
    token_rows = torch.full((tokens * top_k + guard,), -7, **i32)
    group_rows = torch.empty(experts + 1, **i32)
    meta = torch.zeros(4, **i32)
    rc = fn(idx.data_ptr(), tokens, top_k, experts, capacity, row_token.data_ptr(), token_rows.data_ptr(), tile_group.data_ptr(),
            group_rows.data_ptr(), meta.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and int(meta[2]) == 1
    assert bool((row_token[capacity:] == -7).all()) and bool((tile_group[capacity // 128:] == -7).all())
    assert bool((token_rows[tokens * top_k:] == -7).all())
    placed = token_rows[:tokens * top_k]
    assert int(placed.max()) < capacity and bool((placed[placed >= 0] < capacity).all())
    assert bool((placed == -1).any())                     # the routes that did not fit have no row


def test_noalloc_plan_treats_negative_indices_as_dropped_routes():
    from mini_train_sys_b200.ops.native_backend import ext

    fn = _load_symbol()
    torch.manual_seed(4)
    tokens, top_k, experts = 1500, 2, 8
    idx = torch.rand(tokens, experts, device="cuda").topk(top_k, -1).indices.to(torch.int32)
    drop = torch.rand(tokens, top_k, device="cuda") < 0.3
    idx = torch.where(drop, torch.full_like(idx, -1), idx).contiguous()
    capacity = int(ext().moe_capacity_rows(tokens, top_k, experts))
    rc, got = _call(fn, idx, experts, capacity)
    torch.cuda.synchronize()
    assert rc == 0 and int(got["meta"][2]) == 0
    rows = got["token_rows"].view(tokens, top_k)
    assert bool((rows[drop] == -1).all()) and bool((rows[~drop] >= 0).all())
    kept = rows[~drop].long()
    assert kept.unique().numel() == kept.numel()          # every kept route has a row of its own
    starts = got["group_rows"].long()
    expert_of_row = torch.bucketize(kept, starts[1:], right=True)
    assert torch.equal(expert_of_row, idx[~drop].long())  # and it lies in its expert's segment
    tok = torch.arange(tokens, device="cuda").view(-1, 1).expand(-1, top_k)[~drop]
    assert torch.equal(got["row_token"][kept].long(), tok)
