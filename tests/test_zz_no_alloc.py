"""GPU: the allocation-free entry point ffm_group_rows_static against ffm_group_rows.

Some callers of libffmoe cannot allocate device memory where they call it (a frozen allocator in a serving loop,
a language binding that only forwards pointers), so they cannot provide the scratch workspace ffm_group_rows asks
for. ffm_group_rows_static keeps that scratch inside the library. This test drives both entry points through the
C ABI on the same inputs, twice in a row with different inputs, and requires identical integer outputs; the
second call also shows that whatever the first call left in the built-in scratch does not leak into the result.
The file name sorts last so that a run which stops at the first failure has already executed every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

from flashfusedmoe_b200 import _lib  # noqa: E402


def _call_both(ids, E):
    lib = _lib.load()
    dev = ids.device
    T = ids.numel()
    rows_cap = int(lib.ffm_rows_capacity(T, E))
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def outputs():
        return (torch.full((E,), -7, dtype=torch.int32, device=dev),
                torch.full((E + 1,), -7, dtype=torch.int32, device=dev),
                torch.full((T,), -7, dtype=torch.int32, device=dev),
                torch.full((rows_cap,), -7, dtype=torch.int32, device=dev))

    ws = torch.empty(int(lib.ffm_route_workspace_bytes(T, E, 1)), dtype=torch.uint8, device=dev)
    ref = outputs()
    rc = lib.ffm_group_rows(ids.data_ptr(), T, E, ref[0].data_ptr(), ref[1].data_ptr(), ref[2].data_ptr(),
                            ref[3].data_ptr(), rows_cap, ws.data_ptr(), ws.numel(), status.data_ptr(), stream)
    assert rc == 0
    got = outputs()
    rc = lib.ffm_group_rows_static(ids.data_ptr(), T, E, got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(),
                                   got[3].data_ptr(), rows_cap, status.data_ptr(), stream)
    assert rc == 0, _lib.error_string(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return ref, got


def test_static_variant_matches_workspace_variant_twice_in_a_row():
    torch.manual_seed(0)
    # two calls back to back, the second with a different size and expert count
    for T, E in [(50000, 64), (3001, 8)]:
        ids = torch.randint(0, E, (T,), dtype=torch.int32, device="cuda")
        ref, got = _call_both(ids, E)
        for name, a, b in zip(("counts", "tile_start", "pos", "src"), ref, got):
            assert torch.equal(a, b), f"{name} differs for T={T}, E={E}"
        assert int(got[0].sum()) == T


def test_static_variant_rejects_sizes_beyond_its_maximum():
    lib = _lib.load()
    ids = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.zeros(1 << 12, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = out.data_ptr()
    too_many_rows = (1 << 20) + 1
    rc = lib.ffm_group_rows_static(ids.data_ptr(), too_many_rows, 8, p, p, p, p, 1 << 40, status.data_ptr(), 0)
    assert rc == -6 and "built-in scratch" in _lib.error_string(rc)
    rc = lib.ffm_group_rows_static(ids.data_ptr(), 16, 257, p, p, p, p, 1 << 40, status.data_ptr(), 0)
    assert rc == -6
