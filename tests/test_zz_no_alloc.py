"""The allocation-free drift entry point, called through the C ABI.

Some programs that embed this library may not allocate device memory when they call it -- a serving
process whose memory pool took the whole device at start-up, a plug-in boundary that carries only
inputs and outputs -- so `dtb_drift_accumulate_noalloc` keeps its partial sums in a 1 MiB array inside
the library instead of caller-provided scratch.  It must give what `dtb_drift_accumulate` gives, on
consecutive calls (the built-in array is shared and keeps its old contents), and refuse inputs larger
than the array covers.  This file is collected last so that a run stopping at the first failure has
already exercised everything else.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ditango_b200 import _capi
    return _capi, _capi.load()


def _with_scratch(lib, cur, prev, acc):
    n = cur.numel()
    need = lib.dtb_drift_scratch_bytes(n)
    scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")
    rc = lib.dtb_drift_accumulate(cur.data_ptr(), prev.data_ptr(), n, acc.data_ptr(), scratch.data_ptr(), need,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.dtb_last_error()


def _no_alloc(lib, cur, prev, acc):
    rc = lib.dtb_drift_accumulate_noalloc(cur.data_ptr(), prev.data_ptr(), cur.numel(), acc.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.dtb_last_error()


def test_no_alloc_entry_matches_the_scratch_entry_on_two_calls_in_a_row():
    _capi, lib = _lib()
    g = torch.Generator().manual_seed(11)
    cases = []
    for n in (70_001, 3_000_000):          # the second call has to cope with what the first left behind
        prev = torch.randn(n, generator=g)
        cur = prev + 0.03 * torch.randn(n, generator=g)
        cur[5] = float("nan")
        cases.append((cur.cuda(), prev.cuda()))
    want = torch.zeros(2, device="cuda")
    got = torch.zeros(2, device="cuda")
    for i, (cur, prev) in enumerate(cases):
        _with_scratch(lib, cur, prev, want[i:i + 1])
    # Free device memory as the driver reports it: an allocation made inside the library would show
    # here, which torch's own allocator statistics cannot see.  The first call on a device only looks
    # up the address of the built-in array, so it is made before the measurement.
    _no_alloc(lib, *cases[0], torch.zeros(1, device="cuda"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for i, (cur, prev) in enumerate(cases):
        _no_alloc(lib, cur, prev, got[i:i + 1])
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    # same kernel, same reduction order: the tolerance of the drift tests (2e-6 relative) is ample;
    # and both agree with the CPU restatement of the reference's rel_l1
    from oracle import ring_oracle as O
    for (cur, prev), w, g_ in zip(cases, want.cpu().tolist(), got.cpu().tolist()):
        assert w > 0 and abs(w - g_) <= 2e-6 * max(1.0, abs(w))
        ref = O.rel_l1(cur.cpu(), prev.cpu())
        assert abs(g_ - ref) <= 2e-6 * max(1.0, abs(ref))
    # a third call accumulates on top, like the scratch entry does
    _no_alloc(lib, *cases[0], got[0:1])
    assert abs(got[0].item() - 2 * want[0].item()) <= 4e-6 * max(1.0, want[0].item())


def test_no_alloc_entry_rejects_sizes_beyond_its_array():
    _capi, lib = _lib()
    limit = lib.dtb_drift_noalloc_max_elements()
    assert limit == 32760 * 16384
    x = torch.zeros(8, device="cuda")
    acc = torch.zeros(1, device="cuda")
    rc = lib.dtb_drift_accumulate_noalloc(x.data_ptr(), x.data_ptr(), limit + 1, acc.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = lib.dtb_last_error().decode()
    assert str(limit) in msg and "exceeds" in msg
    torch.cuda.synchronize()
    assert acc.item() == 0
