"""The backward entry point that allocates nothing, called through the C ABI.

Some callers may not allocate device memory once they are running -- the framework around them owns
every allocation, or they sit in a loop that must stay free of allocator calls -- so they cannot pass
scratch to ``oeq_tp_backward``.  ``oeq_tp_backward_noalloc`` keeps its scratch inside the library.
Its result must agree with the regular entry point's, also on a second call that finds the scratch
array dirty from the first.  Collected last on purpose: a failure here cannot hide another test.
"""
import numpy as np
import pytest
import torch

from conftest import problem_by_name
from helpers import rel_err, tp_inputs, to_oeq

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,batch", [("uvu_shared", 3000), ("uvw_small", 500)])
def test_matches_the_regular_backward_twice_in_a_row(name, batch):
    from openequivariance_b200 import _native
    p = problem_by_name(name)
    handle = _native.TPHandle(p)
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x, y, w, dz = tp_inputs(p, batch, 100 + call)
        xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, to_oeq(p, w), dz))
        want = [torch.empty_like(xt), torch.empty_like(yt), torch.empty_like(wt)]
        ws_bytes = handle.workspace_bytes(batch)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        handle.backward(batch, xt.data_ptr(), yt.data_ptr(), wt.data_ptr(), dzt.data_ptr(),
                        *(t.data_ptr() for t in want), ws.data_ptr(), ws_bytes, stream)
        got = [torch.full_like(t, float("nan")) for t in want]
        _native.check(lib.oeq_tp_backward_noalloc(handle.ptr, batch, xt.data_ptr(), yt.data_ptr(), wt.data_ptr(),
                                                  dzt.data_ptr(), *(t.data_ptr() for t in got), stream))
        torch.cuda.synchronize()
        handle.check()
        for g, e in zip(got, want):
            assert rel_err(g.cpu().numpy(), e.cpu().numpy()) < 1e-5


def test_refuses_what_does_not_fit_or_needs_no_scratch():
    from openequivariance_b200 import _native
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    buf = torch.zeros(1 << 20, device="cuda")
    per_row = _native.TPHandle(problem_by_name("readme"))
    assert lib.oeq_tp_backward_noalloc(per_row.ptr, 4, *([buf.data_ptr()] * 7), stream) == 1
    assert b"per-row" in lib.oeq_last_error()
    shared = _native.TPHandle(problem_by_name("uvu_shared"))
    assert lib.oeq_tp_backward_noalloc(shared.ptr, 0, *([buf.data_ptr()] * 7), stream) == 1
    assert lib.oeq_tp_backward_noalloc(shared.ptr, 4, 0, *([buf.data_ptr()] * 6), stream) == 1


def test_narrowed_launch_and_a_handle_without_status_word():
    """A weight tensor of 176 KiB leaves room for 46 partial gradients in the 8 MiB array, fewer than the CTAs
    the regular launch would use, so the entry point has to narrow its grid; and it is the first call on a
    new handle, which owns no status word yet.  The regular entry point (called afterwards) must agree."""
    from openequivariance_b200 import _native
    p = problem_by_name("uvw_64")
    batch = 3000
    assert p.weight_numel * 4 > (8 << 20) // 296
    handle = _native.TPHandle(p)
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    x, y, w, dz = tp_inputs(p, batch, 7)
    xt, yt, wt, dzt = (torch.from_numpy(a).cuda() for a in (x, y, to_oeq(p, (w / 8).astype(np.float32)), dz))
    got = [torch.full_like(t, float("nan")) for t in (xt, yt, wt)]
    _native.check(lib.oeq_tp_backward_noalloc(handle.ptr, batch, xt.data_ptr(), yt.data_ptr(), wt.data_ptr(),
                                              dzt.data_ptr(), *(t.data_ptr() for t in got), stream))
    torch.cuda.synchronize()
    handle.check()
    want = [torch.empty_like(t) for t in (xt, yt, wt)]
    ws_bytes = handle.workspace_bytes(batch)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    handle.backward(batch, xt.data_ptr(), yt.data_ptr(), wt.data_ptr(), dzt.data_ptr(),
                    *(t.data_ptr() for t in want), ws.data_ptr(), ws_bytes, stream)
    torch.cuda.synchronize()
    handle.check()
    for g, e in zip(got, want):
        assert rel_err(g.cpu().numpy(), e.cpu().numpy()) < 1e-5
