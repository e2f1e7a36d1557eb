"""The allocation-free matmul entry point against the ordinary one.

``ferric_cuda_matmul_q_noalloc`` exists for hosts that cannot let a plugin allocate device memory
(all of HBM already handed to their own pools; no tolerance for the device-wide stall an allocation
causes; allocator calls simply not permitted).  It keeps its activation scratch in a fixed array
inside the library.  Because that array is shared by every call and keeps whatever the previous call
left in it, the check runs two different products back to back and requires each to equal what
``ferric_cuda_matmul_q`` gives for the same inputs -- bit for bit, since both run the same kernels
on the same fragments.  Collected last on purpose (see the file name)."""
import ctypes as C

import numpy as np
import pytest
import torch

from ferric_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_noalloc_matches_matmul_q_on_two_calls_in_a_row():
    import ferric_b200 as F
    from ferric_b200 import _lib

    lib = _lib.load()
    ctx = F.Context(0)
    cases = [(12, 300, 2048, 3), (14, 130, 1024, 1)]          # a wider product first, then a narrower one
    mats = [F.QMatrix.from_bytes(ctx, synth.matrix(ty, r, c, seed=50 + i), ty, r, c) for i, (ty, r, c, _) in enumerate(cases)]
    xs = [torch.from_numpy(synth.activations(m, c, seed=60 + i)).cuda() for i, (_, _, c, m) in enumerate(cases)]
    want = [qm.matmul(x) for qm, x in zip(mats, xs)]
    outs = [torch.full_like(w, float("nan")) for w in want]
    # the first call on a device does the one-time set-up (address look-up; the driver also loads the
    # library's kernels and its fixed array lazily), so it comes before the memory reading
    mats[0].matmul_noalloc(xs[0], outs[0])
    outs[0].fill_(float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for qm, x, out in zip(mats, xs, outs):                     # two calls in a row through the C ABI
        rc = lib.ferric_cuda_matmul_q_noalloc(ctx._h, qm._h, C.c_void_p(x.data_ptr()), x.shape[0], x.shape[1],
                                              C.c_void_p(out.data_ptr()))
        assert rc == 0, lib.ferric_cuda_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before         # no device memory was taken
    for got, ref in zip(outs, want):
        assert torch.equal(got, ref)
    # and once more in the opposite order, so each call follows the other's leftovers
    for qm, x, out, ref in reversed(list(zip(mats, xs, outs, want))):
        out.fill_(float("nan"))
        assert torch.equal(qm.matmul_noalloc(x, out), ref)
    # beyond the fixed array: refused with a message, nothing launched
    big = F.QMatrix.from_bytes(ctx, synth.matrix(12, 16, 8192, seed=1), 12, 16, 8192)
    assert big.scratch_bytes(64) > (2 << 20)
    xb = torch.zeros((64, 8192), device="cuda")
    yb = torch.zeros((64, 16), device="cuda")
    with pytest.raises(F.FerricError) as e:
        big.matmul_noalloc(xb, yb)
    assert e.value.status == 3 and "fixed" in str(e.value)
    for qm in mats + [big]:
        qm.close()
    ctx.close()


@pytest.mark.parametrize("ty,rows,cols", [(12, 272, 1024), (14, 144, 768)])
@pytest.mark.parametrize("m", [9, 16])
def test_noalloc_above_eight_rows_against_the_oracle(ty, rows, cols, m):
    """Above 8 activation rows the ordinary entry point may pick another kernel (the tensor-core decode kernel) while
    the allocation-free one runs GEMV passes out of its fixed array, so here the check is against the CPU oracle
    directly, element by element (1e-3 relative + 1e-4 absolute), twice in a row -- and against ``ferric_cuda_matmul_q``
    within the same bar."""
    import ferric_b200 as F
    from ferric_b200 import _lib

    lib = _lib.load()
    ctx = F.Context(0)
    raw = synth.matrix(ty, rows, cols, seed=70 + m)
    qm = F.QMatrix.from_bytes(ctx, raw, ty, rows, cols)
    for rep in range(2):
        x = synth.activations(m, cols, seed=80 + rep)
        xd = torch.from_numpy(x).cuda()
        out = torch.full((m, rows), float("nan"), device="cuda")
        rc = lib.ferric_cuda_matmul_q_noalloc(ctx._h, qm._h, C.c_void_p(xd.data_ptr()), m, cols, C.c_void_p(out.data_ptr()))
        assert rc == 0, lib.ferric_cuda_last_error()
        got = out.cpu().numpy()
        ref = O.matmul_q(raw, ty, rows, cols, x)
        assert (np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref)).all()
        other = qm.matmul(xd).cpu().numpy()
        assert (np.abs(got - other) <= 1e-4 + 1e-3 * np.abs(other)).all()
    qm.close()
    ctx.close()
