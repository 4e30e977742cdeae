"""The allocation-free cross-entropy entry point, called through its exported C symbol.

It serves callers that cannot allocate device memory when they need the loss (all memory already
owned by their own arena, or allocation not permitted where they run): its per-row scratch is a
static array inside the library.  The check: same loss and same in-place gradient as the regular
entry point (which allocates its scratch through PyTorch), on two calls in a row, and a clear
refusal above the stated row limit.  Collected last on purpose (file name), so a failure here
cannot hide the result of any other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
MAX_ROWS = 65536


def _lib():
    import pccl_b200._native  # noqa: F401  builds the library if it is missing
    path = os.path.join(os.path.dirname(os.path.abspath(pccl_b200._native.__file__)), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.pccl_cross_entropy_mean_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_void_p]
    return lib, fn


def test_no_alloc_cross_entropy_matches_regular_entry_point_twice():
    from pccl_b200.ops.elementwise import cross_entropy_
    lib, fn = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, vocab) in enumerate([(777, 50257), (2048, 1001)]):      # two calls in a row share the scratch
        ld = (vocab + 7) // 8 * 8
        store = (torch.randn(rows, ld, device="cuda") * 2).bfloat16()
        tgt = torch.randint(0, vocab, (rows,), device="cuda")
        a = store.clone()
        b = store.clone()
        ref_rows = cross_entropy_(a[:, :vocab], tgt, grad_scale=1.0 / rows, ignore_index=-(1 << 62))
        ref = ref_rows.sum() / rows
        out = torch.full((1,), -1.0, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(b.data_ptr(), tgt.data_ptr(), out.data_ptr(), rows, vocab, ld, stream)
        assert rc == 0, (rc, lib.pccl_noalloc_last_cuda_error())
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert abs(out.item() - ref.item()) <= 1e-4 * max(1.0, abs(ref.item())), (call, out.item(), ref.item())
        assert torch.equal(a, b), f"call {call}: gradients differ from the regular entry point"


def test_no_alloc_cross_entropy_treats_out_of_range_targets_as_ignored_rows():
    """A target outside [0, vocab) -- the customary -100, a negative, one past the end -- must not be used as an index:
    such rows get loss 0 and an all-zero gradient, the others are unchanged, and the mean is over all rows."""
    from pccl_b200.ops.elementwise import cross_entropy_
    lib, fn = _lib()
    torch.manual_seed(1)
    rows, vocab = 64, 1000
    store = (torch.randn(rows, vocab, device="cuda") * 2).bfloat16()
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    bad = torch.tensor([3, 17, 40, 63], device="cuda")
    tgt_bad = tgt.clone()
    tgt_bad[bad] = torch.tensor([-100, -1, vocab, 1 << 40], device="cuda")
    a, b = store.clone(), store.clone()
    good = torch.ones(rows, dtype=torch.bool, device="cuda")
    good[bad] = False
    ref_rows = cross_entropy_(a, tgt, grad_scale=1.0 / rows, ignore_index=-(1 << 62))
    out = torch.zeros(1, device="cuda")
    assert fn(b.data_ptr(), tgt_bad.data_ptr(), out.data_ptr(), rows, vocab, vocab, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(a[good], b[good]) and int(b[bad].abs().sum()) == 0
    want = ref_rows[good].sum().item() / rows
    assert abs(out.item() - want) <= 1e-4 * max(1.0, abs(want))


def test_no_alloc_cross_entropy_rejects_what_it_cannot_hold():
    lib, fn = _lib()
    x = torch.zeros(8, 16, device="cuda", dtype=torch.bfloat16)
    t = torch.zeros(8, dtype=torch.int64, device="cuda")
    o = torch.zeros(1, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), t.data_ptr(), o.data_ptr(), MAX_ROWS + 1, 16, 16, s) == -1     # too many rows
    assert fn(x.data_ptr(), t.data_ptr(), o.data_ptr(), 8, 16, 12, s) == -2                # row stride not a multiple of 8
    assert fn(0, t.data_ptr(), o.data_ptr(), 8, 16, 16, s) == -2                           # null logits
    assert fn(x.data_ptr(), t.data_ptr(), o.data_ptr(), 8, 200000, 200000, s) == -2        # row does not fit shared memory
    torch.cuda.synchronize()
