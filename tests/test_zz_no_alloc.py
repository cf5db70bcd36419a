"""The allocation-free sum of squares (for callers that may not allocate device memory, e.g. inside a
graph capture or with all memory owned by another allocator) must agree with the regular entry point,
call after call, although every call reuses the same fixed work area.  Collected last on purpose."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_sum_squares_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    import mccl_b200
    lib = mccl_b200.load()
    regular, noalloc, need = lib.mcclSumSquaresBf16, lib.mcclSumSquaresBf16NoAlloc, lib.mcclSumSquaresScratchFloats
    regular.restype = noalloc.restype = C.c_int
    regular.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_void_p]
    noalloc.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_void_p]
    need.restype, need.argtypes = C.c_uint64, [C.c_uint64]

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    torch.manual_seed(3)
    a, b = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    # Two calls in a row with different data and different sizes: the second must not see the first's leftovers.
    for n in (3_000_001, 70_000, 5):
        x = (torch.randn(n, device=dev) * 3).to(torch.bfloat16)
        scratch = torch.zeros(int(need(n)), device=dev)
        assert regular(x.data_ptr(), n, scratch.data_ptr(), scratch.numel(), a.data_ptr(), 0, stream) == 0
        assert noalloc(x.data_ptr(), n, b.data_ptr(), 0, stream) == 0
        torch.cuda.synchronize()
        ref = x.float().pow(2).sum()
        assert torch.allclose(b, a, rtol=2e-5), (n, a.item(), b.item())
        assert torch.allclose(b[0], ref, rtol=2e-5), (n, b.item(), ref.item())
        assert noalloc(x.data_ptr(), n, b.data_ptr(), 1, stream) == 0          # accumulate on top
        torch.cuda.synchronize()
        assert torch.allclose(b[0], 2 * ref, rtol=2e-5)
    # Exactly the largest count the fixed work area covers: every one of its partial-sum slots is in use.
    n = 4096 * 65536
    x = torch.empty(n, device=dev, dtype=torch.bfloat16)
    for lo in range(0, n, 1 << 26):
        x[lo:lo + (1 << 26)].copy_(torch.randn(min(1 << 26, n - lo), device=dev))
    ref = sum(x[lo:lo + (1 << 26)].double().pow(2).sum().item() for lo in range(0, n, 1 << 26))
    for _ in range(2):                                                        # twice in a row: no leftovers at full size either
        assert noalloc(x.data_ptr(), n, b.data_ptr(), 0, stream) == 0
        torch.cuda.synchronize()
        assert abs(b.item() - ref) <= 1e-4 * ref, (b.item(), ref)
    del x
    x = torch.ones(8, device=dev, dtype=torch.bfloat16)
    # Larger than the fixed work area: refused before anything is launched.
    too_many = 4096 * 65536 + 1
    assert noalloc(x.data_ptr(), too_many, b.data_ptr(), 0, stream) == 4       # mcclInvalidArgument
