"""The allocation-free column-sum entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at call time (all memory already
planned by a host framework, no tensor library in a plain C caller, or a path where the implicit
synchronisation of cudaMalloc is not acceptable). For them ``mtb200_colsum_noalloc`` carries its
workspace inside the library. This test checks it against the regular entry point, which takes
the workspace from the caller, on two calls in a row (the second call reuses the same built-in
workspace with a different shape, so leftovers from the first call would show up), and checks
that a size beyond the built-in workspace is refused.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mini_trainer_b200.ops.native import load_library
    lib = load_library()
    fn = lib.mtb200_colsum_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib, fn


def test_colsum_noalloc_matches_regular_entry_point_twice():
    lib, noalloc = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for T, N in ((1000, 4096), (77, 520)):          # second call: smaller shape over the same workspace
        x = torch.randn(T, N, device="cuda").bfloat16()
        expect = torch.empty(N, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(32 * N, dtype=torch.float32, device="cuda")
        rc = lib.mtb200_colsum(x.data_ptr(), x.stride(0), expect.data_ptr(), scratch.data_ptr(), T, N, stream)
        assert rc == 0
        got = torch.full((N,), float("nan"), dtype=torch.bfloat16, device="cuda")
        # warm-up call: the first call on a device resolves the workspace address and may load the module
        assert noalloc(x.data_ptr(), x.stride(0), got.data_ptr(), T, N, stream) == 0
        torch.cuda.synchronize()
        got.fill_(float("nan"))
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]     # driver-level: would also see a cudaMalloc inside the library
        rc = noalloc(x.data_ptr(), x.stride(0), got.data_ptr(), T, N, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        ref = x.float().sum(0)
        err = ((got.float() - ref).norm() / ref.norm()).item()
        assert err < 6e-3, err                        # same tolerance as the bias-gradient test
        assert torch.equal(got, expect)               # same kernels, same order of additions


def test_colsum_noalloc_rejects_sizes_beyond_its_workspace():
    _, noalloc = _lib()
    N = 16384 + 2
    x = torch.zeros(4, N, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert noalloc(x.data_ptr(), x.stride(0), out.data_ptr(), 4, N, st) == -11
    # other argument errors: an odd column count, a leading dimension smaller than the row
    assert noalloc(x.data_ptr(), x.stride(0), out.data_ptr(), 4, 513, st) == -10
    assert noalloc(x.data_ptr(), 256, out.data_ptr(), 4, 512, st) == -10
