"""The allocation-free C entry point ``plexus_gemm_tn_noalloc`` against the regular GEMM.

Some hosts of this library must not allocate device memory while they run (a serving process
with a fixed memory budget, a plugin inside another framework's memory-planned step).  For them
the weight-gradient GEMM is exported as a plain C symbol that keeps its split-reduction partials
in a fixed array inside the library.  This test calls that symbol directly through ``ctypes``
(no torch binding in between), twice in a row with different operands, and compares each result
with the regular entry point, which runs the same kernel on torch-allocated scratch.  The file
name makes pytest collect it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from plexus_b200.ops import _ext

    _ext.load()  # makes sure libtorch / the CUDA runtime are already mapped
    lib = ctypes.CDLL(_ext.so_path())
    fn = lib.plexus_gemm_tn_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                   ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_int]
    lib.plexus_gemm_tn_noalloc_parts.restype = ctypes.c_int
    lib.plexus_gemm_tn_noalloc_parts.argtypes = [ctypes.c_int64]
    lib.plexus_noalloc_take_status.restype = ctypes.c_int
    lib.plexus_noalloc_take_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    return lib


def _status(lib):
    words = (ctypes.c_int * 8)()
    assert lib.plexus_noalloc_take_status(words) == 0
    return list(words)


def _call(lib, a, b, out):
    err = ctypes.create_string_buffer(256)
    rc = lib.plexus_gemm_tn_noalloc(
        a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), a.shape[0], a.shape[1],
        b.shape[1], torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode()


def _check_device(lib, index):
    """Two calls in a row on one device: a large problem, then a small one that finds the shared
    array full of the first call's partial sums.  Each result is compared with the regular entry
    point and with the fp64 product; the second call must leave the driver's count of free device
    memory (cudaMemGetInfo, which also sees allocations made behind torch's back) unchanged."""
    from plexus_b200 import ops

    dev = torch.device("cuda", index)
    torch.cuda.set_device(dev)
    for seed, (R, Mw, Nw) in enumerate([(20000, 128, 64), (7001, 104, 48)]):
        torch.manual_seed(seed)
        a = torch.randn(R, Mw, device=dev).to(torch.bfloat16)
        b = torch.randn(R, Nw, device=dev).to(torch.bfloat16)
        want = ops.gemm(a, b, trans_a=True, out_dtype=torch.float32)
        out = torch.full((Mw, Nw), float("nan"), dtype=torch.float32, device=dev)
        ref = a.double().t() @ b.double()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc, msg = _call(lib, a, b, out)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info(dev)[0]
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == before
        if seed > 0:  # the first call on a device may load the kernel's module lazily
            assert free_after == free_before
        assert _status(lib)[0] == 0
        assert (out.double() - ref).abs().max() / ref.abs().max() < 1e-3
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-5)


def test_noalloc_gemm_tn_matches_regular_entry_point_twice():
    lib = _lib()
    _check_device(lib, 0)
    if torch.cuda.device_count() > 1:
        # a second device has its own copy of the array and its own cached address
        _check_device(lib, 1)
        torch.cuda.set_device(0)


def test_noalloc_rejects_bad_leading_dimensions():
    lib = _lib()
    dev = torch.device("cuda", 0)
    a = torch.zeros(64, 16, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(16, 16, dtype=torch.float32, device=dev)
    err = ctypes.create_string_buffer(256)
    rc = lib.plexus_gemm_tn_noalloc(a.data_ptr(), 8, a.data_ptr(), 16, out.data_ptr(), 64, 16, 16,
                                    torch.cuda.current_stream().cuda_stream, err, 256)
    assert rc == 1 and b"leading" in err.value


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    lib = _lib()
    dev = torch.device("cuda", 0)
    R, Mw, Nw = 200000, 256, 256
    assert lib.plexus_gemm_tn_noalloc_parts(R) * Mw * Nw > 4 * 1024 * 1024
    a = torch.zeros(R, Mw, dtype=torch.bfloat16, device=dev)
    b = torch.zeros(R, Nw, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(Mw, Nw, dtype=torch.float32, device=dev)
    rc, msg = _call(lib, a, b, out)
    assert rc == 2 and "scratch" in msg
