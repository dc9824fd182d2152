"""The allocation-free routing-plan entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory while they run (they live inside a
fixed memory pool, or must not enter the CUDA allocator because cudaMalloc / cudaFree serialise
against the device).  `mdt_make_plan_noalloc` serves them: same results as the allocating
`make_plan` binding, scratch taken from a fixed array inside the library.  The test calls it
twice in a row (the scratch array keeps the previous call's contents) and compares every output
with the existing entry point; integer outputs must match exactly.  It also checks that neither the
driver's count of free device memory nor torch's allocation counter moves across a call.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from moe_distributed_training_b200.ops import build
    build.load()  # makes sure libtorch and the extension are loaded the usual way first
    lib = ctypes.CDLL(os.path.join(build.EXT_DIR, build.EXT_NAME + ".so"))
    fn = lib.mdt_make_plan_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.mdt_make_plan_noalloc_strerror.restype = ctypes.c_char_p
    lib.mdt_make_plan_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _call(lib, ids, E, block, cap, check_no_allocation=False):
    n = ids.numel()
    dev = ids.device
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    dest = torch.empty(n, dtype=torch.int32, device=dev)
    src = torch.empty(cap, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    # device memory as the driver sees it (any cudaMalloc / cudaFree moves it) and torch's own allocation counter
    free_before = torch.cuda.mem_get_info()[0]
    torch_allocs_before = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = lib.mdt_make_plan_noalloc(ids.data_ptr(), n, E, block, cap, counts.data_ptr(), offs.data_ptr(),
                                   dest.data_ptr(), src.data_ptr(), ctypes.c_void_p(stream))
    assert rc == 0, lib.mdt_make_plan_noalloc_strerror(rc).decode()
    torch.cuda.synchronize()
    if check_no_allocation:
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory in use changed across the call"
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == torch_allocs_before
    return counts, offs, dest, src


def test_noalloc_plan_matches_allocating_entry_point_twice():
    from moe_distributed_training_b200.ops import cuda_ops
    from moe_distributed_training_b200.ops.reference import plan_capacity
    lib = _lib()
    torch.manual_seed(0)
    # The first call on a device does the one-time set-up (address of the scratch array; the driver may load the
    # module that holds it), so memory is compared across the calls after it.
    warm = torch.zeros(64, dtype=torch.int32, device="cuda")
    _call(lib, warm, 4, 128, plan_capacity(64, 4, 128))
    # two different problems back to back: the second one must not see leftovers of the first
    for (T, k, E) in [(5000, 2, 8), (777, 2, 16)]:
        top = torch.randn(T, E, device="cuda").topk(k, dim=-1).indices.int()
        ids = top.reshape(-1).contiguous()
        cap = plan_capacity(T * k, E, 128)
        ref = cuda_ops.ext.make_plan(ids, E, 128, cap)
        got = _call(lib, ids, E, 128, cap, check_no_allocation=True)
        for name, a, b in zip(("counts", "padded_offsets", "dest_row", "src_slot"), got, ref):
            assert torch.equal(a, b), name


def test_noalloc_plan_rejects_oversized_problems():
    lib = _lib()
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.empty(1024, dtype=torch.int32, device="cuda")
    too_many = 262144 + 1
    rc = lib.mdt_make_plan_noalloc(ids.data_ptr(), too_many, 8, 128, 1024, out.data_ptr(), out.data_ptr(),
                                   out.data_ptr(), out.data_ptr(), ctypes.c_void_p(0))
    assert rc == -20 and b"larger" in lib.mdt_make_plan_noalloc_strerror(rc)
    rc = lib.mdt_make_plan_noalloc(ids.data_ptr(), 8, 65, 128, 1024, out.data_ptr(), out.data_ptr(),
                                   out.data_ptr(), out.data_ptr(), ctypes.c_void_p(0))
    assert rc == -20
