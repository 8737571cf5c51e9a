"""The allocation-free Newton-Schulz entry point against the ordinary one.

Some users of the kernel library cannot allocate device memory while they run (a server whose pool
already owns the GPU, a loop that cannot afford the synchronisation an allocation implies, a plugin
with a fixed memory contract).  For them `tyr_newton_schulz_bf16_static` keeps its temporaries in an
array that is part of the library image.  This file calls that symbol through ctypes, twice in a
row, and expects the same result as `tyr_newton_schulz_bf16` with caller-owned scratch.  It is
collected last so that a failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_LIMIT = 19660800


def _lib():
    from tyr_b200._native import kernels
    lib = kernels()
    fn = lib.tyr_newton_schulz_bf16_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return lib


def _normalised(batch, R, C, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(batch, R, C, device="cuda", generator=g)
    x = x / (x.pow(2).sum((1, 2), keepdim=True).sqrt() + 1e-7)
    return x.bfloat16().contiguous()


@pytest.mark.parametrize("batch,R,C", [(1, 1280, 5120), (2, 512, 768), (1, 1024, 256)])
def test_static_scratch_entry_matches_ordinary_entry(batch, R, C):
    from tyr_b200.ops._common import cur_stream, err_word, raise_on_device_error
    from tyr_b200.ops.polar import MUON_COEFFS
    lib = _lib()
    dev = torch.device("cuda:0")
    a, b, c = MUON_COEFFS
    need = lib.tyr_newton_schulz_scratch_bytes(batch, R, C)
    assert need <= STATIC_LIMIT
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    err = err_word(dev)
    for call in range(2):  # two calls in a row: the second one sees the first one's leftovers
        x0 = _normalised(batch, R, C, seed=100 + call)
        ref = x0.clone()
        got = x0.clone()
        stream = cur_stream(dev)
        rc = lib.tyr_newton_schulz_bf16(ctypes.c_void_p(ref.data_ptr()), ctypes.c_void_p(scratch.data_ptr()),
                                        need, batch, R, C, 5, a, b, c, ctypes.c_void_p(err.data_ptr()), stream)
        assert rc == 0
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        reserved_before = torch.cuda.memory_reserved(dev)
        rc = lib.tyr_newton_schulz_bf16_static(ctypes.c_void_p(got.data_ptr()), batch, R, C, 5, a, b, c,
                                               ctypes.c_void_p(err.data_ptr()), stream)
        assert rc == 0
        torch.cuda.synchronize()
        raise_on_device_error(dev)
        if call == 1:      # the first call on a device may load the module and resolve the array's address
            free_after, _ = torch.cuda.mem_get_info(dev)
            assert free_after == free_before and torch.cuda.memory_reserved(dev) == reserved_before, \
                "the entry that must not allocate changed the device's free memory"
        # both entries run the same launches on the same data: the results are identical bit for bit
        assert torch.equal(got, ref), (call, ((got.float() - ref.float()).abs().max().item()))
        # and both are a real orthogonalisation of the input
        sv = torch.linalg.svdvals(got[0].float())
        assert sv.max() < 1.35 and sv.min() > 0.3


def test_static_scratch_entry_rejects_oversize():
    lib = _lib()
    x = torch.zeros(1, 2048, 8192, dtype=torch.bfloat16, device="cuda")
    rc = lib.tyr_newton_schulz_bf16_static(ctypes.c_void_p(x.data_ptr()), 1, 2048, 8192, 1, 1.0, 1.0, 1.0,
                                           None, None)
    assert rc == -8
    rc = lib.tyr_newton_schulz_bf16_static(ctypes.c_void_p(x.data_ptr()), 1, 100, 8, 1, 1.0, 1.0, 1.0, None, None)
    assert rc == -1
