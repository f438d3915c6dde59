"""The allocation-free C entry point, called through its exported symbol.

Some users of the kernels cannot allocate device memory at the point of the call (fixed memory budgets,
allocators that must not be re-entered, C hosts without PyTorch's allocator). For them the library exports
``lmsae_csc_build_noalloc``, whose scratch lives inside the library. This test calls the raw symbol with
ctypes, twice in a row, and checks both results against the regular entry point that takes caller-provided
scratch tensors. The file name makes pytest collect it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from language_model_saes_b200.ops import native

    native.load(required=True)  # makes sure the shared object is built and its dependencies are loaded
    lib = ctypes.CDLL(str(native.so_path()))
    fn = lib.lmsae_csc_build_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def _codes(B, k, F, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, F, (B, k), generator=g, dtype=torch.int32)
    idx[torch.rand(B, k, generator=g) < 0.1] = -1
    return idx.cuda()


def _groups_as_sets(offsets, entries, F):
    off = offsets.cpu().tolist()
    ent = entries.cpu().tolist()
    return [sorted(ent[off[f] : off[f + 1]]) for f in range(F)]


def test_no_alloc_entry_point_matches_regular_entry_point_twice():
    from language_model_saes_b200.ops import sae_kernels as K

    fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (B, k, F, seed) in enumerate([(257, 9, 1000, 1), (64, 50, 5003, 2)]):
        idx = _codes(B, k, F, seed)
        want = K.FeatureGroups(F, B * k, idx.device).build(idx)
        offsets = torch.full((F + 1,), -7, dtype=torch.int32, device="cuda")
        entries = torch.full((B * k,), -7, dtype=torch.int32, device="cuda")
        rc = fn(idx.data_ptr(), idx.numel(), F, offsets.data_ptr(), entries.data_ptr(), stream)
        assert rc == 0, f"call {call}: error code {rc}"
        torch.cuda.synchronize()
        assert torch.equal(offsets, want.offsets), f"call {call}: offsets differ"
        # the order inside one feature's list depends on atomics; compare as sets
        assert _groups_as_sets(offsets, entries, F) == _groups_as_sets(want.offsets, want.entries, F), f"call {call}"


def test_no_alloc_entry_point_rejects_oversized_problems():
    fn = _lib()
    idx = _codes(4, 2, 8, 3)
    out = torch.zeros(16, dtype=torch.int32, device="cuda")
    too_many = (1 << 20) + 1
    rc = fn(idx.data_ptr(), idx.numel(), too_many, out.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    # positions are stored as 32-bit integers: more entries than INT_MAX are refused before anything is launched
    rc = fn(idx.data_ptr(), (1 << 31) + 5, 8, out.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0
