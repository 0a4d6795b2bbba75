"""The entry point that allocates nothing (air_b200/csrc/no_alloc.h), called through its
exported C symbol and compared with the ordinary decode attention, which takes its scratch
memory from the caller.

Some callers of this library cannot allocate device memory when they call it (a host program
with a fixed memory budget, a plug-in inside another runtime); for them the split-KV decode
attention keeps its scratch in a device array inside the library.  This test calls that entry
point twice in a row on different inputs, so that the second call runs on whatever the first one
left in the shared scratch, and checks both results; it also checks that a call too large for
the built-in scratch is refused with a clear message and launches nothing.

The file is named so that pytest collects it last.  It needs no other test to have run.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def library():
    from air_b200.csrc import build
    lib = ctypes.CDLL(build.build())
    f = lib.air_decode_attention_static
    v, i = ctypes.c_void_p, ctypes.c_int
    f.argtypes = [v, v, v, i, v, v, v, i, i, i, i, i, i, ctypes.c_float, i, v]
    f.restype = i
    lib.air_decode_attention_static_capacity.restype = ctypes.c_longlong
    lib.air_decode_attention_static_need.restype = ctypes.c_longlong
    lib.air_decode_attention_static_need.argtypes = [i, i, i, i]
    lib.air_decode_attention_static_error.restype = ctypes.c_char_p
    lib.air_decode_attention_static_error.argtypes = [i]
    return lib


def case(seed, H, K, d, P, lens):
    """Requests with `lens` tokens in shuffled pages, one query each."""
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // P) for n in lens) + 3
    perm = torch.randperm(pages, generator=g)
    cache = torch.randn(pages, 2, K, P, d, generator=g).to(torch.bfloat16)
    width = max(-(-n // P) for n in lens)
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    used = 0
    for s, n in enumerate(lens):
        for b in range(-(-n // P)):
            table[s, b] = perm[used]
            used += 1
    q = torch.randn(len(lens), H, d, generator=g).to(torch.bfloat16)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    slots = torch.arange(len(lens), dtype=torch.int32)
    return [x.cuda() for x in (q, cache, table, slots, positions)]


def reference(q, cache, table, positions, P):
    """float64 softmax attention over the gathered keys and values."""
    T, H, d = q.shape
    K = cache.shape[2]
    out = torch.zeros(T, H, d, dtype=torch.float64)
    q, cache, table = q.double().cpu(), cache.double().cpu(), table.cpu()
    for t in range(T):
        n = int(positions[t]) + 1
        blocks = [cache[int(table[t, b])] for b in range(-(-n // P))]
        k = torch.cat([b[0] for b in blocks], dim=1)[:, :n]       # [K, n, d]
        v = torch.cat([b[1] for b in blocks], dim=1)[:, :n]
        for h in range(H):
            g = h * K // H
            p = torch.softmax(k[g] @ q[t, h] / math.sqrt(d), 0)
            out[t, h] = p @ v[g]
    return out


def free_bytes():
    """Free device memory as the driver counts it (cudaMemGetInfo): any allocation, by whatever route, shows."""
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    from air_b200.csrc import ops
    lib = library()
    H, K, d, P, splits = 14, 2, 128, 16, 5
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, lens) in enumerate(((1, [300, 17, 1, 64, 129]), (2, [40, 500, 33, 7]))):
        q, cache, table, slots, positions = case(seed, H, K, d, P, lens)
        if call == 1:
            slots[2] = -1         # a padding token: skipped; its place in the shared scratch holds the first call's numbers
        want = torch.full_like(q, 3.0)
        ops.decode_attention(q, cache, table, slots, positions, want, 0, 1 / math.sqrt(d), splits=splits)
        got = torch.full_like(q, 3.0)
        assert lib.air_decode_attention_static_need(len(lens), H, d, splits) <= lib.air_decode_attention_static_capacity()
        before = free_bytes()
        rc = lib.air_decode_attention_static(q.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
                                             slots.data_ptr(), positions.data_ptr(), got.data_ptr(), len(lens), H, K,
                                             d, P, 0, 1 / math.sqrt(d), splits, stream)
        assert rc == 0, lib.air_decode_attention_static_error(rc).decode()
        if call == 1:     # (the first call on a device may load the kernels' code; the second finds everything there)
            assert free_bytes() == before, "the entry point obtained device memory"
        torch.cuda.synchronize()
        ref = reference(q, cache, table, positions, P)
        live = (slots >= 0).cpu()
        scale = max(1.0, float(ref.abs().max()))
        assert float((got.double().cpu() - want.double().cpu())[live].abs().max()) <= 1e-2 * scale
        assert float((got.double().cpu() - ref)[live].abs().max()) <= 1e-2 * scale
        assert bool((got[~live.cuda()] == 3.0).all()), "nothing is stored for a padding token"


def test_sizes_that_the_kernel_does_not_take_are_a_bad_argument_not_a_scratch_error():
    lib = library()
    H, K, d, P = 8, 2, 128, 16
    q, cache, table, slots, positions = case(4, H, K, d, P, [20] * 4)
    out = torch.full_like(q, 5.0)
    stream = torch.cuda.current_stream().cuda_stream
    for h, k, dd, pp, splits in ((8, 2, 96, 16, 4), (8, 3, 128, 16, 4), (8, 2, 128, 24, 4), (8, 2, 4096, 16, 32)):
        rc = lib.air_decode_attention_static(q.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
                                             slots.data_ptr(), positions.data_ptr(), out.data_ptr(), 4, h, k, dd, pp,
                                             0, 0.1, splits, stream)
        assert rc == 100001, (h, k, dd, pp, rc)
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())


def test_a_call_beyond_the_built_in_scratch_is_refused():
    lib = library()
    H, K, d, P = 32, 4, 128, 16
    q, cache, table, slots, positions = case(3, H, K, d, P, [20] * 64)
    out = torch.full_like(q, 5.0)
    splits = 32
    assert lib.air_decode_attention_static_need(64, H, d, splits) > lib.air_decode_attention_static_capacity()
    rc = lib.air_decode_attention_static(q.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1],
                                         slots.data_ptr(), positions.data_ptr(), out.data_ptr(), 64, H, K, d, P, 0,
                                         0.1, splits, torch.cuda.current_stream().cuda_stream)
    assert rc == 100002
    assert b"exceeds the built-in scratch" in lib.air_decode_attention_static_error(rc)
    torch.cuda.synchronize()
    assert bool((out == 5.0).all()), "nothing was launched"
