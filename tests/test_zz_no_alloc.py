"""GPU: the allocation-free GEMM entry point against the regular one.

rb_gemm_no_alloc serves hosts that must not allocate device memory while they run (fixed memory budgets,
real-time loops that cannot take cudaMalloc's device-wide synchronisation).  Its scratch is one array inside
the library that every call shares and that keeps the previous call's contents, so the check runs two calls in
a row with different shapes: the second, smaller call must not see anything the first one left behind.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

from rust_ascend_b200 import B200Runtime as RT
from rust_ascend_b200 import DType, InvalidTensor, Transpose
from rust_ascend_b200.runtime import f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def _pair(client, seed, m, n, k, ta, tb, dtype):
    rng = np.random.default_rng(seed)
    a = client.upload(f32_to_bf16_bits(rng.standard_normal((k, m) if ta else (m, k), dtype=np.float32)))
    b = client.upload(f32_to_bf16_bits(rng.standard_normal((n, k) if tb else (k, n), dtype=np.float32)))
    want = client.read(RT.gemm(client, a, b, Transpose(int(ta)), Transpose(int(tb)), dtype))
    out = client.tensor((m, n), dtype)
    client.memset(out, 0xFF)
    client.sync()
    before, free_before = client.stats()["allocations"], _device_free_bytes()
    RT.gemm_no_alloc(client, a, b, Transpose(int(ta)), Transpose(int(tb)), out)
    # Two views of "allocated nothing": the runtime's own storage table did not grow (that counter only sees rb_alloc), and the
    # driver reports the same free device memory as before the call (which would also show a cudaMalloc made behind the table).
    assert client.stats()["allocations"] == before
    assert _device_free_bytes() == free_before
    got = client.read(out)
    return got, want


def _device_free_bytes():
    import torch
    return torch.cuda.mem_get_info(0)[0]


def test_two_calls_in_a_row_match_the_allocating_entry_point(client, oracle):
    # first call fills most of the scratch array (A^T and B rewrites: 2 x 6 MiB), second call is small and ragged
    got, want = _pair(client, 1, 1536, 2048, 2048, True, False, DType.BF16)
    np.testing.assert_array_equal(got, want)                # same kernel, same operands: identical bits
    got, want = _pair(client, 2, 144, 80, 208, True, False, DType.F32)
    np.testing.assert_array_equal(got, want)
    # and against the CPU oracle, so that the check does not rest on the other entry point alone
    rng = np.random.default_rng(2)
    a = rng.standard_normal((208, 144), dtype=np.float32); b = rng.standard_normal((208, 80), dtype=np.float32)
    ref = oracle.gemm_bf16(a, b, True, False, False)
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-4 * np.abs(ref).max())
    got, want = _pair(client, 3, 256, 512, 320, False, True, DType.BF16)   # no rewrite needed at all
    np.testing.assert_array_equal(got, want)


def test_operands_beyond_the_built_in_scratch_are_rejected(client):
    a = client.tensor((4096, 2048), DType.BF16)             # needs no rewrite
    b = client.tensor((2048, 4112), DType.BF16)             # stored [K,N]: 2048*4112*2 B > 16 MiB
    out = client.tensor((4096, 4112), DType.BF16)
    with pytest.raises(InvalidTensor, match="scratch"):
        RT.gemm_no_alloc(client, a, b, Transpose.No, Transpose.No, out)
    for t in (a, b, out):
        client.free(t.handle)
