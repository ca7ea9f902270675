"""More pins of the oracle: the device validation programs of the reference's driver crate and the prefix-rotary tensor
example, restated with their own index formulas, f64 expectations and tolerances."""
import numpy as np
import pytest

import vectors as V
from test_backward import close


@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("out_bf16", [False, True])
def test_driver_gemm_validation_cases(oracle, batch, ta, tb, out_bf16):
    a, b, d = V.driver_gemm_case(batch, ta, tb)                    # deepgemm_validate.rs:32-45, tolerance 0.05 + 0.01 |b|
    close(oracle.gemm_bf16(a, b, ta, tb, out_bf16), d, 0.05, 0.01)


def test_driver_grouped_and_linear_backward_cases(oracle):
    a, w, ends, d = V.driver_grouped_case()                        # deepgemm_validate.rs:47-53
    got = np.concatenate([oracle.gemm_bf16(a[:256], w[0], False, True, False), oracle.gemm_bf16(a[256:], w[2], False, True, False)])
    close(got, d, 0.05, 0.01)
    x, w, dy, dx, dw = V.driver_linear_backward_case()             # deepgemm_validate.rs:55-59
    close(oracle.gemm_bf16(dy, w, False, False, False), dx, 0.05, 0.01)
    close(oracle.gemm_bf16(dy, x, True, False, False), dw, 0.05, 0.01)


@pytest.mark.parametrize("n", V.COMMON_IR_SIZES)
def test_common_ir_silu_programs(oracle, n):
    x, up, dy, y, dgate, dup = V.common_ir_case(n)                 # common_ir_validate.rs:17-31, tolerance 5e-4 + 5e-4 |b|
    close(oracle.silu_mul(x, up), y, 5e-4, 5e-4)
    g, u = oracle.silu_mul_backward(x, up, dy)
    close(g, dgate, 5e-4, 5e-4); close(u, dup, 5e-4, 5e-4)


@pytest.mark.parametrize("table_shape", V.PREFIX_TABLE_SHAPES)
@pytest.mark.parametrize("layout", ["interleaved", "split_half"])
def test_rotary_prefix_tensor_example(oracle, table_shape, layout):
    x, cos, sin, dy, y, dx = V.rotary_prefix_tensor_case(table_shape, layout)   # rotary_prefix_tensor.rs:16-45, 3e-5 + 3e-5 |b|
    got = oracle.rotary_prefix(x, cos, sin, 6, layout)
    close(got, y, 3e-5, 3e-5)
    np.testing.assert_array_equal(got[..., 6:].view(np.uint32), x[..., 6:].view(np.uint32))   # the tail keeps its bits
    close(oracle.rotary_prefix(dy, cos, sin, 6, layout, backward=True), dx, 3e-5, 3e-5)


@pytest.mark.parametrize("shape", V.BIAS_SHAPES)
def test_bias_tensor_example_is_exact(oracle, shape):
    x, r, b, dy, plain, with_res, doubled, db = V.bias_tensor_case(shape)       # examples/bias_tensor.rs:11-41: exact equality
    np.testing.assert_array_equal(oracle.bias_add(x, b), plain)
    np.testing.assert_array_equal(oracle.bias_add(x, b, r), with_res)
    np.testing.assert_array_equal(oracle.bias_add(x, b, x), doubled)
    np.testing.assert_array_equal(oracle.column_sum(dy), db)


@pytest.mark.parametrize("m,n,k", [(16, 32, 32), (32, 48, 16)])
def test_frozen_linear_example(oracle, m, n, k):
    x, w, dy, y, dx = V.frozen_linear_case(m, n, k)                # examples/frozen_bf16_tensor.rs:33-52, 5e-4 + 5e-4 |b|
    close(oracle.gemm_bf16(x, w, False, True, False), y, 5e-4, 5e-4)
    close(oracle.gemm_bf16(dy, w, False, False, False), dx, 5e-4, 5e-4)


@pytest.mark.parametrize("shape", V.PADDED_GQA_SHAPES[:4] + [(2, 1, 1, 3, 7, 5, 9), (1, 1, 1, 17, 33, 7, 3)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_padded_attention_example_shapes(oracle, shape, mode):
    q, k, v, mask = V.padded_attention_case(shape, mode)          # examples/padded_attention_tensor.rs:14-36,47-62
    want = V.padded_attention_expected(q, k, v, mask)
    n, m = shape[4], shape[3]
    if mode == 2:
        got = oracle.attention(q, k, v, 0.25, causal=True, query_start=(1 << 40) + (n - m), key_start=1 << 40)
    else:
        got = oracle.attention(q, k, v, 0.25, mask=mask if mode == 1 else None)
    close(got, want, 2e-3, 3e-3)
