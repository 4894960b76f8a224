"""Shape lists shared by the tests.  EAGER_CASES and FUSED_CASES repeat the
shape tuples of the reference's tests (tests/test_conv2d.py:18-39,
tests_graph/consts.py:71-82) in the order tests/golden/make_golden.py stored
their outputs."""

# (input_shape, weight_shape, bias?, stride, padding, dilation, groups)
EAGER_CASES = [
    ((1, 3, 8, 8), (4, 3, 3, 3), True, 1, 0, 1, 1),
    ((2, 3, 16, 16), (8, 3, 3, 3), False, 1, 1, 1, 1),
    ((2, 3, 15, 17), (6, 3, 5, 5), True, 2, 2, 1, 1),
    ((1, 3, 13, 11), (5, 3, 1, 1), True, 1, 0, 1, 1),
    ((1, 3, 17, 17), (4, 3, 3, 3), True, 1, 2, 2, 1),
    ((2, 3, 19, 21), (7, 3, 3, 3), False, 2, 2, 2, 1),
    ((1, 4, 12, 12), (8, 2, 3, 3), True, 1, 1, 1, 2),
    ((2, 4, 18, 14), (6, 2, 5, 5), False, 2, 2, 1, 2),
    ((1, 4, 10, 11), (4, 1, 3, 3), True, 1, 1, 1, 4),
    ((2, 8, 16, 16), (8, 1, 5, 5), False, 1, 2, 1, 8),
    ((1, 2, 9, 9), (4, 2, 3, 3), True, 1, "same", 1, 1),
    ((1, 4, 13, 13), (8, 2, 3, 3), False, 1, "same", 2, 2),
    ((1, 3, 12, 12), (6, 3, 3, 3), True, 1, "valid", 1, 1),
    ((2, 4, 20, 18), (8, 2, 5, 5), False, 2, "valid", 1, 2),
]

# (input_shape, weight_shape, stride, padding, dilation)
FUSED_CASES = [
    ((2, 8, 16, 16), (16, 8, 3, 3), 1, 1, 1),
    ((1, 4, 15, 17), (6, 4, 3, 5), (2, 1), (1, 2), 1),
    ((2, 3, 8, 8), (5, 3, 1, 1), 1, 0, 1),
    ((1, 6, 20, 18), (8, 6, 5, 3), (1, 2), (2, 1), 1),
    ((2, 4, 12, 10), (7, 4, 3, 3), 2, 1, 1),
    ((1, 5, 19, 21), (9, 5, 3, 3), 1, 2, 2),
    ((1, 3, 32, 32), (8, 3, 3, 3), 1, 1, 1),
    ((2, 8, 9, 11), (4, 8, 1, 1), 1, 0, 1),
    ((1, 4, 18, 18), (4, 4, 3, 3), 1, 0, 1),
    ((2, 12, 13, 15), (10, 12, 3, 3), 1, 1, 1),
    ((1, 64, 14, 14), (64, 64, 3, 3), 1, 1, 1),
    ((2, 256, 7, 7), (64, 256, 1, 1), 1, 0, 1),
    ((1, 128, 6, 6), (128, 128, 3, 3), 1, 1, 1),
    ((1, 3, 30, 30), (64, 3, 7, 7), 2, 3, 1),
]

# Tolerances of the parity contract: fp32 through split TF32 within 1e-4 of the
# CPU oracle; 16-bit inputs with fp32 accumulation within 1e-2 of the fp32 CPU
# oracle evaluated on the same bits.
TOL = {
    "float32": dict(rtol=1e-4, atol=1e-4),
    "bfloat16": dict(rtol=1e-2, atol=1e-2),
    "float16": dict(rtol=1e-2, atol=1e-2),
    "float64": dict(rtol=1e-9, atol=1e-9),
}
