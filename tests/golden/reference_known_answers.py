"""Known-answer values transcribed (as data) from the reference's own test files.

These pin the CPU oracle: every number below is a literal that the reference's tests assert for its
CPU path.  Paths are relative to the candle workspace.  Nothing here was produced by this
repository's code.
"""

# candle-core/tests/quantized_tests.rs:393-405  get_test_vector2(bound, size)
def ramp(bound: float, size: int):
    import numpy as np
    v = np.arange(size, dtype=np.float32)
    return ((v - np.float32(size / 2.0)) * np.float32(bound) / np.float32(size / 2.0)).astype(np.float32)


SPOT_INDICES = [0, 128, 256, 512, 800, 1023]
# quantized_tests.rs:583-587 (identical for Q4K / Q6K / Q8K)
RAMP_SRC_SPOTS = [-0.5, -0.375, -0.25, 0.0, 0.28125, 0.49902344]

# dtype name -> (max abs error on ramp(0.5), spot values rounded to 3 decimals, max abs error on ramp(128))
RAMP_ROUNDTRIP = {
    "Q4K": (0.017, [-0.5, -0.373, -0.25, 0.0, 0.288, 0.498], 4.5),     # quantized_tests.rs:581,589-592,607
    "Q6K": (0.008, [-0.497, -0.372, -0.25, -0.0, 0.284, 0.5], 2.0),    # quantized_tests.rs:675,683-686,701
    "Q8K": (0.008, [-0.5, -0.375, -0.25, -0.0, 0.281, 0.499], 0.6),    # quantized_tests.rs:722,730-733,748
}

# quantized_tests.rs:11-16, 428-469
GGML_TEST_SIZE = 32 * 128
GGML_MAX_QUANTIZATION_TOTAL_ERROR = 0.002
GGML_MAX_DOT_PRODUCT_ERROR = 0.02
# quantized_tests.rs:821-842
GGML_REFERENCE_MATMUL_ERROR = {"Q4K": 0.002425, "Q6K": 0.000952, "Q8_0": 0.000092, "Q4_0": 0.001143}
ERROR_LENIENCY = 0.00001  # quantized_tests.rs:896

# quantized_tests.rs:262-292: Q4_0 quantize->dequantize of 0..127
Q4_0_ROUNDTRIP_0_127 = [
    -0.0, -0.0, 3.875, 3.875, 3.875, 3.875, 7.75, 7.75, 7.75, 7.75, 11.625, 11.625, 11.625,
    11.625, 15.5, 15.5, 15.5, 15.5, 19.375, 19.375, 19.375, 19.375, 23.25, 23.25, 23.25,
    23.25, 27.125, 27.125, 27.125, 27.125, 31.0, 31.0, 31.5, 31.5, 31.5, 31.5, 39.375,
    39.375, 39.375, 39.375, 39.375, 39.375, 39.375, 39.375, 47.25, 47.25, 47.25, 47.25,
    47.25, 47.25, 47.25, 47.25, 55.125, 55.125, 55.125, 55.125, 55.125, 55.125, 55.125,
    55.125, 63.0, 63.0, 63.0, 63.0, 59.375, 59.375, 71.25, 71.25, 71.25, 71.25, 71.25,
    71.25, 71.25, 71.25, 71.25, 71.25, 71.25, 71.25, 83.125, 83.125, 83.125, 83.125,
    83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 83.125, 95.0, 95.0, 95.0, 95.0,
    95.0, 95.0, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 95.25, 111.125, 111.125,
    111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125, 111.125,
    111.125, 111.125, 111.125, 111.125, 111.125, 127.0, 127.0, 127.0, 127.0, 127.0, 127.0,
    127.0, 127.0,
]

# quantized_tests.rs:89-104,136-143: k_quants::matmul((3,64,4)) with Q4_0 weights, lhs = 0..191,
# rhs = 0..255, CPU path, results rounded to integers
Q4_0_MATMUL_RAMP_CPU = [
    85120.0, 214562.0, 345455.0, 474748.0, 213475.0, 604465.0, 1000686.0, 1388317.0,
    341876.0, 994283.0, 1655709.0, 2301518.0,
]
# quantized_tests.rs:149-169,200-207: lhs = v - 96, rhs = v - 256/3
Q4_0_MATMUL_NEG_CPU = [
    243524.0, -19596.0, -285051.0, -549815.0, 23777.0, 21651.0, 19398.0, 18367.0,
    -196472.0, 63012.0, 324585.0, 587902.0,
]

# candle-nn/tests/ops.rs:9-53: softmax_last_dim(log(data)), rounded to 4 decimals
SOFTMAX_DATA = [[[3.0, 1.0, 4.0], [1.0, 5.0, 9.0]], [[2.0, 1.0, 7.0], [8.0, 2.0, 8.0]]]
SOFTMAX_LAST_DIM_OF_LOG = [[[0.375, 0.125, 0.5], [0.0667, 0.3333, 0.6]], [[0.2, 0.1, 0.7], [0.4444, 0.1111, 0.4444]]]

# candle-core/tests/tensor_tests.rs:222-255: silu, rounded to 4 decimals
SILU_IN = [[-3.0, 1.0, 4.0, -0.1, 0.5], [2.7, -1.8, -0.28, 1.8, 2.8]]
SILU_OUT = [[-0.1423, 0.7311, 3.9281, -0.0475, 0.3112], [2.53, -0.2553, -0.1205, 1.5447, 2.6395]]

# candle-core/tests/tensor_tests.rs:1008-1023: zeros(6,3).index_add([5,0,1,0], arange(12).reshape(4,3), dim 0)
INDEX_ADD_IDS = [5, 0, 1, 0]
INDEX_ADD_OUT = [[12.0, 14.0, 16.0], [6.0, 7.0, 8.0], [0.0, 0.0, 0.0], [0.0, 0.0, 0.0], [0.0, 0.0, 0.0], [0.0, 1.0, 2.0]]

# candle-nn/tests/ops.rs:55-66: rms_norm(data, alpha = [1, 2, 3], eps = 1e-5), rounded to 4 decimals
RMS_NORM_DATA = [[[3.0, 1.0, 4.0], [1.0, 5.0, 9.0]], [[2.0, 1.0, 7.0], [8.0, 2.0, 8.0]]]
RMS_NORM_ALPHA = [1.0, 2.0, 3.0]
RMS_NORM_EPS = 1e-5
RMS_NORM_EXPECTED = [[[1.019, 0.6794, 4.0762], [0.1674, 1.6744, 4.521]],
                     [[0.4714, 0.4714, 4.9497], [1.206, 0.603, 3.6181]]]
