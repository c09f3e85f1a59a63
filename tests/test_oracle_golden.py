"""The CPU oracle against the vectors of the reference's own unit tests.

tests/golden/reference_cases.json holds, for every graph the reference's
conv2d / depthwise / pooling / fully-connected / softmax tests build, the
tensors, the node parameters, the inputs and the vector the test compares with
(see tests/golden/make_goldens.py).  Here each case is rebuilt through the C
ABI on the oracle library and checked against that vector.

Tolerances: the fixture's own (0 for EXPECT_EQ on integers, the ArraysMatch
argument otherwise), except that float32 results the reference compares with
EXPECT_EQ are compared within 1e-5: exact float equality depends on the
hardware's exp/accumulation and cannot be pinned by a different machine.
"""
import numpy as np
import pytest

import oracle_paths

FLOAT_EXACT_TOL = 1e-5


def check_case(lib, case):
    g, inputs, expects, _ = oracle_paths.graph_from_case(lib, case)
    try:
        g.compile()
        for tid, arr in inputs:
            g.write(tid, arr)
        g.run()
        assert expects, "case without expectation"
        for tid, want, tol in expects:
            got = g.read(tid).reshape(-1)
            assert got.shape == want.shape
            if want.dtype == np.float32:
                np.testing.assert_allclose(got, want, rtol=0, atol=max(tol, FLOAT_EXACT_TOL))
            else:
                diff = np.abs(got.astype(np.int64) - want.astype(np.int64)).max()
                assert diff <= tol, "max |diff| %d > %g" % (diff, tol)
    finally:
        g.close()


def test_fixture_is_complete(reference_cases):
    names = {c["name"] for c in reference_cases}
    # the quantized tests that pin the integer path
    for must in ["Conv2d.shape_4_2_1_2_uint8_QuantizedTest1", "Conv2d.shape_4_2_1_2_uint8_QuantizedTest2",
                 "Conv2d.shape_6_3_1_1_uint8_AnisotropicStridesQuantizedTest",
                 "Conv2d.shape_9_9_1_1_uint8_DilationQuantizedTest",
                 "Conv2d.shape_3_2_2_1_int8_QuantizedPerTensorTest",
                 "Conv2d.shape_3_2_2_1_int8_QuantizedPerChannelTest",
                 "Conv2d.shape_w_h_128_1_ksize_1_1_stride_2_int8_QuantizedPerChannelTest",
                 "DepthwiseConv.shape_2_3_2_1_uint8_QuantizedTest",
                 "DepthwiseConv.shape_3_3_8_1_int8_PerChannelSameTest",
                 "AVG.shape_3_3_1_1_uint8_kernel_2_stride_1",
                 "AVG_ANDROID.shape_60_52_3_5_uint8_kernel_35_stride_5"]:
        assert must in names
    assert len(reference_cases) >= 100


def test_oracle_matches_reference_vectors(oracle_lib, reference_cases):
    failures = []
    for case in reference_cases:
        try:
            check_case(oracle_lib, case)
        except AssertionError as e:
            failures.append("%s: %s" % (case["name"], str(e).splitlines()[0]))
    assert not failures, "\n".join(failures)


def test_recorded_oracle_outputs_are_reproduced(oracle_lib, reference_cases):
    """The outputs stored in the fixture are what the oracle produces today (bit for bit)."""
    for case in reference_cases[::7]:
        g, inputs, _, recorded = oracle_paths.graph_from_case(oracle_lib, case)
        g.compile()
        for tid, arr in inputs:
            g.write(tid, arr)
        g.run()
        for tid, want in recorded.items():
            got = g.read(tid).reshape(-1)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), case["name"]
        g.close()
