"""Cross-checks the restated codecs against the reference's own C++ conversion oracle
(crates/eider-cuda/native/fp4_oracle.cpp compiled into oracle/_ref/ by oracle/Makefile),
the same comparison the reference makes in crates/eider-cuda/src/format.rs:470-518."""
import math
import struct

import numpy as np
import pytest

from tests.test_oracle_golden import E2M1_VALUES


@pytest.fixture(scope="module")
def ref(oracle):
    lib = oracle.load_reference_codec()
    if lib is None:
        pytest.skip("oracle/_ref/libfp4_oracle.so not built (reference tree absent)")
    return lib


def test_e2m1_matches_reference_header_conversion(oracle, ref):
    for v in E2M1_VALUES:
        assert oracle.e2m1_code(v) == (ref.infer_cuda_e2m1_rn(v) & 0x0F), v


def test_ue4m3_matches_reference_for_positive_scales(oracle, ref):
    for v in [0.0, 0.0001, 0.001, 0.01, 0.1, 0.25, 0.5, 1.0, 2.0, 6.0, 16.0, 448.0, 1000.0]:
        assert oracle.ue4m3_code(v) == ref.infer_cuda_e4m3_satfinite(v), v


def test_codecs_match_reference_on_dense_sweep(oracle, ref):
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 3.0,
        np.exp(rng.uniform(-12, 7, 4000)).astype(np.float32),
        # every E4M3 midpoint and value, to exercise ties
        np.array([(oracle.e4m3_value(c) + oracle.e4m3_value(c + 1)) / 2 for c in range(0, 0x7E)], np.float32),
        np.array([oracle.e4m3_value(c) for c in range(0, 0x7F)], np.float32),
    ])
    for v in vals.tolist():
        assert oracle.e2m1_code(v) == (ref.infer_cuda_e2m1_rn(v) & 0x0F), v
        if v >= 0:
            assert oracle.ue4m3_code(v) == ref.infer_cuda_e4m3_satfinite(v), v
        assert oracle.e4m3_code(v) == ref.infer_cuda_e4m3_satfinite(v) or v == 0.0, v
