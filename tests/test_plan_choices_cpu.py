"""The choices a dense plan makes for a shape (tile code, K splits), checked without a GPU: they are plain functions of
the shape and the SM count, exported so that a binding can show or log them.  The expectations are the measured winners on
a 148-SM device (see the comments in csrc/gemm_umma.cu)."""
import pytest

SMS = 148


@pytest.fixture(scope="module")
def lib():
    from eider_b200 import _lib
    return _lib.load()


@pytest.mark.parametrize("m,n,code", [
    (512, 27648, 512),    # the prefill chunk: 216 pair tiles of 256 x 256, three turns of the 74 pairs
    (4096, 27648, 512),
    (16384, 27648, 512),
    (512, 5120, 384),     # 20 column tiles of 256 leave half of the pairs idle; 27 of 192 fill 54
    (1024, 5120, 384),
    (2048, 5120, 384),
    (8192, 5120, 512),
    (256, 27648, 384),    # 108 tiles need two turns either way; the narrower ones are shorter
    (128, 27648, 192),    # one row tile: no pairs; 144 tiles of 192 fit in one wave
    (384, 27648, 192),    # three row tiles: no pairs (an odd count below nine wastes half a pair tile)
    (128, 5120, 64),      # ties go to the narrower tile: more SMs streaming
    (512, 7168, 512),     # 76 narrow pair tiles would need a second turn
    (1, 16, 64),
])
def test_tile_choice(lib, m, n, code):
    assert lib.eider_b200_gemm_pick_tile(m, n, SMS) == code


def test_tile_choice_depends_on_the_device_size(lib):
    # half the SMs: 216 pair tiles take six turns, 288 narrow ones eight
    assert lib.eider_b200_gemm_pick_tile(512, 27648, 74) == 512
    assert lib.eider_b200_gemm_pick_tile(0, 128, SMS) == 0
    assert lib.eider_b200_gemm_pick_tile(128, 128, 1) == 0


@pytest.mark.parametrize("m,n,k,block_n,splits", [
    (128, 2560, 13824, 64, 3),     # 40 tiles, 54 K stages: three splits still fit in one wave
    (128, 5120, 13824, 64, 1),     # 80 tiles: two splits would need a second wave
    (128, 5120, 13824, 128, 3),    # the same shape on 128-wide tiles (40 of them)
    (256, 5120, 13824, 512, 1),    # more than one row tile: the partial sums cost more than they save
    (512, 27648, 5120, 512, 1),
    (128, 27648, 5120, 192, 1),    # 20 K stages: two splits of ten, but 288 items do not fit in one wave
    (64, 1024, 4096, 128, 1),      # 16 K stages: too short a K for a second launch to pay
])
def test_split_choice(lib, m, n, k, block_n, splits):
    assert lib.eider_b200_gemm_pick_k_splits(1, m, n, k, block_n, SMS) == splits


def test_split_choice_counts_fp8_stages_in_bytes(lib):
    # FP8 rows are twice as long in bytes: 13824 elements are 108 stages of 128 bytes
    assert lib.eider_b200_gemm_pick_k_splits(0, 128, 2560, 13824, 64, SMS) == 3
    assert lib.eider_b200_gemm_pick_k_splits(1, 128, 2560, 0, 64, SMS) == 0
