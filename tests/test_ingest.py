"""Host-side ingest against the reference's own tests and the CPU oracle (no GPU): the Nvfp4Artifact file
(crates/eider-format/src/nvfp4_artifact.rs), compressed-tensors globals, MXFP4 scale widening, the GGUF nibble repack
(crates/eider-format/src/gguf_nvfp4.rs:220-241), the requantisers and the prepared-layout cache."""
import struct

import numpy as np
import pytest

from eider_b200 import ingest
from eider_b200.ingest import FormatError, ModelOptNvfp4Linear, PreparedWeightCache, ShapeError


def test_artifact_round_trip_and_byte_layout(tmp_path):
    # crates/eider-format/src/nvfp4_artifact.rs round_trips_host_bytes
    a = ModelOptNvfp4Linear("model.layers.7.mlp.down_proj", 2, 16, np.arange(16, dtype=np.uint8).reshape(2, 8),
                            np.array([[11], [22]], np.uint8), 0.75, 1.25)
    path = tmp_path / "a.nvfp4"
    a.write_artifact(path)
    raw = path.read_bytes()
    # the reference's layout, field by field: magic, version, five u64, two f32, prefix, packed bytes, scales
    assert raw[:8] == b"EIDNVF4\0" and struct.unpack("<I", raw[8:12]) == (1,)
    assert struct.unpack("<5Q", raw[12:52]) == (2, 16, 16, 2, len(a.prefix))
    assert struct.unpack("<2f", raw[52:60]) == (0.75, 1.25)
    assert raw[60:60 + len(a.prefix)] == a.prefix.encode()
    assert raw[60 + len(a.prefix):] == bytes(range(16)) + bytes([11, 22])
    b = ModelOptNvfp4Linear.read_artifact(path)
    assert (b.prefix, b.out_features, b.in_features, b.weight_scale_2, b.input_scale) == (a.prefix, 2, 16, 0.75, 1.25)
    assert np.array_equal(b.packed_weight, a.packed_weight) and np.array_equal(b.weight_scale, a.weight_scale)
    assert not list(tmp_path.glob("*.tmp-*"))  # written through a temporary file that is gone afterwards


def test_artifact_rejects_bad_files(tmp_path):
    a = ModelOptNvfp4Linear("p", 2, 16, np.zeros((2, 8), np.uint8), np.zeros((2, 1), np.uint8))
    path = tmp_path / "a.nvfp4"
    a.write_artifact(path)
    raw = path.read_bytes()
    (tmp_path / "trunc").write_bytes(raw[:-1])
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.read_artifact(tmp_path / "trunc")
    (tmp_path / "magic").write_bytes(b"X" + raw[1:])
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.read_artifact(tmp_path / "magic")
    (tmp_path / "version").write_bytes(raw[:8] + struct.pack("<I", 2) + raw[12:])
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.read_artifact(tmp_path / "version")
    with pytest.raises(OSError):
        ModelOptNvfp4Linear.read_artifact(tmp_path / "missing")
    for bad in (ModelOptNvfp4Linear("p", 2, 24, np.zeros((2, 12), np.uint8), np.zeros((2, 1), np.uint8)),       # K % 16
                ModelOptNvfp4Linear("p", 2, 16, np.zeros((2, 7), np.uint8), np.zeros((2, 1), np.uint8))):       # byte count
        with pytest.raises(ShapeError):
            bad.write_artifact(tmp_path / "bad")
    for bad in (ModelOptNvfp4Linear("", 2, 16, np.zeros((2, 8), np.uint8), np.zeros((2, 1), np.uint8)),         # empty prefix
                ModelOptNvfp4Linear("p", 2, 16, np.zeros((2, 8), np.uint8), np.zeros((2, 1), np.uint8), float("nan"))):
        with pytest.raises(FormatError):
            bad.write_artifact(tmp_path / "bad")


def test_compressed_tensors_globals_are_reciprocals():
    lin = ModelOptNvfp4Linear.from_compressed_tensors("p", np.zeros((4, 8), np.uint8), np.zeros((4, 1), np.uint8), 2688.0, 8.0)
    assert lin.weight_scale_2 == np.float32(1.0) / np.float32(2688.0) and lin.input_scale == 0.125
    assert (lin.out_features, lin.in_features) == (4, 16)
    for wg, ig in ((0.0, 1.0), (1.0, -2.0), (float("inf"), 1.0), (1.0, float("nan"))):
        with pytest.raises(FormatError):
            ModelOptNvfp4Linear.from_compressed_tensors("p", np.zeros((4, 8), np.uint8), np.zeros((4, 1), np.uint8), wg, ig)


def test_mxfp4_scales_widen_to_k16(oracle):
    # E8M0 127 = 1.0 -> UE4M3 0x38, 128 = 2.0 -> 0x40, 118 = 2^-9 -> 0x01 (the smallest subnormal), 135 = 256 -> 0x78
    w = np.zeros((2, 32), np.uint8)
    lin = ModelOptNvfp4Linear.from_mxfp4("p", w, np.array([[127, 128], [118, 135]], np.uint8))
    assert lin.in_features == 64 and lin.weight_scale.tolist() == [[0x38, 0x38, 0x40, 0x40], [0x01, 0x01, 0x78, 0x78]]
    for code in (127, 128, 118, 135):
        assert oracle.e4m3_value(oracle.ue4m3_code(oracle.e8m0_value(code))) == oracle.e8m0_value(code)
    for bad in (255, 117, 136):  # NaN, below the smallest subnormal, above 448's power of two
        with pytest.raises(FormatError):
            ModelOptNvfp4Linear.from_mxfp4("p", w, np.array([[127, bad], [127, 127]], np.uint8))
    with pytest.raises(ShapeError):
        ModelOptNvfp4Linear.from_mxfp4("p", np.zeros((2, 24), np.uint8), np.zeros((2, 1), np.uint8))


def test_gguf_unpack_preserves_every_nibble_and_scale():
    # crates/eider-format/src/gguf_nvfp4.rs:220-241
    blocks = bytearray()
    for block in range(4):
        blocks += bytes([0, 1 + block, 0x38, 0x7E])
        for group in range(4):
            for j in range(8):
                blocks.append(((j + group + block) & 15) | (((j + 8 + group + block) & 15) << 4))
    out = ModelOptNvfp4Linear.from_gguf_blocks(np.frombuffer(bytes(blocks), np.uint8), 2, 128, 0.125)
    packed, scales = out.packed_weight.reshape(-1), out.weight_scale.reshape(-1)
    for i in range(256):
        block, group, lane = i // 64, (i % 64) // 16, i % 16
        assert (packed[i // 2] >> ((i % 2) * 4)) & 15 == (lane + group + block) & 15
        assert scales[i // 16] == blocks[block * 36 + group]
    assert out.weight_scale_2 == 0.125 and out.input_scale == 1.0
    # crates/eider-format/src/gguf_nvfp4.rs rejects_bad_lengths_tails_and_scales
    good = np.frombuffer(bytes(blocks), np.uint8)
    for rows, cols, scale in ((1, 16, 1.0), (0, 64, 1.0), (1, 64, 0.0), (1, 64, float("nan"))):
        with pytest.raises(FormatError):
            ModelOptNvfp4Linear.from_gguf_blocks(good[:36], rows, cols, scale)
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.from_gguf_blocks(good[:35], 1, 64, 1.0)
    bad = good[:36].copy()
    bad[2] = 0x7F
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.from_gguf_blocks(bad, 1, 64, 1.0)


def test_requantisers_match_the_oracle(oracle):
    rng = np.random.default_rng(0)
    # the reference's own known answer: every E2M1 value once, scale byte 0x38 (crates/eider-format/src/modelopt.rs:1281-1294)
    row = np.array([[0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]], np.float32)
    lin = ModelOptNvfp4Linear.quantize_f32("p", row)
    assert lin.weight_scale.tolist() == [[0x38]]
    assert lin.packed_weight.tolist() == [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]]
    w = (rng.standard_normal((130, 272)) * np.exp(rng.uniform(-3, 3, (130, 1)))).astype(np.float32)
    w[3, :16] = 0.0
    w[5, 7] = np.inf
    p_ref, s_ref, _ = oracle.quantize_weight(w, 1.0)
    lin = ModelOptNvfp4Linear.quantize_f32("p", w)
    assert np.array_equal(lin.packed_weight, p_ref) and np.array_equal(lin.weight_scale, s_ref)
    wb = oracle.bf16_round(w)
    wb[5, 7] = 1.0
    p_ref, s_ref, _ = oracle.quantize_weight(wb, 1.0)
    lin = ModelOptNvfp4Linear.quantize_bf16("p", oracle.f32_to_bf16_bits(wb))
    assert np.array_equal(lin.packed_weight, p_ref) and np.array_equal(lin.weight_scale, s_ref)
    # FP8 sources: per-tensor scale, per-channel scales, 128 x 128 E8M0 blocks
    codes = rng.integers(0, 256, (256, 384)).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x38  # no NaN codes
    vals = oracle.e4m3_decode(codes)
    lin = ModelOptNvfp4Linear.quantize_fp8("p", codes, 0.0625)
    p_ref, s_ref, _ = oracle.quantize_weight(vals * np.float32(0.0625), 1.0)
    assert np.array_equal(lin.packed_weight, p_ref) and np.array_equal(lin.weight_scale, s_ref)
    ch = rng.uniform(0.01, 0.1, 256).astype(np.float32)
    lin = ModelOptNvfp4Linear.quantize_fp8("p", codes, 1.0, ch)
    p_ref, s_ref, _ = oracle.quantize_weight(vals * ch[:, None], 1.0)
    assert np.array_equal(lin.packed_weight, p_ref) and np.array_equal(lin.weight_scale, s_ref)
    blk = rng.integers(120, 130, (2, 3)).astype(np.uint8)
    scale = np.array([[oracle.e8m0_value(int(c)) for c in r] for r in blk], np.float32)
    lin = ModelOptNvfp4Linear.quantize_block_scaled_fp8("p", codes, blk)
    p_ref, s_ref, _ = oracle.quantize_weight(vals * np.kron(scale, np.ones((128, 128), np.float32)), 1.0)
    assert np.array_equal(lin.packed_weight, p_ref) and np.array_equal(lin.weight_scale, s_ref)
    blk[0, 0] = 255
    with pytest.raises(FormatError):
        ModelOptNvfp4Linear.quantize_block_scaled_fp8("p", codes, blk)
    with pytest.raises(ShapeError):
        ModelOptNvfp4Linear.quantize_f32("p", np.zeros((2, 24), np.float32))


def test_prepared_cache_round_trip(tmp_path, oracle):
    rng = np.random.default_rng(1)
    w = rng.standard_normal((130, 96)).astype(np.float32)  # 130 rows: the second scale tile is mostly padding
    lin = ModelOptNvfp4Linear.quantize_f32("p", w)
    lin.weight_scale_2 = 0.5
    tiled = lin.tiled_scales()
    assert np.array_equal(tiled, oracle.scales_to_tiled(lin.weight_scale, 130, 96))
    # crates/eider-format/src/modelopt.rs:1323-1330: packed[0] = src[0], packed[16] = src[blocks], packed[4] = src[32 * blocks]
    blocks = 96 // 16
    src = lin.weight_scale.reshape(-1)
    assert tiled[0] == src[0] and tiled[16] == src[blocks] and tiled[4] == src[32 * blocks]
    path = tmp_path / "w.b2p"
    PreparedWeightCache.write(path, lin)
    assert PreparedWeightCache.matches(path, 130, 96) and not PreparedWeightCache.matches(path, 130, 128)
    raw = path.read_bytes()
    assert raw[:8] == b"EIDB2P01" and struct.unpack("<I4Qf", raw[8:48]) == (1, 130, 96, 130 * 48, tiled.size, 0.5)
    pw, ts, w2 = PreparedWeightCache.read(path, 130, 96)
    assert np.array_equal(pw, lin.packed_weight) and np.array_equal(ts, tiled) and w2 == 0.5
    (tmp_path / "short").write_bytes(raw[:-3])
    assert not PreparedWeightCache.matches(tmp_path / "short", 130, 96)
    with pytest.raises(FormatError):
        PreparedWeightCache.read(tmp_path / "short", 130, 96)
    assert not PreparedWeightCache.matches(tmp_path / "nope", 130, 96)
