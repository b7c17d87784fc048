"""Host-side weight ingest: the records and conversions between a checkpoint and the device image of an NVFP4 linear.

Mirrors crates/eider-format of the reference (Nvfp4Artifact, the compressed-tensors / MXFP4 / GGUF importers, the
requantisers of ModelOptNvfp4Linear) and adds the prepared-layout cache of this library.  Everything is computed by the
C-ABI host entry points of libeider_b200.so on numpy arrays; no GPU is needed.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib


class ShapeError(ValueError):
    """crates/eider-format Error::Shape."""


class FormatError(ValueError):
    """crates/eider-format Error::Format."""


def _raise(code: int, what: str) -> None:
    if code == 0:
        return
    raise {1: ShapeError, 2: FormatError}.get(code, OSError)(f"{what} failed (code {code})")


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class ModelOptNvfp4Linear:
    """Host record of one NVFP4 linear (crates/eider-format/src/modelopt.rs:11-26): packed E2M1 bytes [out, in/2], E4M3
    K16 scales [out, in/16], the tensor-wide weight scale and the static activation scale."""
    prefix: str
    out_features: int
    in_features: int
    packed_weight: np.ndarray
    weight_scale: np.ndarray
    weight_scale_2: float = 1.0
    input_scale: float = 1.0

    # -- Nvfp4Artifact (crates/eider-format/src/nvfp4_artifact.rs) ------------------------------------------------
    def write_artifact(self, path: str) -> None:
        pw, ws = _u8(self.packed_weight).reshape(-1), _u8(self.weight_scale).reshape(-1)
        _raise(_lib.load().eider_b200_nvfp4_artifact_write(str(path).encode(), self.prefix.encode(), self.out_features,
                                                           self.in_features, _p(pw), pw.size, _p(ws), ws.size,
                                                           self.weight_scale_2, self.input_scale), "artifact write")

    @staticmethod
    def read_artifact(path: str) -> "ModelOptNvfp4Linear":
        lib = _lib.load()
        v = [C.c_uint64() for _ in range(5)]
        w2, isc = C.c_float(), C.c_float()
        _raise(lib.eider_b200_nvfp4_artifact_read_header(str(path).encode(), *[C.byref(x) for x in v], C.byref(w2), C.byref(isc)),
               "artifact header")
        out_f, in_f, packed_len, scale_len, prefix_len = [int(x.value) for x in v]
        prefix = C.create_string_buffer(prefix_len + 1)
        pw, ws = np.empty(packed_len, np.uint8), np.empty(scale_len, np.uint8)
        _raise(lib.eider_b200_nvfp4_artifact_read(str(path).encode(), prefix, prefix_len + 1, _p(pw), pw.size, _p(ws), ws.size),
               "artifact read")
        return ModelOptNvfp4Linear(prefix.value.decode(), out_f, in_f, pw.reshape(out_f, in_f // 2), ws.reshape(out_f, in_f // 16),
                                   float(w2.value), float(isc.value))

    # -- importers -------------------------------------------------------------------------------------------------
    @staticmethod
    def from_compressed_tensors(prefix, weight_packed, weight_scale, weight_global_scale: float, input_global_scale: float):
        """compressed-tensors NVFP4: the two globals are divisors (crates/eider-format/src/modelopt.rs:480-519)."""
        w2, isc = C.c_float(), C.c_float()
        _raise(_lib.load().eider_b200_compressed_tensors_globals(weight_global_scale, input_global_scale, C.byref(w2), C.byref(isc)),
               "compressed-tensors globals")
        pw = _u8(weight_packed)
        return ModelOptNvfp4Linear(prefix, pw.shape[0], pw.shape[1] * 2, pw, _u8(weight_scale), float(w2.value), float(isc.value))

    @staticmethod
    def from_mxfp4(prefix, weight, e8m0_scales):
        """MXFP4 (K32 E8M0 scales) -> NVFP4 K16 records (crates/eider-format/src/modelopt.rs:173-248)."""
        pw, sc = _u8(weight), _u8(e8m0_scales)
        out_f, in_f = pw.shape[0], pw.shape[1] * 2
        if in_f % 32 != 0 or sc.shape != (out_f, in_f // 32):
            raise ShapeError(f"MXFP4 needs in_features % 32 == 0 and scales [{out_f}, {in_f // 32}], got {sc.shape}")
        ws = np.empty((out_f, in_f // 16), np.uint8)
        _raise(_lib.load().eider_b200_mxfp4_scales_to_nvfp4(_p(sc), sc.size, _p(ws)), "MXFP4 scale widening")
        return ModelOptNvfp4Linear(prefix, out_f, in_f, pw, ws, 1.0, 1.0)

    @staticmethod
    def from_gguf_blocks(blocks, out_features: int, in_features: int, global_scale: float):
        """GGML NVFP4 blocks -> row-major ModelOpt storage, no requantisation (crates/eider-format/src/gguf_nvfp4.rs:12-64)."""
        b = _u8(blocks).reshape(-1)
        pw = np.empty((out_features, max(in_features // 2, 1)), np.uint8)
        ws = np.empty((out_features, max(in_features // 16, 1)), np.uint8)
        _raise(_lib.load().eider_b200_gguf_nvfp4_unpack(_p(b), b.size, out_features, in_features, global_scale, _p(pw), _p(ws)),
               "GGUF NVFP4 unpack")
        return ModelOptNvfp4Linear("", out_features, in_features, pw, ws, float(global_scale), 1.0)

    # -- requantisers (crates/eider-format/src/modelopt.rs:524-716), unit global scale --------------------------------
    @staticmethod
    def _requantize(prefix, kind, values, out_f, in_f, channel=None, tensor_scale=1.0, block=None):
        if in_f % 16 != 0 or out_f == 0 or values.size != out_f * in_f:
            raise ShapeError(f"NVFP4 quantization needs [{out_f}, {in_f}] values with in_features % 16 == 0")
        pw, ws = np.empty((out_f, in_f // 2), np.uint8), np.empty((out_f, in_f // 16), np.uint8)
        _raise(_lib.load().eider_b200_nvfp4_requantize_host(kind, _p(values), None if channel is None else _p(channel), tensor_scale,
                                                            None if block is None else _p(block), out_f, in_f, _p(pw), _p(ws)),
               "NVFP4 requantisation")
        return ModelOptNvfp4Linear(prefix, out_f, in_f, pw, ws, 1.0, 1.0)

    @staticmethod
    def quantize_f32(prefix, values):
        v = np.ascontiguousarray(values, np.float32)
        return ModelOptNvfp4Linear._requantize(prefix, 0, v, v.shape[0], v.shape[1])

    @staticmethod
    def quantize_bf16(prefix, bits):
        v = np.ascontiguousarray(bits, np.uint16)
        return ModelOptNvfp4Linear._requantize(prefix, 1, v, v.shape[0], v.shape[1])

    @staticmethod
    def quantize_fp8(prefix, codes, weight_scale: float = 1.0, channel_weight_scale=None):
        v = _u8(codes)
        ch = None if channel_weight_scale is None else np.ascontiguousarray(channel_weight_scale, np.float32)
        if ch is not None and ch.size != v.shape[0]:
            raise ShapeError("one channel scale per output feature")
        return ModelOptNvfp4Linear._requantize(prefix, 2, v, v.shape[0], v.shape[1], channel=ch, tensor_scale=weight_scale)

    @staticmethod
    def quantize_block_scaled_fp8(prefix, codes, e8m0_block_scales):
        v, b = _u8(codes), _u8(e8m0_block_scales)
        if v.shape[0] % 128 or v.shape[1] % 128 or b.size != (v.shape[0] // 128) * (v.shape[1] // 128):
            raise ShapeError("block-scaled FP8 needs 128-aligned dimensions and one E8M0 scale per 128 x 128 block")
        return ModelOptNvfp4Linear._requantize(prefix, 3, v, v.shape[0], v.shape[1], block=b)

    # -- prepared layout ---------------------------------------------------------------------------------------------
    def tiled_scales(self) -> np.ndarray:
        """The 128 x 4 tiled scale image the tensor-core kernels read (modelopt_scales_to_cublaslt)."""
        lib = _lib.load()
        out = np.empty(lib.eider_b200_nvfp4_scale_layout_len(self.out_features, self.in_features), np.uint8)
        ws = _u8(self.weight_scale).reshape(-1)
        lib.eider_b200_nvfp4_scales_to_tiled_host(_p(ws), _p(out), self.out_features, self.in_features)
        return out


class PreparedWeightCache:
    """"EIDB2P01" files: packed bytes + tiled scales of one linear, so that a restart skips the scale repack; the
    counterpart of the reference's prepared-weight cache (crates/eider-cuda/src/kernels/sm121_w4a16.rs:146-240)."""

    @staticmethod
    def write(path: str, linear: ModelOptNvfp4Linear) -> None:
        pw = _u8(linear.packed_weight).reshape(-1)
        tiled = linear.tiled_scales()
        _raise(_lib.load().eider_b200_prepared_cache_write(str(path).encode(), linear.out_features, linear.in_features, _p(pw), _p(tiled),
                                                           linear.weight_scale_2), "prepared cache write")

    @staticmethod
    def matches(path: str, out_features: int, in_features: int) -> bool:
        return bool(_lib.load().eider_b200_prepared_cache_matches(str(path).encode(), out_features, in_features))

    @staticmethod
    def read(path: str, out_features: int, in_features: int):
        """-> (packed [out, in/2] u8, tiled scales u8, weight_scale_2)."""
        lib = _lib.load()
        pw = np.empty((out_features, in_features // 2), np.uint8)
        tiled = np.empty(lib.eider_b200_nvfp4_scale_layout_len(out_features, in_features), np.uint8)
        w2 = C.c_float()
        _raise(lib.eider_b200_prepared_cache_read(str(path).encode(), out_features, in_features, _p(pw), _p(tiled), C.byref(w2)),
               "prepared cache read")
        return pw, tiled, float(w2.value)
