"""ctypes front end of the test-only checkers in this directory.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference arm.  The shipped package never imports it.

``cpu``  -> oracle/_build/libp92_oracle.so, the CPU restatement (p92_moe_oracle.cpp)
``pin``  -> oracle/_build/libp92_cvt_pin.so, the CUDA toolkit's host E2M1/E4M3 conversions
``ref``  -> oracle/_ref/libp92_ref.so, the reference's own cuda/nvfp4_ops.cu compiled for
            sm_100a plus ref_driver.cu; only present when it was built where the
            reference tree is mounted (the binary travels, the sources never do)
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
CPU_LIB = os.path.join(_HERE, "_build", "libp92_oracle.so")
PIN_LIB = os.path.join(_HERE, "_build", "libp92_cvt_pin.so")
REF_LIB = os.path.join(_HERE, "_ref", "libp92_ref.so")

_cpu = None
_pin = None
_ref = None

u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
c_int, c_long, c_float, c_void_p = ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_void_p


def build(ref: bool = False) -> None:
    """Runs the Makefile (CPU oracle + conversion pin; with ref=True also oracle/_ref)."""
    subprocess.run(["make", "-s", "-C", _HERE] + (["ref"] if ref else []), check=True)


def cpu() -> ctypes.CDLL:
    global _cpu
    if _cpu is None:
        if not os.path.exists(CPU_LIB):
            build()
        lib = ctypes.CDLL(CPU_LIB)
        lib.orc_threads.restype = c_int
        lib.orc_set_threads.argtypes = [c_int]
        lib.orc_float_to_bf16.argtypes = [f32p, u16p, c_long]
        lib.orc_bf16_to_float.argtypes = [u16p, f32p, c_long]
        lib.orc_encode_e4m3_array.argtypes = [f32p, u8p, c_long]
        lib.orc_encode_e2m1_array.argtypes = [f32p, u8p, c_long]
        lib.orc_decode_e4m3.argtypes = [ctypes.c_uint8]
        lib.orc_decode_e4m3.restype = c_float
        lib.orc_decode_e2m1.argtypes = [ctypes.c_uint8]
        lib.orc_decode_e2m1.restype = c_float
        lib.orc_router_logits.argtypes = [u16p, u16p, f32p, c_int, c_int, c_int, c_int]
        lib.orc_router_top8.argtypes = [f32p, f32p, i32p, f32p, c_void_p, c_int, c_int, c_float]
        lib.orc_permute.argtypes = [i32p, c_int, c_int, i32p, c_void_p, i32p, i32p]
        lib.orc_permute_ranking.argtypes = [i32p, c_int, i32p]
        lib.orc_nvfp4_quantize.argtypes = [u16p, u8p, u8p, c_long, c_float]
        lib.orc_nvfp4_pack_weight.argtypes = [u16p, u8p, u8p, c_long]
        lib.orc_nvfp4_pack_weight.restype = c_float
        lib.orc_swizzled_scale_bytes.argtypes = [c_int, c_int]
        lib.orc_swizzled_scale_bytes.restype = c_long
        lib.orc_swizzle_scales.argtypes = [u8p, u8p, c_int, c_int]
        lib.orc_nvfp4_gemv.argtypes = [u8p, u8p, u8p, u8p, u16p, c_int, c_int, c_int, c_float]
        lib.orc_swiglu.argtypes = [u16p, u16p, u16p, c_long]
        lib.orc_expert_combine_rows.argtypes = [u16p, f32p, u16p, c_int, c_int, c_int]
        lib.orc_scatter_add_scaled_rows.argtypes = [u16p, u16p, i32p, f32p, c_int, c_int]
        lib.orc_add_inplace.argtypes = [u16p, u16p, c_long]
        lib.orc_dense_forward.argtypes = [u16p, u8p, u8p, f32p, c_long, c_long, u16p, c_int, c_int, c_int]
        lib.orc_rmsnorm.argtypes = [u16p, u16p, u16p, c_int, c_int, c_float]
        lib.orc_moe_forward.argtypes = [u16p, u16p, f32p, u8p, u8p, f32p, c_long, c_long, u16p, c_int, c_int, c_int,
                                        c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.orc_fnv1a_bf16.argtypes = [u16p, c_long]
        lib.orc_fnv1a_bf16.restype = ctypes.c_uint64
        _cpu = lib
    return _cpu


def pin() -> ctypes.CDLL:
    global _pin
    if _pin is None:
        if not os.path.exists(PIN_LIB):
            build()
        lib = ctypes.CDLL(PIN_LIB)
        lib.pin_encode_e4m3_array.argtypes = [f32p, u8p, c_long]
        lib.pin_encode_e2m1x2_array.argtypes = [f32p, u8p, c_long]
        lib.pin_decode_e4m3.argtypes = [ctypes.c_uint8]
        lib.pin_decode_e4m3.restype = c_float
        lib.pin_decode_e2m1.argtypes = [ctypes.c_uint8]
        lib.pin_decode_e2m1.restype = c_float
        _pin = lib
    return _pin


def have_ref() -> bool:
    return os.path.exists(REF_LIB)


def ref() -> ctypes.CDLL:
    """The reference's own kernels on the GPU (device pointers, C ABI of ref_driver.cu)."""
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(REF_LIB)
        P = c_void_p
        lib.ref_bf16_gemv_f32.argtypes = [P, P, P, c_int, c_int, P]
        lib.ref_bf16_gemm_f32.argtypes = [P, P, P, c_int, c_int, c_int, P]
        lib.ref_router_top8_rows.argtypes = [P, P, P, P, c_int, c_float, P]
        lib.ref_router_top8.argtypes = [P, P, P, P, c_float, P]
        lib.ref_nvfp4_quantize.argtypes = [P, P, P, c_int, c_float, P]
        lib.ref_nvfp4_swizzled_scale_bytes.argtypes = [c_int, c_int]
        lib.ref_nvfp4_swizzled_scale_bytes.restype = c_long
        lib.ref_nvfp4_swizzle_scales.argtypes = [P, P, c_int, c_int, P]
        lib.ref_nvfp4_gemv.argtypes = [P, P, P, P, P, c_int, c_int, c_float, P]
        lib.ref_swiglu.argtypes = [P, P, P, c_int, P]
        lib.ref_expert_combine_rows.argtypes = [P, P, P, c_int, c_int, c_int, P]
        lib.ref_add_inplace.argtypes = [P, P, c_int, P]
        if hasattr(lib, "ref_rmsnorm"):
            lib.ref_rmsnorm.argtypes = [P, P, P, c_int, c_int, c_float, P]
        lib.ref_moe_forward_rows.argtypes = [P, P, P, P, P, f32p, c_long, c_long, P, c_int, c_int, c_int, c_int,
                                             c_float, P, P, P, P, P]
        _ref = lib
    return _ref


# ---- numpy conveniences -----------------------------------------------------

def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    cpu().orc_float_to_bf16(a.reshape(-1), out.reshape(-1), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    cpu().orc_bf16_to_float(a.reshape(-1), out.reshape(-1), a.size)
    return out


def router_logits(x: np.ndarray, w: np.ndarray, gemv_order: bool | None = None) -> np.ndarray:
    rows, columns = x.shape
    experts = w.shape[0]
    out = np.empty((rows, experts), dtype=np.float32)
    if gemv_order is None:
        gemv_order = rows == 1
    cpu().orc_router_logits(x, w, out, rows, experts, columns, int(gemv_order))
    return out


def router_top8(logits: np.ndarray, bias: np.ndarray, routed_scale: float = 2.5):
    rows, experts = logits.shape
    ids = np.empty((rows, 8), dtype=np.int32)
    weights = np.empty((rows, 8), dtype=np.float32)
    margin = np.empty(rows, dtype=np.float32)
    cpu().orc_router_top8(np.ascontiguousarray(logits), np.ascontiguousarray(bias), ids, weights,
                          margin.ctypes.data, rows, experts, routed_scale)
    return ids, weights, margin


def permute(ids: np.ndarray, experts: int = 256):
    flat = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    n = flat.size
    order = np.empty(n, dtype=np.int32)
    position = np.empty(n, dtype=np.int32)
    counts = np.empty(experts, dtype=np.int32)
    offsets = np.empty(experts + 1, dtype=np.int32)
    cpu().orc_permute(flat, n, experts, order, position.ctypes.data, counts, offsets)
    return order, position, counts, offsets


def nvfp4_quantize(x: np.ndarray, global_scale: float = 1.0):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    groups = x.size // 16
    packed = np.empty(x.size // 2, dtype=np.uint8)
    scales = np.empty(groups, dtype=np.uint8)
    cpu().orc_nvfp4_quantize(x.reshape(-1), packed, scales, groups, global_scale)
    return packed.reshape(x.shape[:-1] + (x.shape[-1] // 2,)), scales.reshape(x.shape[:-1] + (x.shape[-1] // 16,))


def nvfp4_pack_weight(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.uint16)
    packed = np.empty(w.size // 2, dtype=np.uint8)
    scales = np.empty(w.size // 16, dtype=np.uint8)
    alpha = cpu().orc_nvfp4_pack_weight(w.reshape(-1), packed, scales, w.size)
    return (packed.reshape(w.shape[0], w.shape[1] // 2), scales.reshape(w.shape[0], w.shape[1] // 16),
            np.float32(alpha))


def swizzle_scales(linear: np.ndarray) -> np.ndarray:
    rows, cols = linear.shape
    out = np.empty(cpu().orc_swizzled_scale_bytes(rows, cols), dtype=np.uint8)
    cpu().orc_swizzle_scales(np.ascontiguousarray(linear), out, rows, cols)
    return out


def rmsnorm(x: np.ndarray, weight: np.ndarray, epsilon: float = 1.0e-5) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty_like(x)
    cpu().orc_rmsnorm(x.reshape(-1), np.ascontiguousarray(weight, dtype=np.uint16), out.reshape(-1), x.shape[0], x.shape[1],
                      epsilon)
    return out


def dense_forward(x, weights, scales, alphas, hidden, intermediate):
    """weights [3, stride] packed (gate, up, down), scales [3, stride] linear, alphas [3]."""
    rows = x.shape[0]
    out = np.empty((rows, hidden), dtype=np.uint16)
    cpu().orc_dense_forward(np.ascontiguousarray(x), weights.reshape(-1), scales.reshape(-1),
                            np.ascontiguousarray(alphas, dtype=np.float32), weights.shape[1], scales.shape[1], out, rows,
                            hidden, intermediate)
    return out


def moe_forward(x, router_w, bias, weights, scales, alphas, hidden, intermediate, experts=256,
                routed_scale=2.5, host_law=False, want_intermediates=False):
    """weights [ (experts+1)*3, stride ] uint8 packed, scales likewise (linear), alphas [(experts+1)*3] f32."""
    rows = x.shape[0]
    out = np.empty((rows, hidden), dtype=np.uint16)
    extra = {}
    ptrs = [None, None, None, None]
    if want_intermediates:
        extra = {
            "logits": np.empty((rows, experts), dtype=np.float32),
            "expert_ids": np.empty((rows, 8), dtype=np.int32),
            "expert_weights": np.empty((rows, 8), dtype=np.float32),
            "mixed": np.empty((rows * 8, hidden), dtype=np.uint16),
        }
        ptrs = [extra[k].ctypes.data for k in ("logits", "expert_ids", "expert_weights", "mixed")]
    cpu().orc_moe_forward(np.ascontiguousarray(x), np.ascontiguousarray(router_w), np.ascontiguousarray(bias),
                          weights.reshape(-1), scales.reshape(-1), np.ascontiguousarray(alphas, dtype=np.float32),
                          weights.shape[1], scales.shape[1], out, rows, hidden, intermediate, experts,
                          routed_scale, int(host_law), *ptrs)
    return (out, extra) if want_intermediates else out
