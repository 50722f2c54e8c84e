"""Host-side mirror of the reference engine's MoE operator interface, over the C ABI.

The product is ``libp92moe_b200.so`` (hand-written sm_100a CUDA behind
``include/p92b_moe.h``).  This package is the thin host layer a Python harness
needs: it loads the library with ctypes, hands it raw device pointers of torch
tensors (torch is used for device memory, streams and torch.distributed only)
and exposes the same operator names and argument meaning as the reference's
``p92::cuda`` free functions (include/p92/kernels.h), ``ProjectionExecutor``
(include/p92/executor.h:31-45) and ``Model::Impl::run_moe_rows``
(src/model.cpp:1486-1573).

There is no CPU or eager fallback: importing works without a GPU (so the
symbol table can be checked), but every operator raises if the library is
missing or a call returns a CUDA error, like the reference's ``check()``
(src/executor.cpp:12-16).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

HIDDEN = 2560
INTERMEDIATE = 1024
EXPERTS = 256
TOP_K = 8
ROUTED_SCALE = 2.5

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libp92moe_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "p92b_moe.h")

_lib: Optional[ctypes.CDLL] = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_size_t = ctypes.c_size_t


class ExpertProjection(ctypes.Structure):
    """Binary layout of p92::cuda::Nvfp4ExpertProjection (include/p92/kernels.h:12-16)."""

    _fields_ = [("weight", c_void_p), ("scales_swizzled", c_void_p), ("alpha", c_void_p)]


class ArtifactRecord(ctypes.Structure):
    """Binary layout of p92::Nvfp4Record (include/p92/nvfp4_artifact.h:24-32)."""

    _pack_ = 1
    _fields_ = [("name", ctypes.c_char * 96), ("rows", ctypes.c_uint32), ("columns", ctypes.c_uint32),
                ("weight_offset", ctypes.c_uint64), ("scale_offset", ctypes.c_uint64), ("weight_scale_2", c_float),
                ("reserved", ctypes.c_uint32)]


class PlanViews(ctypes.Structure):
    _fields_ = [
        ("logits", c_void_p),
        ("expert_ids", c_void_p),
        ("expert_weights", c_void_p),
        ("order", c_void_p),
        ("position", c_void_p),
        ("counts", c_void_p),
        ("offsets", c_void_p),
        ("mixed", c_void_p),
        ("mixed_index", c_void_p),
        ("status", c_void_p),
        ("router_stats", c_void_p),
        ("trace", c_void_p),
        ("trace_blocks", c_int),
    ]


# name -> (restype, argtypes); must list every symbol include/p92b_moe.h declares.
SIGNATURES = {
    "p92b_bf16_gemv_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "p92b_bf16_gemm_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "p92b_router_top8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "p92b_router_top8_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_nvfp4_quantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_nvfp4_swizzled_scale_bytes": (c_size_t, [c_int, c_int]),
    "p92b_nvfp4_swizzle_scales": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "p92b_nvfp4_pack_weight": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "p92b_nvfp4_pack_weight_batch": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p, c_void_p]),
    "p92b_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_expert_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "p92b_expert_combine_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "p92b_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]),
    "p92b_rmsnorm_strided": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]),
    "p92b_add_inplace": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_moe_permute": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "p92b_moe_permute_static": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "p92b_moe_permute_static_status": (c_int, [ctypes.POINTER(c_int), c_void_p]),
    "p92b_ep_row_bytes": (c_size_t, [c_int]),
    "p92b_ep_route": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "p92b_ep_experts": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "p92b_ep_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_ep_fixed_block_bytes": (c_size_t, [c_int, c_int, c_int]),
    "p92b_ep_route_fixed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_void_p]),
    "p92b_ep_experts_fixed": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "p92b_ep_combine_fixed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_ep_window_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int]),
    "p92b_ep_window_destroy": (None, [c_void_p]),
    "p92b_ep_window_bytes": (c_size_t, [c_void_p]),
    "p92b_ep_window_handle": (c_int, [c_void_p, c_void_p]),
    "p92b_ep_window_connect": (c_int, [c_void_p, c_void_p]),
    "p92b_ep_window_connect_local": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "p92b_ep_window_create_bulk": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int]),
    "p92b_ep_forward_bulk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_ep_forward_gathered": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_ep_forward_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_ep_forward_fused_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_bank_create": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(ExpertProjection), c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "p92b_bank_destroy": (None, [c_void_p]),
    "p92b_bank_bytes": (c_size_t, [c_void_p]),
    "p92b_artifact_open": (c_int, [ctypes.POINTER(c_void_p), ctypes.c_char_p]),
    "p92b_artifact_close": (None, [c_void_p]),
    "p92b_artifact_tensor_count": (c_int, [c_void_p]),
    "p92b_artifact_has_swizzled_scales": (c_int, [c_void_p]),
    "p92b_artifact_at": (c_int, [c_void_p, c_int, ctypes.POINTER(ArtifactRecord)]),
    "p92b_artifact_find": (c_int, [c_void_p, ctypes.c_char_p, ctypes.POINTER(ArtifactRecord)]),
    "p92b_artifact_weight": (c_void_p, [c_void_p, ctypes.POINTER(ArtifactRecord)]),
    "p92b_artifact_scales": (c_void_p, [c_void_p, ctypes.POINTER(ArtifactRecord)]),
    "p92b_artifact_last_error": (ctypes.c_char_p, []),
    "p92b_bank_create_from_artifact": (c_int, [ctypes.POINTER(c_void_p), c_void_p, c_int, c_int, c_int, c_void_p]),
    "p92b_dense_bank_create_from_artifact": (c_int, [ctypes.POINTER(c_void_p), c_void_p, c_int, c_void_p]),
    "p92b_plan_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int]),
    "p92b_plan_destroy": (None, [c_void_p]),
    "p92b_plan_bytes": (c_size_t, [c_void_p]),
    "p92b_moe_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_moe_forward_normed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_dense_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_moe_forward_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_plan_host_flush": (c_int, [c_void_p, c_void_p]),
    "p92b_moe_forward_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "p92b_project_expert_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_project_expert_down": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "p92b_nvfp4_grouped_plan_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int]),
    "p92b_nvfp4_grouped_plan_destroy": (None, [c_void_p]),
    "p92b_nvfp4_grouped_plan_status": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "p92b_nvfp4_grouped_m1": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "p92b_nvfp4_grouped_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "p92b_plan_get_views": (c_int, [c_void_p, ctypes.POINTER(PlanViews)]),
    "p92b_plan_set_path": (c_int, [c_void_p, c_int]),
    "p92b_plan_last_launches": (c_int, [c_void_p]),
    "p92b_plan_stage_timing": (c_int, [c_void_p, c_int]),
    "p92b_plan_stage_times": (c_int, [c_void_p, ctypes.POINTER(c_float), ctypes.POINTER(c_int)]),
    "p92b_version": (ctypes.c_char_p, []),
}

_CUDA_ERROR_NAMES = {1: "cudaErrorInvalidValue", 2: "cudaErrorMemoryAllocation", 301: "cudaErrorFileNotFound",
                     801: "cudaErrorNotSupported"}


class P92Error(RuntimeError):
    """A C-ABI call returned a CUDA error (the reference throws std::runtime_error here)."""

    def __init__(self, operation: str, code: int):
        self.code = code
        super().__init__(f"{operation}: {_CUDA_ERROR_NAMES.get(code, 'cudaError')} ({code})")


def load_library() -> ctypes.CDLL:
    """Loads libp92moe_b200.so; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise FileNotFoundError(
            f"{LIBRARY_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()); this package has no CPU path")
    lib = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def _check(code: int, operation: str) -> None:
    if code != 0:
        raise P92Error(operation, code)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def _require(t, dtype, name: str):
    import torch

    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name}: expected a contiguous CUDA tensor of {dtype}")
    return t


# --------------------------------------------------------------------------
# Operator functions: same names and argument meaning as p92::cuda::*.
# BF16 tensors are torch.bfloat16 (or int16/uint16 views of the same bits).
# --------------------------------------------------------------------------

def bf16_gemv_f32(input, weight, output) -> None:
    rows, columns = weight.shape
    _check(load_library().p92b_bf16_gemv_f32(_ptr(input), _ptr(weight), _ptr(output), rows, columns, _stream()),
           "bf16_gemv_f32")


def bf16_gemm_f32(input, weight, output, batch_rows: int) -> None:
    rows, columns = weight.shape
    _check(load_library().p92b_bf16_gemm_f32(_ptr(input), _ptr(weight), _ptr(output), batch_rows, rows, columns,
                                             _stream()), "bf16_gemm_f32")


def router_top8_rows(logits, correction_bias, expert_ids, expert_weights, rows: int,
                     routed_scale: float = ROUTED_SCALE) -> None:
    _check(load_library().p92b_router_top8_rows(_ptr(logits), _ptr(correction_bias), _ptr(expert_ids),
                                                _ptr(expert_weights), rows, routed_scale, _stream()),
           "router_top8_rows")


def nvfp4_quantize(input, output, scales, elements: int, global_scale: float = 1.0) -> None:
    _check(load_library().p92b_nvfp4_quantize(_ptr(input), _ptr(output), _ptr(scales), elements, global_scale,
                                              _stream()), "nvfp4_quantize")


def nvfp4_swizzled_scale_bytes(rows: int, scale_columns: int) -> int:
    return int(load_library().p92b_nvfp4_swizzled_scale_bytes(rows, scale_columns))


def nvfp4_swizzle_scales(linear, swizzled, rows: int, scale_columns: int) -> None:
    _check(load_library().p92b_nvfp4_swizzle_scales(_ptr(linear), _ptr(swizzled), rows, scale_columns, _stream()),
           "nvfp4_swizzle_scales")


def nvfp4_pack_weight(input, packed, scales, weight_scale_2) -> None:
    _check(load_library().p92b_nvfp4_pack_weight(_ptr(input), _ptr(packed), _ptr(scales), input.numel(),
                                                 _ptr(weight_scale_2), _stream()), "nvfp4_pack_weight")


def nvfp4_pack_weight_batch(input, packed, scales, weight_scale_2) -> None:
    """input BF16 [matrices, elements]: every matrix quantised with its own per-tensor scale."""
    matrices = input.shape[0]
    _check(load_library().p92b_nvfp4_pack_weight_batch(_ptr(input), _ptr(packed), _ptr(scales),
                                                       input.numel() // matrices, matrices, _ptr(weight_scale_2),
                                                       _stream()), "nvfp4_pack_weight_batch")


def swiglu(gate, up, output, elements: int) -> None:
    _check(load_library().p92b_swiglu(_ptr(gate), _ptr(up), _ptr(output), elements, _stream()), "swiglu")


def expert_combine_rows(expert_rows, route_weights, output, batch_rows: int, experts: int, elements: int) -> None:
    _check(load_library().p92b_expert_combine_rows(_ptr(expert_rows), _ptr(route_weights), _ptr(output), batch_rows,
                                                   experts, elements, _stream()), "expert_combine_rows")


def rmsnorm(input, weight, output, rows: int, elements: int, epsilon: float = 1.0e-5) -> None:
    _check(load_library().p92b_rmsnorm(_ptr(input), _ptr(weight), _ptr(output), rows, elements, epsilon, _stream()),
           "rmsnorm")


def add_inplace(destination, source, elements: int) -> None:
    _check(load_library().p92b_add_inplace(_ptr(destination), _ptr(source), elements, _stream()), "add_inplace")


STATIC_PERMUTE_MAX_ASSIGNMENTS = 65536


def moe_permute_static(expert_ids, order, position, counts, offsets) -> None:
    """Permutation without a plan, for hosts that cannot allocate device memory (engines whose arena
    already owns the whole card, processes that forbid further CUDA allocations, loops that must not
    hit an allocation's device-wide synchronisation).  Scratch is a fixed array inside the library,
    shared by all calls on a device: at most 65536 assignments, calls must not overlap on the GPU,
    and the first call on a device (which looks up the array's address) belongs before any stream
    capture."""
    _check(load_library().p92b_moe_permute_static(_ptr(expert_ids), expert_ids.numel(), _ptr(order), _ptr(position),
                                                  _ptr(counts), _ptr(offsets), _stream()), "moe_permute_static")


def moe_permute_static_status() -> int:
    """Status word of the last moe_permute_static call on the current stream: 0, or 1 if an expert id
    outside 0..255 was met (and counted as expert 0 or 255).  Synchronises the stream; allocates nothing."""
    word = c_int(-1)
    _check(load_library().p92b_moe_permute_static_status(ctypes.byref(word), _stream()), "moe_permute_static_status")
    return int(word.value)


class ExpertBank:
    """One layer's expert weights in the library's layout (replaces the expert table of src/model.cpp:772-805).

    ``entries``: sequence of (weight, scales_swizzled, alpha) CUDA tensors in the
    reference's bank order ``expert * 3 + kind`` (kind 0/1/2 = gate/up/down), the
    shared expert's three entries last.  The tensors may be freed afterwards.
    """

    def __init__(self, entries: Sequence[tuple], first_expert: int = 0, local_experts: int = EXPERTS,
                 hidden: int = HIDDEN, intermediate: int = INTERMEDIATE):
        if len(entries) != (local_experts + 1) * 3:
            raise ValueError("invalid expert bank: need (local_experts + 1) * 3 entries")
        array = (ExpertProjection * len(entries))()
        for i, (w, s, a) in enumerate(entries):
            array[i].weight, array[i].scales_swizzled, array[i].alpha = w.data_ptr(), s.data_ptr(), a.data_ptr()
        handle = c_void_p()
        _check(load_library().p92b_bank_create(ctypes.byref(handle), array, first_expert, local_experts, hidden,
                                               intermediate, 0, _stream()), "bank_create")
        self.handle = handle
        self.first_expert, self.local_experts = first_expert, local_experts
        self.hidden, self.intermediate = hidden, intermediate

    @classmethod
    def _adopt(cls, handle, first_expert: int, local_experts: int) -> "ExpertBank":
        bank = cls.__new__(cls)
        bank.handle = handle
        bank.first_expert, bank.local_experts = first_expert, local_experts
        bank.hidden = bank.intermediate = None          # the library knows; a plan of the wrong shape is rejected by it
        return bank

    @property
    def nbytes(self) -> int:
        return int(load_library().p92b_bank_bytes(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            load_library().p92b_bank_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Nvfp4Artifact:
    """The engine's NVFP4 weight container, opened read-only (mirrors p92::Nvfp4Artifact,
    include/p92/nvfp4_artifact.h:36-71).  Needs no GPU."""

    def __init__(self, directory: str):
        handle = c_void_p()
        code = load_library().p92b_artifact_open(ctypes.byref(handle), os.fsencode(directory))
        if code != 0:
            raise P92Error("artifact_open: " + load_library().p92b_artifact_last_error().decode(), code)
        self.handle = handle

    @property
    def tensor_count(self) -> int:
        return int(load_library().p92b_artifact_tensor_count(self.handle))

    @property
    def has_swizzled_scales(self) -> bool:
        return bool(load_library().p92b_artifact_has_swizzled_scales(self.handle))

    def at(self, index: int) -> ArtifactRecord:
        record = ArtifactRecord()
        code = load_library().p92b_artifact_at(self.handle, index, ctypes.byref(record))
        if code != 0:
            raise P92Error("artifact_at: " + load_library().p92b_artifact_last_error().decode(), code)
        return record

    def find(self, name: str) -> ArtifactRecord:
        record = ArtifactRecord()
        code = load_library().p92b_artifact_find(self.handle, name.encode(), ctypes.byref(record))
        if code != 0:
            raise P92Error("artifact_find: " + load_library().p92b_artifact_last_error().decode(), code)
        return record

    def weight_bytes(self, record: ArtifactRecord) -> bytes:
        ptr = load_library().p92b_artifact_weight(self.handle, ctypes.byref(record))
        return ctypes.string_at(ptr, record.rows * record.columns // 2)

    def scale_bytes(self, record: ArtifactRecord) -> bytes:
        ptr = load_library().p92b_artifact_scales(self.handle, ctypes.byref(record))
        return ctypes.string_at(ptr, record.rows * record.columns // 16)

    def load_bank(self, layer_index: int, first_expert: int = 0, local_experts: int = EXPERTS) -> "ExpertBank":
        """One layer's experts + shared expert uploaded into a bank (ResidentWeights::open + the table build)."""
        handle = c_void_p()
        code = load_library().p92b_bank_create_from_artifact(ctypes.byref(handle), self.handle, layer_index, first_expert,
                                                             local_experts, _stream())
        if code != 0:
            raise P92Error("bank_create_from_artifact: " + load_library().p92b_artifact_last_error().decode(), code)
        return ExpertBank._adopt(handle, first_expert, local_experts)

    def load_dense_bank(self, layer_index: int) -> "ExpertBank":
        handle = c_void_p()
        code = load_library().p92b_dense_bank_create_from_artifact(ctypes.byref(handle), self.handle, layer_index, _stream())
        if code != 0:
            raise P92Error("dense_bank_create_from_artifact: " + load_library().p92b_artifact_last_error().decode(), code)
        return ExpertBank._adopt(handle, 0, 0)

    def close(self) -> None:
        if getattr(self, "handle", None):
            load_library().p92b_artifact_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoePlan:
    """Scratch for up to ``max_rows`` tokens (replaces Nvfp4GroupedPlan + the executor's scratch)."""

    def __init__(self, max_rows: int, hidden: int = HIDDEN, intermediate: int = INTERMEDIATE):
        handle = c_void_p()
        _check(load_library().p92b_plan_create(ctypes.byref(handle), max_rows, hidden, intermediate), "plan_create")
        self.handle = handle
        self.max_rows, self.hidden, self.intermediate = max_rows, hidden, intermediate

    @property
    def nbytes(self) -> int:
        return int(load_library().p92b_plan_bytes(self.handle))

    def host_flush(self) -> None:
        """Make the current stream wait for the copy-outs of run_moe_rows_host_async calls still in flight."""
        _check(load_library().p92b_plan_host_flush(self.handle, _stream()), "plan_host_flush")

    @property
    def last_launches(self) -> int:
        return int(load_library().p92b_plan_last_launches(self.handle))

    STAGES = ("router_logits", "router_top8", "permute", "quantize", "gate_up_swiglu", "down", "combine_shared")

    def stage_timing(self, enable: bool) -> None:
        _check(load_library().p92b_plan_stage_timing(self.handle, int(enable)), "plan_stage_timing")

    def stage_times(self) -> tuple:
        """(dict stage -> summed ms since enabling, number of forwards accumulated)."""
        ms = (c_float * len(self.STAGES))()
        calls = c_int()
        _check(load_library().p92b_plan_stage_times(self.handle, ms, ctypes.byref(calls)), "plan_stage_times")
        return dict(zip(self.STAGES, [float(v) for v in ms])), int(calls.value)

    def views(self, rows: int) -> dict:
        """Copies of the last forward's intermediates as torch tensors (tests / tracing)."""
        import torch

        v = PlanViews()
        _check(load_library().p92b_plan_get_views(self.handle, ctypes.byref(v)), "plan_get_views")
        grab = _device_copy

        a = rows * TOP_K
        mixed_index = grab(v.mixed_index, (a + rows,), torch.int32)
        mixed = None
        if int(mixed_index.min()) >= 0:            # (the expert-parallel paths keep other things in this index)
            span = int(mixed_index.max()) + 1
            typestr_rows = torch.as_tensor(_DeviceSpan(v.mixed, (span, self.hidden), "<i2"), device="cuda")
            mixed = typestr_rows[mixed_index.long()].contiguous().view(torch.bfloat16)
        return {
            "mixed": mixed,            # [rows*8 + rows, hidden] in (row, slot) order, shared rows last
            "logits": grab(v.logits, (rows, EXPERTS), torch.float32),
            "expert_ids": grab(v.expert_ids, (rows, TOP_K), torch.int32),
            "expert_weights": grab(v.expert_weights, (rows, TOP_K), torch.float32),
            "order": grab(v.order, (a,), torch.int32),
            "position": grab(v.position, (a,), torch.int32),
            "counts": grab(v.counts, (EXPERTS,), torch.int32),
            "offsets": grab(v.offsets, (EXPERTS + 1,), torch.int32),
            "mixed_index": mixed_index,
            "status": grab(v.status, (1,), torch.int32),
            "router_stats": grab(v.router_stats, (2,), torch.int32),
            "trace": torch.as_tensor(_DeviceSpan(v.trace, (v.trace_blocks, 64), "<i8"), device="cuda").clone(),
        }

    def status(self) -> int:
        """The plan's status word: 0, or the first error a kernel recorded (synchronises the device)."""
        import torch

        v = PlanViews()
        _check(load_library().p92b_plan_get_views(self.handle, ctypes.byref(v)), "plan_get_views")
        return int(_device_copy(v.status, (1,), torch.int32)[0])

    def device_counts(self):
        """Zero-copy int32 [256] view of the last call's per-expert row counts (valid until the next call)."""
        import torch

        v = PlanViews()
        _check(load_library().p92b_plan_get_views(self.handle, ctypes.byref(v)), "plan_get_views")
        return torch.as_tensor(_DeviceSpan(v.counts, (EXPERTS,), "<i4"), device="cuda")

    PATH_AUTO, PATH_TENSOR_CORE, PATH_FUSED_DECODE = 0, 2, 3

    def set_path(self, path: int) -> None:
        _check(load_library().p92b_plan_set_path(self.handle, path), "plan_set_path")

    def permute(self, expert_ids, order, position, counts, offsets) -> None:
        _check(load_library().p92b_moe_permute(self.handle, _ptr(expert_ids), expert_ids.numel(), _ptr(order),
                                               _ptr(position), _ptr(counts), _ptr(offsets), _stream()),
               "moe_permute")

    def close(self) -> None:
        if getattr(self, "handle", None):
            load_library().p92b_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GroupedPlan:
    """Stand-in for p92::cuda::Nvfp4GroupedPlan (include/p92/kernels.h:25-53): `groups` problems of a
    [rows x columns] matrix; grouped_rows reads the caller's device table of Nvfp4ExpertProjection in place."""

    def __init__(self, groups: int, rows: int, columns: int):
        handle = c_void_p()
        _check(load_library().p92b_nvfp4_grouped_plan_create(ctypes.byref(handle), groups, rows, columns),
               "nvfp4_grouped_plan_create")
        self.handle, self.groups, self.rows, self.columns = handle, groups, rows, columns

    def grouped_rows(self, packed_input, input_scales_swizzled, expert_bank, expert_ids, first_output, second_output,
                     projection_kind: int, batch_rows: int, expert_distinct_input_rows: bool) -> None:
        _check(load_library().p92b_nvfp4_grouped_rows(self.handle, _ptr(packed_input), _ptr(input_scales_swizzled),
                                                      _ptr(expert_bank), _ptr(expert_ids), _ptr(first_output),
                                                      _ptr(second_output), projection_kind, batch_rows,
                                                      int(expert_distinct_input_rows), _stream()), "nvfp4_grouped_rows")

    def status(self) -> int:
        import torch

        word = c_void_p()
        _check(load_library().p92b_nvfp4_grouped_plan_status(self.handle, ctypes.byref(word)), "nvfp4_grouped_plan_status")
        return int(_device_copy(word.value, (1,), torch.int32)[0])

    def close(self) -> None:
        if getattr(self, "handle", None):
            load_library().p92b_nvfp4_grouped_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _DeviceSpan:
    """Zero-copy view of library-owned device memory through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape: tuple, typestr: str):
        self.__cuda_array_interface__ = {"data": (int(ptr), False), "shape": tuple(shape), "typestr": typestr,
                                         "version": 2}


def _device_copy(ptr: int, shape: tuple, dtype):
    import torch

    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.bfloat16: "<i2", torch.uint8: "|u1"}[dtype]
    view = torch.as_tensor(_DeviceSpan(ptr, shape, typestr), device="cuda")
    out = view.clone()
    return out.view(torch.bfloat16) if dtype == torch.bfloat16 else out


def run_dense_rows(plan: "MoePlan", bank: "ExpertBank", normalized, hidden_out, rows: int) -> None:
    """Model::Impl::run_dense_rows (src/model.cpp:1476-1484): the dense SwiGLU MLP; `bank` was created with
    local_experts=0 from the MLP's (gate, up, down) entries, `plan` with its intermediate size."""
    _check(load_library().p92b_dense_forward(plan.handle, bank.handle, _ptr(normalized), _ptr(hidden_out), rows, _stream()),
           "dense_forward")


class MoeBlock:
    """The MoE block of one layer: mirrors Model::Impl::run_moe / run_moe_rows."""

    def __init__(self, bank: ExpertBank, router_weight, correction_bias, plan: MoePlan,
                 routed_scale: float = ROUTED_SCALE):
        self.bank, self.plan = bank, plan
        self.router_weight, self.correction_bias = router_weight, correction_bias
        self.routed_scale = routed_scale

    def run_moe_rows(self, normalized, hidden_out, rows: int) -> None:
        """normalized BF16 [rows, hidden] -> hidden_out BF16 [rows, hidden] (src/model.cpp:1486-1573)."""
        _check(load_library().p92b_moe_forward(self.plan.handle, self.bank.handle, _ptr(normalized),
                                               _ptr(self.router_weight), _ptr(self.correction_bias),
                                               _ptr(hidden_out), rows, self.routed_scale, _stream()),
               "moe_forward")

    def run_moe_rows_normed(self, mixed, pre_norm_weight, post_norm_weight, normalized_out, rows: int,
                            epsilon: float = 1.0e-5) -> None:
        """rmsnorm(pre_mlp_norm) -> run_moe_rows -> rmsnorm(post_mlp_norm) as one call (src/model.cpp:211-218,
        1210-1217); either weight may be None."""
        _check(load_library().p92b_moe_forward_normed(self.plan.handle, self.bank.handle, _ptr(mixed),
                                                      _ptr(pre_norm_weight), _ptr(post_norm_weight), epsilon,
                                                      _ptr(self.router_weight), _ptr(self.correction_bias),
                                                      _ptr(normalized_out), rows, self.routed_scale, _stream()),
               "moe_forward_normed")

    def run_moe(self, normalized, hidden_out) -> None:
        """Single-token form (src/model.cpp:1677-1729)."""
        self.run_moe_rows(normalized, hidden_out, 1)

    def run_moe_rows_host(self, host_in, host_out, rows: int) -> None:
        """Same call with HOST (pinned) tensors: H2D, block, D2H, stream synchronised on return."""
        _check(load_library().p92b_moe_forward_host(self.plan.handle, self.bank.handle, host_in.data_ptr(),
                                                    _ptr(self.router_weight), _ptr(self.correction_bias),
                                                    host_out.data_ptr(), rows, self.routed_scale, _stream()),
               "moe_forward_host")

    def run_moe_rows_host_async(self, pinned_in, pinned_out, rows: int) -> None:
        """The same as a pipeline (copies on the plan's own streams): outputs are valid after
        ``plan.host_flush()`` and a synchronisation of the current stream."""
        _check(load_library().p92b_moe_forward_host_async(self.plan.handle, self.bank.handle, pinned_in.data_ptr(),
                                                          _ptr(self.router_weight), _ptr(self.correction_bias),
                                                          pinned_out.data_ptr(), rows, self.routed_scale, _stream()),
               "moe_forward_host_async")

    def project_expert_gate_up(self, expert_ids, input, gate_output, up_output, batch_rows: int = 1) -> None:
        """ProjectionExecutor::project_expert_gate_up (src/executor.cpp:39-71)."""
        _check(load_library().p92b_project_expert_gate_up(self.plan.handle, self.bank.handle, _ptr(expert_ids),
                                                          _ptr(input), _ptr(gate_output), _ptr(up_output),
                                                          batch_rows, _stream()), "project_expert_gate_up")

    def project_expert_down(self, expert_ids, input_rows, output_rows, batch_rows: int = 1) -> None:
        """ProjectionExecutor::project_expert_down (src/executor.cpp:73-107)."""
        _check(load_library().p92b_project_expert_down(self.plan.handle, self.bank.handle, _ptr(expert_ids),
                                                       _ptr(input_rows), _ptr(output_rows), batch_rows, _stream()),
               "project_expert_down")
