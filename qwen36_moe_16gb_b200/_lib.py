"""ctypes binding of ``libb200moe.so`` (the C ABI declared in ``include/b200moe.h``).

The library is built in-tree by :mod:`qwen36_moe_16gb_b200.build`.  There is no fallback: if the
shared object is missing or an entry point returns non-zero, the caller gets an exception.
"""
from __future__ import annotations

import ctypes as C
import pathlib
import threading

_HERE = pathlib.Path(__file__).resolve().parent
LIB_PATH = _HERE / "libb200moe.so"
_lock = threading.Lock()
_lib = None

c_void_p, c_int, c_i64 = C.c_void_p, C.c_int, C.c_int64


class SlotTables(C.Structure):
    _fields_ = [("slot_for_id", c_void_p), ("id_of_slot", c_void_p), ("usage", c_void_p), ("step", c_void_p),
                ("src_indices", c_void_p), ("evict_slots", c_void_p), ("num_indices", c_void_p), ("stats", c_void_p),
                ("num_layers", C.c_int32), ("num_experts", C.c_int32), ("cache_size", C.c_int32)]


class Banks(C.Structure):
    _fields_ = [("gate_up", c_void_p), ("gate_up_scale", c_void_p), ("gate_up_global", c_void_p), ("down", c_void_p),
                ("down_scale", c_void_p), ("down_global", c_void_p), ("num_slots", C.c_int32), ("hidden", C.c_int32),
                ("intermediate", C.c_int32), ("slot_stride", C.c_int64 * 6)]


class Dense(C.Structure):
    _fields_ = [("router_w", c_void_p), ("shared_gate_up", c_void_p), ("shared_down", c_void_p),
                ("shared_gate", c_void_p), ("num_experts", C.c_int32), ("shared_intermediate", C.c_int32)]


P = C.POINTER
# name -> (restype, argtypes); every symbol include/b200moe.h declares
SIGNATURES = {
    "b200moe_abi_version": (c_int, []),
    "b200moe_build_id": (C.c_char_p, []),
    "b200moe_error_string": (C.c_char_p, [c_int]),
    "b200moe_host_register": (c_int, [c_void_p, c_i64]),
    "b200moe_host_unregister": (c_int, [c_void_p]),
    "b200moe_host_device_ptr": (c_int, [c_void_p, P(c_void_p)]),
    "b200moe_router_topk": (c_int, [c_void_p, c_int, c_i64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                    c_void_p, c_void_p]),
    "b200moe_permute_workspace_bytes": (c_i64, [c_int, c_int]),
    "b200moe_permute": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_i64, c_void_p]),
    "b200moe_slot_reset": (c_int, [P(SlotTables), c_void_p]),
    "b200moe_slot_ensure": (c_int, [P(SlotTables), c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_slot_ensure_host": (c_int, [P(SlotTables), c_int, c_void_p, c_int, c_void_p]),
    "b200moe_prefill_split": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p]),
    "b200moe_pregate_predict": (c_int, [c_void_p, c_void_p, C.c_float, c_void_p, c_i64, c_int, c_int, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_slot_materialize": (c_int, [P(SlotTables), c_int, c_void_p]),
    "b200moe_slot_fill": (c_int, [c_int, P(c_void_p), P(c_void_p), P(c_i64), c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_slot_gather": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_void_p]),
    "b200moe_decode_workspace_bytes": (c_i64, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200moe_decode_experts": (c_int, [c_void_p, P(Banks), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_i64,
                                       c_void_p]),
    "b200moe_decode_experts_static": (c_int, [c_void_p, P(Banks), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_decode_block_route": (c_int, [c_void_p, P(Dense), c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_i64, c_void_p]),
    "b200moe_decode_dense_rows": (c_int, [c_void_p, P(Dense), c_int, c_int, c_int, c_void_p, c_void_p, c_i64, c_void_p]),
    "b200moe_decode_block_experts": (c_int, [c_void_p, P(Banks), P(Dense), c_void_p, c_void_p, c_int, c_int, c_void_p,
                                             c_void_p, c_i64, c_void_p]),
    "b200moe_decode_block": (c_int, [c_void_p, P(Banks), P(Dense), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_i64, c_void_p]),
    "b200moe_set_pdl": (c_int, [c_int]),
    "b200moe_offload_create": (c_void_p, [P(SlotTables), c_int, P(c_void_p), P(c_void_p), P(c_i64), c_int, P(c_int)]),
    "b200moe_offload_destroy": (None, [c_void_p]),
    "b200moe_offload_decode_step": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_i64, c_void_p,
                                            P(Banks), P(Dense), c_i64, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p,
                                            c_void_p, P(c_i64), c_void_p, c_void_p]),
    "b200moe_prefill_workspace_bytes": (c_i64, [c_int, c_int, c_int, c_int, c_int]),
    "b200moe_prefill_experts": (c_int, [c_void_p, P(Banks), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_i64, c_void_p, c_void_p]),
    "b200moe_prefill_stages": (c_int, [c_void_p, P(Banks), c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_i64, c_void_p, c_int, c_void_p]),
    "b200moe_fused_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, C.c_float, c_int, c_i64, c_int, c_void_p]),
    "b200moe_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, C.c_float, c_int, c_i64, c_int, c_void_p]),
    "b200moe_dense_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200moe_row_dot": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200moe_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200moe_shared_epilogue": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "b200moe_sum_routes": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200moe_combine_routes": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                       c_void_p]),
    "b200moe_prefill_ep_routes": (c_int, [c_void_p, P(Banks), c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                          c_int, c_void_p, c_i64, c_void_p, c_void_p]),
    "b200moe_prefill_ic3_offset": (c_i64, [c_int, c_int, c_int, c_int, c_int]),
}


class B200MoeError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (there is no other code path)."""
    global _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise B200MoeError(
                    f"{LIB_PATH} is missing: build it with `python -m qwen36_moe_16gb_b200.build` "
                    "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
            handle = C.CDLL(str(LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(handle, name)  # AttributeError if the .so is stale
                fn.restype, fn.argtypes = res, args
            if handle.b200moe_abi_version() != 1:
                raise B200MoeError("libb200moe.so ABI version mismatch")
            _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().b200moe_error_string(code).decode()
        raise B200MoeError(f"{what} failed with code {code}: {msg}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
