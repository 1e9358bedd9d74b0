"""ctypes binding of the C ABI in ``include/kvmig.h`` (no torch involved).

Used by the parity tests and the benchmark to call the library the way a
foreign-language host would; the torch operator shim is the other client.
"""
from __future__ import annotations

import ctypes as C
from array import array
from typing import Optional, Sequence

from . import kvmig_library_path

HANDLE_WORDS = 24
MAX_INFLIGHT = 8

OK, EINVAL, ENOTREG, ECUDA, EDEVICE, ELIMIT = 0, -1, -2, -3, -4, -5


class PoolShape(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("num_blocks", "num_layers", "num_heads", "block_size", "head_dim", "elem_size")]

    @classmethod
    def of(cls, num_blocks, num_layers, num_heads, block_size, head_dim, elem_size=2):
        return cls(num_blocks, num_layers, num_heads, block_size, head_dim, elem_size)

    @property
    def block_bytes(self) -> int:
        return self.num_layers * self.num_heads * self.block_size * self.head_dim * self.elem_size


class KvmigError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"{text} (kvmig status {code})")
        self.code = code


_I64P = C.POINTER(C.c_int64)
_SHAPEP = C.POINTER(PoolShape)

# name -> (restype, argtypes); one entry per declaration in include/kvmig.h
SIGNATURES = {
    "kvmig_abi_version": (C.c_int, []),
    "kvmig_last_error": (C.c_char_p, []),
    "kvmig_get_ipc_mem_handle": (C.c_int, [C.c_void_p, _SHAPEP, _I64P]),
    "kvmig_handle_is_local": (C.c_int, [_I64P, C.c_int64]),
    "kvmig_register_ipc_mem_handle": (C.c_int, [_I64P, C.c_int64, _I64P, C.c_int64, C.c_int64, C.c_int64, _I64P, _I64P]),
    "kvmig_migrate_blocks": (C.c_int, [C.c_int64, C.c_int64, _I64P, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                       _I64P, C.c_int64, C.c_void_p, C.c_void_p, _SHAPEP, C.c_void_p]),
    "kvmig_migrate_blocks_async": (C.c_int, [C.c_int64, C.c_int64, _I64P, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                             C.c_int64, _I64P, C.c_int64, C.c_void_p, C.c_void_p, _SHAPEP, C.c_void_p,
                                             C.POINTER(C.c_uint64)]),
    "kvmig_migrate_layers_async": (C.c_int, [C.c_int64, C.c_int64, _I64P, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                             C.c_int64, _I64P, C.c_int64, C.c_void_p, C.c_void_p, _SHAPEP, C.c_int64,
                                             C.c_int64, C.c_void_p, C.POINTER(C.c_uint64)]),
    "kvmig_migrate_wait": (C.c_int, [C.c_uint64]),
    "kvmig_migrate_blocks_static": (C.c_int, [C.c_int64, C.c_int64, _I64P, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                              C.c_int64, _I64P, C.c_int64, C.c_void_p, C.c_void_p, _SHAPEP, C.c_void_p]),
    "kvmig_swap": (C.c_int, [_I64P, C.c_int64, _I64P, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, _SHAPEP, C.c_void_p,
                             C.c_void_p, C.c_int64, C.c_void_p]),
    "kvmig_set_option": (C.c_int, [C.c_char_p, C.c_int64]),
    "kvmig_get_option": (C.c_int64, [C.c_char_p]),
    "kvmig_get_counter": (C.c_int64, [C.c_char_p]),
    "kvmig_reset_registry": (C.c_int, []),
}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        handle = C.CDLL(str(kvmig_library_path()))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise KvmigError(rc, lib().kvmig_last_error().decode())


def as_i64(values: Sequence[int]):
    """A ctypes int64 array holding `values`; block lists that are passed again and again can be converted
    once and handed to the calls below in this form."""
    packed = array("q", values) if len(values) else array("q", (0,))      # one pass in C; non-integers raise TypeError
    return (C.c_int64 * len(packed)).from_buffer(packed)                 # shares (and keeps alive) the packed buffer


class I64List:
    """A block-index list converted once for repeated use (keeps its logical length: an empty list still
    needs a non-empty ctypes array)."""

    __slots__ = ("array", "n")

    def __init__(self, values: Sequence[int]) -> None:
        self.array = as_i64(values)
        self.n = len(values)

    def __len__(self) -> int:
        return self.n


def _i64(values):
    return values.array if isinstance(values, I64List) else as_i64(values)


def get_ipc_mem_handle(pool_ptr: int, shape: PoolShape) -> list:
    out = (C.c_int64 * HANDLE_WORDS)()
    _check(lib().kvmig_get_ipc_mem_handle(pool_ptr, C.byref(shape), out))
    return list(out)


def handle_is_local(handle) -> bool:
    """Was this handle exported by the calling process (pid and per-process number both match)?"""
    rc = lib().kvmig_handle_is_local(_i64(handle), len(handle))
    if rc < 0:
        raise KvmigError(rc, lib().kvmig_last_error().decode())
    return bool(rc)


def register_ipc_mem_handle(k_handle, v_handle, num_layers, num_heads, ctx_pc, dec_pc) -> None:
    if len(ctx_pc) != 4 or len(dec_pc) != 4:
        raise ValueError("parallel configs must be [tp_size, tp_rank, pp_size, pp_rank]")
    _check(lib().kvmig_register_ipc_mem_handle(_i64(k_handle), len(k_handle), _i64(v_handle), len(v_handle),
                                               num_layers, num_heads, _i64(ctx_pc), _i64(dec_pc)))


def migrate_blocks(ctx_pp, ctx_tp, ctx_blocks, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks,
                   k_ptr: int, v_ptr: int, shape: PoolShape, stream: int = 0) -> None:
    _check(lib().kvmig_migrate_blocks(ctx_pp, ctx_tp, _i64(ctx_blocks), len(ctx_blocks), dec_pp, dec_tp, dec_pp_rank,
                                      dec_tp_rank, _i64(dec_blocks), len(dec_blocks), k_ptr, v_ptr, C.byref(shape), stream))


def migrate_blocks_async(ctx_pp, ctx_tp, ctx_blocks, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks,
                         k_ptr: int, v_ptr: int, shape: PoolShape, stream: int = 0) -> int:
    ticket = C.c_uint64(0)
    _check(lib().kvmig_migrate_blocks_async(ctx_pp, ctx_tp, _i64(ctx_blocks), len(ctx_blocks), dec_pp, dec_tp,
                                            dec_pp_rank, dec_tp_rank, _i64(dec_blocks), len(dec_blocks), k_ptr, v_ptr,
                                            C.byref(shape), stream, C.byref(ticket)))
    return ticket.value


def migrate_layers_async(ctx_pp, ctx_tp, ctx_blocks, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks,
                         k_ptr: int, v_ptr: int, shape: PoolShape, layer_begin: int, layer_end: int, stream: int = 0) -> int:
    """Enqueue the copy of the global layers [layer_begin, layer_end) only; returns a ticket."""
    ticket = C.c_uint64(0)
    _check(lib().kvmig_migrate_layers_async(ctx_pp, ctx_tp, _i64(ctx_blocks), len(ctx_blocks), dec_pp, dec_tp,
                                            dec_pp_rank, dec_tp_rank, _i64(dec_blocks), len(dec_blocks), k_ptr, v_ptr,
                                            C.byref(shape), layer_begin, layer_end, stream, C.byref(ticket)))
    return ticket.value


STATIC_MAX_BLOCKS = 4096


def migrate_blocks_static(ctx_pp, ctx_tp, ctx_blocks, dec_pp, dec_tp, dec_pp_rank, dec_tp_rank, dec_blocks,
                          k_ptr: int, v_ptr: int, shape: PoolShape, stream: int = 0) -> None:
    """kvmig_migrate_blocks_static: the same copy for hosts that may not allocate device memory
    once serving has started; at most STATIC_MAX_BLOCKS blocks per call."""
    _check(lib().kvmig_migrate_blocks_static(ctx_pp, ctx_tp, _i64(ctx_blocks), len(ctx_blocks), dec_pp, dec_tp,
                                             dec_pp_rank, dec_tp_rank, _i64(dec_blocks), len(dec_blocks), k_ptr, v_ptr,
                                             C.byref(shape), stream))


def migrate_wait(ticket: int) -> None:
    _check(lib().kvmig_migrate_wait(ticket))


def swap(source_ids, target_ids, is_swap_in: bool, k_ptr, v_ptr, shape: PoolShape, k_swap_ptr, v_swap_ptr,
         num_cpu_blocks: int, stream: int = 0) -> None:
    _check(lib().kvmig_swap(_i64(source_ids), len(source_ids), _i64(target_ids), len(target_ids), int(bool(is_swap_in)),
                            k_ptr, v_ptr, C.byref(shape), k_swap_ptr, v_swap_ptr, num_cpu_blocks, stream))


def set_option(name: str, value: int) -> None:
    _check(lib().kvmig_set_option(name.encode(), value))


def get_option(name: str) -> int:
    return lib().kvmig_get_option(name.encode())


def get_counter(name: str) -> int:
    return lib().kvmig_get_counter(name.encode())


def reset_registry() -> None:
    _check(lib().kvmig_reset_registry())
