"""ctypes binding of libqvx_cuda.so: one prototype per declaration in include/qvx.h.

There is no fallback: if the library is missing it is built with nvcc, and if that fails the
import fails.  Nothing here computes anything.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

from . import build as _build

c_u32p = C.POINTER(C.c_uint32)
c_u64p = C.POINTER(C.c_uint64)
c_f32p = C.POINTER(C.c_float)
c_szp = C.POINTER(C.c_size_t)


class Geometry(C.Structure):
    _fields_ = [("block_tokens", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("dtype", C.c_uint32), ("layout", C.c_uint32)]


class Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("capacity", C.c_uint64), ("kv_pool", C.c_uint64), ("timing", C.c_uint32)]


class Prelude(C.Structure):
    """qvx_prelude: DeviceMoeAttention's clip / qk_norm / eps / rope (crates/qubivex-compute/src/discrete.rs:281-289)."""
    _fields_ = [("has_clip", C.c_uint32), ("clip", C.c_float), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p),
                ("eps", C.c_double), ("rope", C.c_void_p)]


class Usage(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("capacity", "used", "peak", "refused")]


class TransferStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "uploads", "upload_bytes", "activations_in", "activations_out", "submissions", "transfer_ns",
        "fence_waits", "submit_ns", "wait_ns", "timed", "gpu_ns", "gpu_busy_ns")]


K_COUNT = 6
KERNEL_NAMES = ("sync", "append", "attn", "prelude", "exact", "copy")


class KernelTimes(C.Structure):
    _fields_ = [("launches", C.c_uint64 * K_COUNT), ("gpu_ns", C.c_uint64 * K_COUNT)]


class KvPoolStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "bytes", "allocated", "blocks", "free", "layers", "synced_rows", "full",
        "cow_copies", "compaction_moves", "bytes_moved", "shared_blocks")]


class PrefixStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("lookups", "hits", "tokens_reused", "inserted", "evicted", "entries", "cost")]


RELEASE_FN = C.CFUNCTYPE(None, C.c_uint64, C.c_void_p)

P = C.c_void_p
_GEO = C.POINTER(Geometry)

# name -> (restype, argtypes); must list every function include/qvx.h declares.
PROTOTYPES = {
    "qvx_block_bytes": (C.c_size_t, [_GEO]),
    "qvx_elem_offset": (C.c_size_t, [_GEO, C.c_size_t, C.c_int, C.c_size_t, C.c_size_t]),
    "qvx_open": (C.c_int32, [C.POINTER(Config), C.POINTER(P)]),
    "qvx_close": (None, [P]),
    "qvx_name": (C.c_char_p, []),
    "qvx_describe": (C.c_int32, [P, C.c_char_p, C.c_size_t]),
    "qvx_supports": (C.c_int32, [P, C.c_uint32]),
    "qvx_last_error": (C.c_char_p, [P]),
    "qvx_kv_pool": (C.c_uint64, [P]),
    "qvx_max_arena": (C.c_uint64, [P]),
    "qvx_routes_moe_attention": (C.c_int32, [P, C.c_size_t, C.c_size_t, C.c_size_t]),
    "qvx_upload": (C.c_int32, [P, P, C.c_size_t, C.POINTER(P)]),
    "qvx_alloc": (C.c_int32, [P, C.c_size_t, C.POINTER(P)]),
    "qvx_write": (C.c_int32, [P, P, C.c_size_t, P, C.c_size_t]),
    "qvx_read": (C.c_int32, [P, P, C.c_size_t, P, C.c_size_t]),
    "qvx_retain": (None, [P]),
    "qvx_free": (None, [P]),
    "qvx_buffer_ptr": (P, [P]),
    "qvx_buffer_len": (C.c_size_t, [P]),
    "qvx_get_usage": (C.c_int32, [P, C.POINTER(Usage)]),
    "qvx_get_transfers": (C.c_int32, [P, C.POINTER(TransferStats)]),
    "qvx_get_kernel_times": (C.c_int32, [P, C.POINTER(KernelTimes)]),
    "qvx_reset_kernel_times": (C.c_int32, [P]),
    "qvx_kv_sync": (C.c_int32, [P, _GEO, P, C.c_size_t, P, P, C.c_size_t, P]),
    "qvx_kv_append": (C.c_int32, [P, _GEO, P, C.c_size_t, P, P, P, P, P, C.c_size_t, P]),
    "qvx_tables_create": (C.c_int32, [P, _GEO, C.c_size_t, C.c_size_t, C.c_size_t, P, P, C.c_size_t, P, C.POINTER(P)]),
    "qvx_tables_free": (None, [P]),
    "qvx_tables_pos": (P, [P]),
    "qvx_tables_blocks": (P, [P]),
    "qvx_tables_table_at": (P, [P]),
    "qvx_attn_decode": (C.c_int32, [P, P, P, P, P, C.c_uint32, P]),
    "qvx_kv_append_attn_decode": (C.c_int32, [P, P, P, P, P, P, P, C.c_uint32, P]),
    "qvx_attn_decode_static": (C.c_int32, [P, _GEO, P, C.c_size_t, C.c_size_t, P, P, P, P, C.c_uint32, P, P]),
    "qvx_block_copy": (C.c_int32, [P, _GEO, P, C.c_size_t, P, P, C.c_size_t, P]),
    "qvx_comm_unique_id": (C.c_int32, [P]),
    "qvx_comm_init": (C.c_int32, [P, C.c_int32, C.c_int32, P, C.c_size_t, C.c_size_t, C.c_size_t, C.POINTER(P)]),
    "qvx_comm_destroy": (None, [P]),
    "qvx_comm_peer_handle": (C.c_int32, [P, P]),
    "qvx_comm_peer_open": (C.c_int32, [P, P]),
    "qvx_comm_send_slot": (P, [P, C.c_size_t, C.c_size_t, C.c_size_t]),
    "qvx_allgather_heads": (C.c_int32, [P, P, P, C.c_size_t, C.c_size_t, C.c_size_t, P]),
    "qvx_paged_attention_host": (C.c_int32, [P, P, _GEO, C.c_size_t, C.c_size_t, P, P, P, P, P, C.c_size_t, P, P, P,
                                             C.c_size_t, P, C.c_uint32]),
    "qvx_paged_attention_host_async": (C.c_int32, [P, P, _GEO, C.c_size_t, C.c_size_t, P, P, P, P, P, C.c_size_t, P,
                                                   P, P, C.c_size_t, P, C.c_uint32]),
    "qvx_wait": (C.c_int32, [P]),
    "qvx_attn_prelude": (C.c_int32, [P, _GEO, C.c_size_t, C.c_size_t, P, P, P, C.POINTER(Prelude), P]),
    "qvx_attention_stage_host": (C.c_int32, [P, P, _GEO, C.c_size_t, C.c_size_t, P, P, P, C.POINTER(Prelude), P, P, C.c_size_t,
                                             P, P, P, C.c_size_t, P, C.c_uint32]),
    "qvx_block_copy_host": (C.c_int32, [P, P, _GEO, P, P, C.c_size_t]),
    "qvx_kvpool_blocks_for": (C.c_uint64, [_GEO, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]),
    "qvx_kvpool_new": (P, [_GEO, C.c_uint32]),
    "qvx_kvpool_delete": (None, [P]),
    "qvx_kvpool_set_free_order": (C.c_int32, [P, P, C.c_size_t]),
    "qvx_kvpool_stats_get": (C.c_int32, [P, C.POINTER(KvPoolStats)]),
    "qvx_kvpool_refcount": (C.c_uint32, [P, C.c_uint32]),
    "qvx_kvpool_note_allocated": (None, [P, C.c_int]),
    "qvx_seq_new": (P, [P, C.c_uint64]),
    "qvx_seq_delete": (None, [P]),
    "qvx_seq_blocks": (C.c_size_t, [P, C.c_size_t, P, C.c_size_t]),
    "qvx_seq_synced": (C.c_size_t, [P, C.c_size_t]),
    "qvx_seq_fork": (P, [P, C.c_size_t, C.c_uint64]),
    "qvx_plan_build": (C.c_int32, [P, C.POINTER(P), P, P, C.c_size_t, C.c_size_t, C.POINTER(P)]),
    "qvx_plan_free": (None, [P]),
    "qvx_plan_counts": (C.c_size_t, [P, c_szp, c_szp, c_szp]),
    "qvx_plan_pos": (c_u32p, [P]),
    "qvx_plan_table_at": (c_u32p, [P]),
    "qvx_plan_blocks": (c_u32p, [P]),
    "qvx_plan_sync_to": (c_u32p, [P]),
    "qvx_plan_sync_seq": (c_u32p, [P]),
    "qvx_plan_sync_pos": (c_u32p, [P]),
    "qvx_plan_copy_src": (c_u32p, [P]),
    "qvx_plan_copy_dst": (c_u32p, [P]),
    "qvx_plan_commit": (None, [P, P, C.POINTER(P), C.c_size_t]),
    "qvx_kvpool_compact": (C.c_int32, [P, P, P, C.c_size_t, c_szp]),
    "qvx_prefix_new": (P, [C.c_uint64, RELEASE_FN, P]),
    "qvx_prefix_delete": (None, [P]),
    "qvx_prefix_lookup": (C.c_int32, [P, C.c_char_p, P, C.c_size_t, c_u64p, c_szp, c_u64p]),
    "qvx_prefix_hit_release": (None, [P, C.c_uint64]),
    "qvx_prefix_insert": (C.c_int32, [P, C.c_char_p, P, C.c_size_t, C.c_uint64, C.c_uint64]),
    "qvx_prefix_evict_oldest": (C.c_int32, [P]),
    "qvx_prefix_clear": (None, [P]),
    "qvx_prefix_stats_get": (None, [P, C.POINTER(PrefixStats)]),
    "qvx_prefix_budget": (C.c_uint64, [P]),
}

HEADER = Path(__file__).resolve().parent.parent / "include" / "qvx.h"


def declared_symbols() -> list[str]:
    """Every function name include/qvx.h declares."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(qvx_[a-z0-9_]+)\s*\(", text)) - {"qvx_release_fn"})


_libs: dict = {}


def load(experiments: bool | str = False) -> C.CDLL:
    """The library (or its experiment build; "short_waits": the test build with short bounded waits), built
    first if absent.  Raises when it cannot be loaded."""
    if experiments not in _libs:
        short = experiments == "short_waits"
        path = _build.LIB_SHORT_WAITS if short else _build.LIB_EXPERIMENTS if experiments else _build.LIB
        if not path.exists():
            _build.build(experiments=bool(experiments) and not short, short_waits=short)
        lib = C.CDLL(str(path))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError here = the build is stale or broken
            fn.restype = res
            fn.argtypes = args
        _libs[experiments] = lib
    return _libs[experiments]
