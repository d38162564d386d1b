"""Python face of the CPU oracle (oracle/qvx_oracle.c).  TEST INFRASTRUCTURE ONLY.

Imported by tests/, by `__graft_entry__.smoke()` and by bench.py's CPU-baseline legs, as the
checker and the timed CPU baseline.  The shipped package (qubivex_b200) never imports it.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libqvx_oracle.so"

F32, BF16, F16 = 0, 1, 2
LAYOUT_REFERENCE, LAYOUT_NATIVE = 0, 1


class Geometry(C.Structure):
    _fields_ = [("block_tokens", C.c_uint32), ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("dtype", C.c_uint32), ("layout", C.c_uint32)]


def build(force: bool = False) -> Path:
    src = HERE / "qvx_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B"], check=True, capture_output=True)
    return LIB


_lib = None
P = C.c_void_p
_G = C.POINTER(Geometry)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB))
        L.qvo_exp.restype = C.c_float
        L.qvo_exp.argtypes = [C.c_float]
        L.qvo_exp_array.argtypes = [P, P, C.c_size_t]
        L.qvo_narrow_array.argtypes = [P, P, C.c_size_t, C.c_uint32]
        L.qvo_widen_array.argtypes = [P, P, C.c_size_t, C.c_uint32]
        L.qvo_softmax.argtypes = [P, C.c_size_t]
        L.qvo_attend.argtypes = [P, P, P, C.c_size_t, C.c_size_t, P, P]
        L.qvo_reduce_dot.restype = C.c_float
        L.qvo_reduce_dot.argtypes = [P, P, C.c_size_t]
        L.qvo_rms_scale_of.restype = C.c_float
        L.qvo_rms_scale_of.argtypes = [C.c_float, C.c_float, C.c_float]
        L.qvo_rms_norm.argtypes = [P, P, C.c_size_t, C.c_double]
        L.qvo_rope_rotate.argtypes = [P, P, C.c_size_t]
        L.qvo_attn_prelude.argtypes = [P, P, P, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_float, P, P,
                                       C.c_double, P]
        L.qvo_f32_to_bf16.restype = C.c_uint16
        L.qvo_f32_to_bf16.argtypes = [C.c_float]
        L.qvo_bf16_to_f32.restype = C.c_float
        L.qvo_bf16_to_f32.argtypes = [C.c_uint16]
        L.qvo_f32_to_f16.restype = C.c_uint16
        L.qvo_f32_to_f16.argtypes = [C.c_float]
        L.qvo_f16_to_f32.restype = C.c_float
        L.qvo_f16_to_f32.argtypes = [C.c_uint16]
        L.qvo_block_bytes.restype = C.c_size_t
        L.qvo_block_bytes.argtypes = [_G]
        L.qvo_geometry_ok.argtypes = [_G]
        L.qvo_elem_offset.restype = C.c_size_t
        L.qvo_elem_offset.argtypes = [_G, C.c_size_t, C.c_int, C.c_size_t, C.c_size_t]
        L.qvo_kv_write.argtypes = [P, C.c_size_t, _G, C.c_size_t, P, P, P, P, C.c_size_t, P, P, P, C.c_size_t]
        L.qvo_attn_decode.argtypes = [P, C.c_size_t, _G, C.c_size_t, C.c_size_t, P, P, P, C.c_size_t, P, P]
        L.qvo_attn_decode_par.argtypes = [P, C.c_size_t, _G, C.c_size_t, C.c_size_t, P, P, P, C.c_size_t, P, P, C.c_int]
        L.qvo_paged_attention.argtypes = [P, C.c_size_t, _G, C.c_size_t, C.c_size_t, P, P, P, P, P, C.c_size_t, P, P,
                                          P, C.c_size_t, P]
        L.qvo_block_copy.argtypes = [P, C.c_size_t, _G, P, P, C.c_size_t]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint32)


def geometry(block_tokens, kv_heads, head_dim, dtype=F32, layout=LAYOUT_NATIVE) -> Geometry:
    return Geometry(block_tokens, kv_heads, head_dim, dtype, layout)


def exp(x: float) -> float:
    return lib().qvo_exp(x)


def exp_bits(x: float) -> int:
    return int(np.float32(lib().qvo_exp(x)).view(np.uint32))


def exp_array(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().qvo_exp_array(_p(x), _p(y), x.size)
    return y


def narrow(x, dtype: int) -> np.ndarray:
    """f32 -> the 16-bit pool element's bits."""
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().qvo_narrow_array(_p(x), _p(y), x.size, dtype)
    return y


def widen(h, dtype: int) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    y = np.empty(h.shape, dtype=np.float32)
    lib().qvo_widen_array(_p(h), _p(y), h.size, dtype)
    return y


def softmax(x) -> np.ndarray:
    a = _f32(x).copy()
    lib().qvo_softmax(_p(a), a.size)
    return a


def attend(q, k, v, pos: int) -> np.ndarray:
    q, k, v = _f32(q), _f32(k), _f32(v)
    d = q.size
    out = np.zeros(d, dtype=np.float32)
    scores = np.zeros(pos + 1, dtype=np.float32)
    lib().qvo_attend(_p(q), _p(k), _p(v), d, pos, _p(out), _p(scores))
    return out


def reduce_dot(w, x) -> float:
    w, x = _f32(w), _f32(x)
    return lib().qvo_reduce_dot(_p(w), _p(x), w.size)


def attn_prelude(q, k_new, v_new, heads: int, kv_heads: int, d: int, rope, clip=None, qk_norm=None, eps: float = 1e-6):
    """clip, full-width Q/K norms, RoPE (sim.rs:333-357) on copies of the raw projections: returns (q, k_new, v_new)."""
    q, k_new, v_new = (np.array(a, dtype=np.float32, copy=True).reshape(-1) for a in (q, k_new, v_new))
    s = k_new.size // (kv_heads * d)
    rope = _f32(rope)
    qn = kn = None
    if qk_norm is not None:
        qn, kn = _f32(qk_norm[0]), _f32(qk_norm[1])
    lib().qvo_attn_prelude(_p(q), _p(k_new), _p(v_new), s, heads, kv_heads, d, 0 if clip is None else 1,
                           0.0 if clip is None else float(clip), None if qn is None else _p(qn), None if kn is None else _p(kn),
                           float(eps), _p(rope))
    return q.reshape(s, heads, d), k_new.reshape(s, kv_heads * d), v_new.reshape(s, kv_heads * d)


def block_bytes(geo: Geometry) -> int:
    return lib().qvo_block_bytes(C.byref(geo))


def elem_offset(geo: Geometry, at: int, kv: int, g: int, i: int) -> int:
    return lib().qvo_elem_offset(C.byref(geo), at, kv, g, i)


def kv_write(pool: np.ndarray, geo: Geometry, k_new, v_new, pos, blocks, table_at, sync=None, sync_to=None) -> int:
    """Sync rows then new rows into `pool` (a uint8 array), in place.  Returns the status."""
    k_new, v_new, sync = _f32(k_new), _f32(v_new), _f32(sync)
    pos, blocks, table_at, sync_to = _u32(pos), _u32(blocks), _u32(table_at), _u32(sync_to)
    s = 0 if pos is None else len(pos)
    return lib().qvo_kv_write(_p(pool), pool.size // block_bytes(geo), C.byref(geo), s, _p(k_new), _p(v_new), _p(pos),
                              _p(blocks), 0 if blocks is None else len(blocks), _p(table_at), _p(sync), _p(sync_to),
                              0 if sync_to is None else len(sync_to))


def attn_decode(pool: np.ndarray, geo: Geometry, heads: int, q, pos, blocks, table_at, threads: int = 0):
    """(status, att[s, heads, d]).  threads > 0: the host path's (token, head) tasks on that many threads."""
    q, pos, blocks, table_at = _f32(q), _u32(pos), _u32(blocks), _u32(table_at)
    s = len(pos)
    att = np.zeros((s, heads, geo.head_dim), dtype=np.float32)
    args = (_p(pool), pool.size // block_bytes(geo), C.byref(geo), heads, s, _p(q), _p(pos), _p(blocks), len(blocks),
            _p(table_at), _p(att))
    rc = lib().qvo_attn_decode_par(*args, threads) if threads > 0 else lib().qvo_attn_decode(*args)
    return rc, att


def paged_attention(pool: np.ndarray, geo: Geometry, heads: int, q, k_new, v_new, pos, blocks, table_at, sync=None,
                    sync_to=None):
    """The whole op in the reference's order.  (status, att)."""
    q, k_new, v_new, sync = _f32(q), _f32(k_new), _f32(v_new), _f32(sync)
    pos, blocks, table_at, sync_to = _u32(pos), _u32(blocks), _u32(table_at), _u32(sync_to)
    s = len(pos)
    att = np.zeros((s, heads, geo.head_dim), dtype=np.float32)
    rc = lib().qvo_paged_attention(_p(pool), pool.size // block_bytes(geo), C.byref(geo), heads, s, _p(q), _p(k_new),
                                   _p(v_new), _p(pos), _p(blocks), len(blocks), _p(table_at), _p(sync), _p(sync_to),
                                   0 if sync_to is None else len(sync_to), _p(att))
    return rc, att


def block_copy(pool: np.ndarray, geo: Geometry, src, dst) -> int:
    src, dst = _u32(src), _u32(dst)
    return lib().qvo_block_copy(_p(pool), pool.size // block_bytes(geo), C.byref(geo), _p(src), _p(dst), len(src))
