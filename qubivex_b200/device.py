"""The CUDA device as the reference's runtime sees a discrete device.

`CudaDevice` mirrors the subset of `trait DiscreteDevice`
(crates/qubivex-compute/src/discrete.rs:433-570) that the paged decode path uses, with the
same names, argument meaning and error behaviour; every method is one call through the C ABI
of libqvx_cuda.so.  Errors mirror `ComputeError` (crates/qubivex-compute/src/lib.rs:26-83).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import Config, Geometry, KernelTimes, Prelude, TransferStats, Usage

F32, BF16, F16 = 0, 1, 2
LAYOUT_REFERENCE, LAYOUT_NATIVE = 0, 1
ATTN_AUTO, ATTN_SPLIT, ATTN_EXACT = 0, 1, 2
ATTN_POOL_SETTLED = 0x100  # or-ed into a variant: see QVX_ATTN_POOL_SETTLED in include/qvx.h
KV_BLOCK = 256  # crates/qubivex-compute/src/discrete.rs:248


class ComputeError(Exception):
    """crates/qubivex-compute/src/lib.rs:26-83."""


class ShapeError(ComputeError):
    pass


class Unsupported(ComputeError):
    pass


class CoreError(ComputeError):
    pass


class OutOfDeviceMemory(ComputeError):
    pass


class DeviceError(ComputeError):
    pass


_ERRORS = {-1: ShapeError, -2: Unsupported, -3: CoreError, -4: ComputeError, -5: ComputeError,
           -6: OutOfDeviceMemory, -7: DeviceError}


def ptr(x):
    """A raw address for the C ABI from a numpy array, a torch tensor, an int or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return C.c_void_p(x)
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("host arrays must be contiguous")
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):
        if not x.is_contiguous():
            raise ValueError("tensors must be contiguous")
        return C.c_void_p(x.data_ptr())
    raise TypeError(f"cannot pass {type(x)} through the C ABI")


def geometry(block_tokens: int, kv_heads: int, head_dim: int, dtype: int = F32, layout: int = LAYOUT_NATIVE) -> Geometry:
    return Geometry(block_tokens, kv_heads, head_dim, dtype, layout)


def block_bytes(geo: Geometry) -> int:
    """kv_block_words x element size (discrete.rs:253-256)."""
    return _lib.load().qvx_block_bytes(C.byref(geo))


def elem_offset(geo: Geometry, at: int, kv: int, g: int, i: int) -> int:
    """kv_key_word / kv_value_word in bytes (discrete.rs:317-329)."""
    return _lib.load().qvx_elem_offset(C.byref(geo), at, kv, g, i)


@dataclass
class DeviceBuffer:
    """crates/qubivex-compute/src/discrete.rs:36-95: device memory, freed with its last holder."""
    device: "CudaDevice"
    handle: int

    def __len__(self) -> int:
        return self.device.lib.qvx_buffer_len(self.handle)

    @property
    def ptr(self) -> int:
        return self.device.lib.qvx_buffer_ptr(self.handle) or 0

    def free(self) -> None:
        if self.handle:
            self.device.lib.qvx_free(self.handle)
            self.handle = 0


class CudaDevice:
    """`impl DiscreteDevice for CudaDevice`, the decode-attention subset."""

    def __init__(self, device: int = 0, capacity: int = 0, kv_pool: int = 0, timing: int | bool = False,
                 experiments: bool = False):
        # experiments: the build whose chunk and run-length rules can be set through the environment
        self.lib = _lib.load(experiments)
        self.h = C.c_void_p()
        cfg = Config(device, capacity, kv_pool, int(timing))  # timing = n: CUDA events around every n-th launch
        rc = self.lib.qvx_open(C.byref(cfg), C.byref(self.h))
        if rc:
            raise _ERRORS.get(rc, ComputeError)(self.lib.qvx_last_error(None).decode())

    def close(self) -> None:
        if self.h:
            self.lib.qvx_close(self.h)
            self.h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def check(self, rc: int) -> bool:
        """0 -> True (ran), 1 -> False (declined, nothing written), < 0 -> the ComputeError."""
        if rc == 0:
            return True
        if rc == 1:
            return False
        raise _ERRORS.get(rc, ComputeError)(self.lib.qvx_last_error(self.h).decode())

    # -- DiscreteDevice ------------------------------------------------------------------
    def name(self) -> str:
        return self.lib.qvx_name().decode()

    def describe(self) -> str:
        buf = C.create_string_buffer(256)
        self.check(self.lib.qvx_describe(self.h, buf, 256))
        return buf.value.decode()

    def supports(self, dtype: int) -> bool:
        return bool(self.lib.qvx_supports(self.h, dtype))

    def upload(self, host) -> DeviceBuffer:
        a = np.ascontiguousarray(host)
        out = C.c_void_p()
        self.check(self.lib.qvx_upload(self.h, ptr(a), a.nbytes, C.byref(out)))
        return DeviceBuffer(self, out.value)

    def alloc(self, length: int) -> DeviceBuffer:
        out = C.c_void_p()
        self.check(self.lib.qvx_alloc(self.h, length, C.byref(out)))
        return DeviceBuffer(self, out.value)

    def write(self, buffer: DeviceBuffer, offset: int, host) -> None:
        a = np.ascontiguousarray(host)
        self.check(self.lib.qvx_write(self.h, buffer.handle, offset, ptr(a), a.nbytes))

    def read(self, buffer: DeviceBuffer, offset: int, length: int) -> np.ndarray:
        out = np.empty(length, dtype=np.uint8)
        self.check(self.lib.qvx_read(self.h, buffer.handle, offset, ptr(out), length))
        return out

    def usage(self) -> Usage:
        u = Usage()
        self.check(self.lib.qvx_get_usage(self.h, C.byref(u)))
        return u

    def transfers(self) -> TransferStats:
        t = TransferStats()
        self.check(self.lib.qvx_get_transfers(self.h, C.byref(t)))
        return t

    def kernel_times(self) -> dict:
        k = KernelTimes()
        self.check(self.lib.qvx_get_kernel_times(self.h, C.byref(k)))
        return {n: (int(k.launches[i]), int(k.gpu_ns[i])) for i, n in enumerate(_lib.KERNEL_NAMES)}

    def reset_kernel_times(self) -> None:
        self.check(self.lib.qvx_reset_kernel_times(self.h))

    def kv_pool(self):
        v = self.lib.qvx_kv_pool(self.h)
        return v or None

    def max_arena(self) -> int:
        return self.lib.qvx_max_arena(self.h)

    def routes_moe_attention(self, experts: int, k: int, s: int) -> bool:
        return bool(self.lib.qvx_routes_moe_attention(self.h, experts, k, s))

    # -- the attention stage of routed_moe (DeviceMoeAttention, discrete.rs:266-307) -----------
    def paged_attention(self, pool: DeviceBuffer, geo: Geometry, heads: int, q, k_new, v_new, pos, blocks, table_at,
                        sync=None, sync_to=None, out=None, variant: int = ATTN_AUTO, wait: bool = True):
        """Sync rows, new rows, attention over 0..=pos[t].  Host arrays in, host array out."""
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        blocks = np.ascontiguousarray(blocks, dtype=np.uint32)
        table_at = np.ascontiguousarray(table_at, dtype=np.uint32)
        s = len(pos)
        kv_out = geo.kv_heads * geo.head_dim
        n_sync = 0 if sync_to is None else len(sync_to)
        if sync_to is not None:
            sync_to = np.ascontiguousarray(sync_to, dtype=np.uint32)
        # The length checks of sim.rs:313-324 (a slice carries its length, a pointer does not).
        sizes_ok = (len(table_at) == s and _numel(q) == s * heads * geo.head_dim and _numel(k_new) == s * kv_out
                    and _numel(v_new) == s * kv_out and (0 if sync is None else _numel(sync)) == n_sync * 2 * kv_out)
        if not sizes_ok or heads % max(geo.kv_heads, 1) != 0:
            raise ShapeError(f"shape mismatch in routed moe attention: {s} tokens, {heads} heads, "
                             f"{geo.kv_heads} KV heads of {geo.head_dim}")
        if out is None:
            out = np.empty((s, heads, geo.head_dim), dtype=np.float32)
        fn = self.lib.qvx_paged_attention_host if wait else self.lib.qvx_paged_attention_host_async
        keep = (pos, blocks, table_at, sync_to, q, k_new, v_new, sync)
        rc = fn(self.h, pool.handle, C.byref(geo), heads, s, ptr(q), ptr(k_new), ptr(v_new), ptr(pos), ptr(blocks),
                len(blocks), ptr(table_at), ptr(sync), ptr(sync_to), n_sync, ptr(out), variant)
        self.check(rc)
        if not wait:
            self._keep = getattr(self, "_keep", [])
            self._keep.append(keep)
        return out

    def attention_stage(self, pool: DeviceBuffer, geo: Geometry, heads: int, q, k_new, v_new, rope, pos, blocks, table_at,
                        clip=None, qk_norm=None, eps: float = 1e-6, sync=None, sync_to=None, variant: int = ATTN_AUTO):
        """DeviceMoeAttention after the projections (sim.rs:325-429): clip, full-width Q/K norms, RoPE, then the
        sync rows, the new rows and attention.  k_new and v_new (f32 host arrays) are rewritten in place,
        as the reference leaves them for the host cache; returns the attention outputs."""
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        blocks = np.ascontiguousarray(blocks, dtype=np.uint32)
        table_at = np.ascontiguousarray(table_at, dtype=np.uint32)
        s, d = len(pos), geo.head_dim
        kv_out = geo.kv_heads * d
        n_sync = 0 if sync_to is None else len(sync_to)
        if sync_to is not None:
            sync_to = np.ascontiguousarray(sync_to, dtype=np.uint32)
        rope = np.ascontiguousarray(rope, dtype=np.float32)
        for a in (k_new, v_new):
            if not (isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]):
                raise TypeError("k_new and v_new are written back: contiguous float32 arrays")
        sizes_ok = (len(table_at) == s and rope.size == s * d and _numel(q) == s * heads * d and k_new.size == s * kv_out
                    and v_new.size == s * kv_out and (0 if sync is None else _numel(sync)) == n_sync * 2 * kv_out)
        qn = kn = None
        if qk_norm is not None:
            qn = np.ascontiguousarray(qk_norm[0], dtype=np.float32)
            kn = np.ascontiguousarray(qk_norm[1], dtype=np.float32)
            sizes_ok = sizes_ok and qn.size == heads * d and kn.size == kv_out
        if not sizes_ok or heads % max(geo.kv_heads, 1) != 0:
            raise ShapeError(f"shape mismatch in routed moe attention: {s} tokens, {heads} heads, "
                             f"{geo.kv_heads} KV heads of {d}")
        pre = Prelude(0 if clip is None else 1, 0.0 if clip is None else float(clip),
                      None if qn is None else qn.ctypes.data, None if kn is None else kn.ctypes.data, float(eps), rope.ctypes.data)
        out = np.empty((s, heads, d), dtype=np.float32)
        self.check(self.lib.qvx_attention_stage_host(self.h, pool.handle, C.byref(geo), heads, s, ptr(q), ptr(k_new), ptr(v_new),
                                                     C.byref(pre), ptr(pos), ptr(blocks), len(blocks), ptr(table_at), ptr(sync),
                                                     ptr(sync_to), n_sync, ptr(out), variant))
        return out

    def wait(self) -> None:
        rc = self.lib.qvx_wait(self.h)
        self._keep = []
        self.check(rc)

    def block_copy(self, pool: DeviceBuffer, geo: Geometry, src, dst) -> None:
        src = np.ascontiguousarray(src, dtype=np.uint32)
        dst = np.ascontiguousarray(dst, dtype=np.uint32)
        if len(src) != len(dst):
            raise ShapeError("shape mismatch in block copy: lists differ in length")
        self.check(self.lib.qvx_block_copy_host(self.h, pool.handle, C.byref(geo), ptr(src), ptr(dst), len(src)))


def _numel(x) -> int:
    if x is None:
        return 0
    if isinstance(x, np.ndarray):
        return x.size
    return x.numel()
