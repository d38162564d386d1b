"""The C-ABI library loads here (no GPU) and exports every symbol include/qvx.h declares."""
import ctypes as C

import pytest

from qubivex_b200 import _lib
from qubivex_b200 import device as qd


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) > 60
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert sorted(_lib.PROTOTYPES) == declared, "the Python binding and the header list different functions"


def test_geometry_functions_need_no_device():
    geo = qd.geometry(16, 4, 128, qd.BF16, qd.LAYOUT_NATIVE)
    assert qd.block_bytes(geo) == 2 * 16 * 4 * 128 * 2
    assert qd.block_bytes(qd.geometry(16, 2, 16, qd.F32, qd.LAYOUT_NATIVE)) == 0
    assert qd.block_bytes(qd.geometry(256, 16, 128, qd.F32, qd.LAYOUT_REFERENCE)) == 4 * 2 * 256 * 16 * 128  # 4 MiB, the reference's block
    assert _lib.load().qvx_name() == b"cuda"


def test_the_library_and_the_oracle_agree_on_every_address():
    import oracle
    for layout, B, kvh, d, dt in [(0, 256, 2, 32, 0), (0, 16, 3, 24, 1), (1, 16, 4, 128, 1), (1, 32, 2, 64, 0), (1, 16, 1, 256, 2)]:
        go, gd = oracle.geometry(B, kvh, d, dt, layout), qd.geometry(B, kvh, d, dt, layout)
        assert oracle.block_bytes(go) == qd.block_bytes(gd)
        for at in (0, 1, B - 1, B, 3 * B + 5, 7 * B + 9):
            for kv in (0, 1):
                for g in range(kvh):
                    for i in (0, 1, 7, 8, d // 2, d - 1):
                        assert oracle.elem_offset(go, at, kv, g, i) == qd.elem_offset(gd, at, kv, g, i)


def test_without_a_gpu_the_device_refuses_to_open():
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a GPU is present")
    except ImportError:
        pass
    with pytest.raises(qd.DeviceError) as e:
        qd.CudaDevice(0)
    assert "no CPU path" in str(e.value)
