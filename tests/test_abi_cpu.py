"""The C-ABI library on a machine without a GPU: it builds, loads, exports every symbol the
public header declares, validates arguments, and its unpack tables are self-consistent.
No kernel is launched here."""
import ctypes

import pytest


def test_library_exports_every_declared_symbol(built_lib):
    from nativebit_b200 import _lib
    handle = ctypes.CDLL(built_lib)
    names = _lib.declared_symbols()
    assert {"nb_unpack", "nb_pack", "nb_dequant", "nb_gemv", "nb_gemv_workspace_bytes"} <= set(names)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/nativebit_b200.h but not exported"
    assert set(_lib._SIGNATURES) == set(names), "ctypes signatures out of sync with the header"


def test_unpack_tables_self_test(built_lib):
    from nativebit_b200 import _lib
    assert _lib.lib().nb_selftest_tables() == 0
    assert _lib.lib().nb_version() >= 100
    assert _lib.lib().nb_status_string(3).decode() == "shape not supported"


def test_argument_validation_needs_no_gpu(built_lib):
    from nativebit_b200 import _lib
    l = _lib.lib()
    assert l.nb_unpack(None, 3, 8, None, None) == 1                      # NB_ERR_ARG
    assert l.nb_pack(None, 3, 8, None, None) == 1
    assert l.nb_dequant(None, None, 1, 3, 128, 4, 128, None, 0, None) == 1
    fake = ctypes.c_void_p(4096)
    assert l.nb_unpack(fake, 5, 8, fake, None) == 1                      # 5-bit is not supported
    assert l.nb_gemv(None, 2, 1, None, None, 1, 3, 128, 16, 128, None, 2, None, 0, None) == 1
    assert l.nb_gemv(fake, 2, 17, fake, fake, 1, 3, 128, 16, 128, fake, 2, None, 0, None) == 3   # M > 16
    assert l.nb_gemv(fake, 2, 1, fake, fake, 1, 3, 128, 16, 100, fake, 2, None, 0, None) == 3    # K % 128
    assert l.nb_gemv(fake, 2, 1, fake, fake, 1, 5, 128, 16, 128, fake, 2, None, 0, None) == 3    # 5-bit GEMV
    odd = ctypes.c_void_p(4100)
    assert l.nb_gemv(fake, 2, 1, odd, fake, 1, 3, 128, 16, 128, fake, 2, None, 0, None) == 2     # alignment


def test_workspace_size_is_bounded(built_lib):
    from nativebit_b200 import _lib
    l = _lib.lib()
    for m in (1, 4, 16):
        for n, k in ((6912, 2560), (2560, 6912), (2560, 2560), (7680, 2560)):
            b = l.nb_gemv_workspace_bytes(m, n, k, 3, 128)
            assert 0 < b < 32 << 20
    assert l.nb_gemv_workspace_bytes(1, 16, 100, 3, 128) == 0


def test_python_wrappers_refuse_cpu_tensors(built_lib):
    import torch
    import nativebit_b200 as nbt
    from nativebit_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.unpack(torch.zeros(3, dtype=torch.uint8), 3, 8)
    lin = nbt.PackedLinear(torch.zeros(48 * 16, dtype=torch.uint8), torch.zeros(16, 8, dtype=torch.float16), 16, 128)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        lin(torch.zeros(1, 128))
