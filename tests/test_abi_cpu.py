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


def test_decode_entry_points_validate_without_a_gpu(built_lib):
    """Row limits, scratch sizes and argument checks of the decode-step entry points are host arithmetic."""
    from nativebit_b200 import _lib
    l = _lib.lib()
    fake = ctypes.c_void_p(4096)
    odd = ctypes.c_void_p(4100)
    # rows one launch of the multi-row matvec takes: what the staged rows leave of the shared memory
    assert l.nb_gemv_stream_max_rows(3, 2560) == 8 and l.nb_gemv_stream_max_rows(2, 2560) == 8
    assert l.nb_gemv_stream_max_rows(3, 6912) == 3 and l.nb_gemv_stream_max_rows(3, 128) == 8
    assert l.nb_gemv_stream_max_rows(3, 100) == 0 and l.nb_gemv_stream_max_rows(5, 2560) == 0
    assert l.nb_gemv_stream_rows(0, fake, 4, None, None, 0.0, None, fake, 3, 64, 6912, fake, 0, None) == 3      # four rows of 6912
    assert l.nb_gemv_stream_rows(1, fake, 2, None, None, 0.0, None, fake, 3, 64, 2560, fake, 0, None) == 1      # norm without a weight
    assert l.nb_gemv_stream_rows(0, odd, 2, None, None, 0.0, None, fake, 3, 64, 2560, fake, 0, None) == 2
    assert l.nb_gemv_stream(0, fake, 0, None, None, 0.0, None, fake, 3, 64, 7296, fake, 0, None) == 3        # K > 7168
    # LM head
    assert l.nb_lm_head_scratch_bytes() == 8192
    assert l.nb_lm_head(fake, None, None, 0.0, fake, 32000, 2500, 30.0, fake, fake, None, fake, None) == 3    # C % 256
    assert l.nb_lm_head(fake, None, None, 0.0, fake, 32000, 4096, 30.0, fake, fake, None, fake, None) == 3    # C > 3072
    assert l.nb_lm_head(fake, None, None, 0.0, fake, 32000, 2560, 0.0, fake, fake, None, fake, None) == 1     # cap must be positive
    # prompt attention
    args = (fake, 1, 16, 4, 80, fake, fake, 0, fake, fake, 64, fake, 320, 0, None)
    assert l.nb_prefill_attention(*args[:4], 130, *args[5:]) == 3                                            # head_dim > 128
    assert l.nb_prefill_attention(*args[:7], 60, *args[8:]) == 3                                             # pos0 + T > ctx
    assert l.nb_prefill_attention(*args[:12], 300, *args[13:]) == 3                                          # heads wider than the output row
    assert l.nb_prefill_attention(None, *args[1:]) == 1


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


def test_fused_and_exchange_argument_checks(built_lib):
    """Argument validation of the prologue / tensor-parallel entry points runs before any device call."""
    from nativebit_b200 import _lib
    l = _lib.lib()
    fake = ctypes.c_void_p(4096)
    ws = ctypes.c_void_p(8192)
    # nb_gemv_fused(prologue, x, delta, norm_weight, eps, x_out, M, packed, codebook, cb_dtype, bits, bs, N, K, y, y_dtype, ws, bytes, stream)
    assert l.nb_gemv_fused(3, fake, None, fake, 1e-6, None, 1, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20, None) == 1   # unknown prologue
    assert l.nb_gemv_fused(1, fake, None, None, 1e-6, None, 1, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20, None) == 1   # no norm weight
    assert l.nb_gemv_fused(1, fake, None, fake, 1e-6, fake, 1, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20, None) == 1   # x_out == x
    assert l.nb_gemv_fused(1, fake, None, fake, 1e-6, None, 9, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20, None) == 3   # M > 8
    odd = ctypes.c_void_p(4100)
    assert l.nb_gemv_fused(2, odd, None, None, 0.0, None, 1, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20, None) == 2     # x alignment
    # exchange
    assert l.nb_exchange_buffer_bytes(9, 1024) == 0 and l.nb_exchange_buffer_bytes(2, 1022) == 0
    assert l.nb_exchange_buffer_bytes(4, 2560) == 2 * 4 * 2560 * 4 + (2 * 4 + 2) * 4 + 64
    arr = (ctypes.c_uint64 * 2)(4096, 8192)
    assert l.nb_exchange_init(fake, arr, 2, 2, 1024) == 1            # rank out of range
    assert l.nb_exchange_init(fake, arr, 2, 1, 1024) == 1            # entry `rank` is not the own buffer
    assert l.nb_exchange_init(fake, (ctypes.c_uint64 * 2)(4096, 8200), 2, 0, 1024) == 2   # peer alignment
    # nb_gemv_tp(..., ws, bytes, exchange, world, rank, max_count, gather, push, spin, stream)
    common = (fake, None, fake, 1e-6, None, 1, fake, fake, 1, 3, 128, 16, 128, fake, 0, ws, 1 << 20)
    assert l.nb_gemv_tp(1, *common, None, 2, 0, 1024, 1, 0, 0, None) == 1       # no exchange buffer
    assert l.nb_gemv_tp(0, *common, fake, 2, 0, 1024, 1, 0, 0, None) == 3       # gather needs the RMSNorm prologue
    assert l.nb_gemv_tp(1, *common, fake, 2, 0, 64, 1, 0, 0, None) == 3         # M*K > max_count
    assert l.nb_gemv_tp(0, *common, fake, 2, 0, 8, 0, 1, 0, None) == 3          # M*N > max_count
    assert l.nb_gemv_tp(1, *common, fake, 2, 0, 1024, 0, 1, 0, None) == 1       # push after the RMSNorm prologue is not a row-parallel layer
    assert l.nb_exchange_gather(fake, 6, fake, 2, 0, 1024, 0, None, None) == 3  # count % 4
    # step ends
    assert l.nb_softcap_argmax(fake, 1, 1, 32000, 30.0, fake, fake, None, None) == 1     # fp16 logits are not supported
    assert l.nb_softcap_argmax(fake, 2, 1, 32000, 0.0, fake, fake, None, None) == 1      # cap must be positive
    assert l.nb_embed_rows(None, fake, 1, 10, 8, fake, None) == 1
    assert l.nb_decode_attention(fake, fake, fake, fake, 1, 4, 82, 64, fake, 328, 0, None) == 3   # head_dim % 4


def test_group_plan_shares_the_weight_bytes_evenly():
    """nb_group_build is host code: the plan of the benchmark's 78 matrices (no GPU needed; 148 CTAs are assumed
    without a device).  Every CTA's stretch of row tiles must be contiguous, cover the sequence exactly once and
    hold the mean share of units to within one row tile; bad lists are refused with a message."""
    import ctypes
    import struct
    from nativebit_b200 import _lib
    from nativebit_b200.stream import GroupItem
    l = _lib.lib()
    shapes = [(6912, 2560), (6912, 2560), (2560, 6912)] * 26
    arr = (GroupItem * len(shapes))()
    for i, (n, k) in enumerate(shapes):
        arr[i].w, arr[i].x, arr[i].y = 0x10000 * (i + 1), 0x1000 if k == 2560 else 0x2000, 0x7000000 + 0x10000 * i
        arr[i].n, arr[i].k, arr[i].x_dtype, arr[i].y_dtype = n, k, _lib.NB_BF16, _lib.NB_BF16
    nbytes = l.nb_group_plan_bytes(arr, len(shapes))
    buf = ctypes.create_string_buffer(nbytes)
    assert l.nb_group_build(arr, len(shapes), 3, buf, nbytes) == 0
    n_items, n_x, total_tiles, ctas, bits = struct.unpack_from("5i", buf.raw, 0)
    assert (n_items, n_x, bits) == (78, 2, 3) and total_tiles == 52 * 432 + 26 * 160 and ctas >= 1
    off = 32 + 6 * 32                                     # header, then six activation records
    cta_lo = struct.unpack_from("513i", buf.raw, off)
    assert cta_lo[0] == 0 and cta_lo[ctas] == total_tiles and all(a <= b for a, b in zip(cta_lo, cta_lo[1:]))
    off_items = (off + 513 * 4 + 7) // 8 * 8              # 256 records of 48 bytes, 8-byte aligned; the tile list follows them
    tile_list = struct.unpack_from(f"{total_tiles}i", buf.raw, off_items + 256 * 48)
    assert sorted(tile_list) == list(range(total_tiles))  # every row tile exactly once
    units = []                                            # units of every row tile, in the order of the matrices
    for n, k in shapes:
        units += [k // 128] * ((n + 15) // 16)
    share = sum(units) / ctas
    for c in range(ctas):
        mine = [units[t] for t in tile_list[cta_lo[c]:cta_lo[c + 1]]]
        assert mine == sorted(mine, reverse=True)         # the longest tiles first
        assert abs(sum(mine) - share) <= 20, (c, sum(mine), share)     # within one short tile of the mean
    # refusals
    arr[3].k = 100
    assert l.nb_group_build(arr, len(shapes), 3, buf, nbytes) != 0 and b"matvec 3" in l.nb_last_cuda_error()
    arr[3].k = 2560
    for i in range(7):
        arr[i].x = 0x100000 + 0x10000 * i                 # seven distinct activation vectors
    assert l.nb_group_build(arr, len(shapes), 3, buf, nbytes) != 0


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on the host cores alone (the oracle's mirror of the reference CPU path) and
    prints one JSON line with the keys the benchmark contract names."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "dequant_matvec_hbm_gbs" and line["unit"] == "GB/s"
    assert line["higher_is_better"] is True and line["scaling"] == "strong" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]
