"""The CPU oracle against golden vectors produced by the reference's own functions
(tests/golden/make_golden.py), plus the round-trip cases of the reference's tests/test_pack.py."""
import os

import numpy as np
import pytest
import torch

from oracle import nb_oracle as o


def test_pack3_matches_reference_bytes(golden):
    for name in golden["p3_names"]:
        idx, packed = golden[f"p3_idx_{name}"], golden[f"p3_packed_{name}"]
        assert np.array_equal(o.pack_3bit(idx), packed), name
        assert np.array_equal(o.unpack_3bit(packed, idx.size), idx), name
        assert np.array_equal(o.pack_indices_to_3bit(idx), packed), name


def test_pack3_known_answer():
    # indices 0..7 -> 24-bit word 0o76543210 little endian (nativebit/pack.py:37-39)
    assert o.pack_3bit(np.arange(8)).tolist() == [0x88, 0xC6, 0xFA]
    assert o.pack_3bit(np.full(16, 7)).tolist() == [0xFF] * 6
    assert o.pack_3bit(np.zeros(16)).tolist() == [0] * 6
    assert o.pack_3bit(np.arange(8)).size == 3


@pytest.mark.parametrize("n", [1, 3, 7, 10, 13, 100, 1001, 100_000])
def test_pack3_roundtrip_lengths(n):
    idx = np.random.default_rng(n).integers(0, 8, n, dtype=np.uint8)
    assert np.array_equal(o.unpack_3bit(o.pack_3bit(idx), n), idx)


def test_pack4_and_nbits_match_reference(golden):
    assert np.array_equal(o.pack_4bit(golden["p4_idx"]), golden["p4_packed"])
    assert np.array_equal(o.unpack_4bit(golden["p4_packed"], 101), golden["p4_idx"])
    assert golden["p4_packed"].size == 51
    assert np.array_equal(o.pack_nbits(golden["p2_idx"], 2), golden["p2_packed"])
    assert np.array_equal(o.unpack_nbits(golden["p2_packed"], 203, 2), golden["p2_idx"])
    assert np.array_equal(o.pack_nbits(golden["p5_idx"], 5), golden["p5_packed"])
    assert np.array_equal(o.unpack_nbits(golden["p5_packed"], 50, 5), golden["p5_idx"])
    i3 = np.random.default_rng(0).integers(0, 8, 24, dtype=np.uint8)
    assert np.array_equal(o.pack_nbits(i3, 3), o.pack_3bit(i3))


def test_reconstruct_weight_matches_reference(golden):
    w = o.reconstruct_weight(golden["rw_small_idx"], golden["rw_small_cb"], (4, 8), 8, 32)
    assert np.array_equal(w, golden["rw_small_w"])
    for i in range(8):
        assert w.reshape(-1)[i] == golden["rw_small_cb"][0, golden["rw_small_idx"][i]]
    wp = o.reconstruct_weight(golden["rw_pad_idx"], golden["rw_pad_cb"], (2, 5), 8, 10)
    assert wp.shape == (2, 5) and np.array_equal(wp, golden["rw_pad_w"])


@pytest.mark.parametrize("bits", [3, 2])
def test_linear_matches_reference(golden, bits):
    tag = f"lin{bits}"
    n, k = golden[f"{tag}_shape"]
    packed, cb16, x = golden[f"{tag}_packed"], golden[f"{tag}_cb16"], golden[f"{tag}_x"]
    assert np.array_equal(o.pack_nbits(golden[f"{tag}_idx"], bits), packed)
    w = o.dequant_packed(packed, cb16.astype(np.float32), n, k, bits)
    assert np.array_equal(w, golden[f"{tag}_w"])          # bit-exact gather
    y = o.packed_linear_forward(x, packed, cb16.astype(np.float32), n, k, bits)
    # fp32 GEMM summation order differs between BLAS builds: tolerance 1e-5 of max|y|
    ref = golden[f"{tag}_y"]
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
    y64 = o.packed_linear_forward(x, packed, cb16.astype(np.float32), n, k, bits, acc_dtype=np.float64)
    assert np.abs(y64 - ref).max() <= 1e-5 * np.abs(ref).max()
    if bits == 3:
        assert np.array_equal(golden[f"{tag}_y_packedlinear"], ref) or \
            np.abs(golden[f"{tag}_y_packedlinear"] - ref).max() <= 1e-5 * np.abs(ref).max()


def test_fused_scalar_kernel_restatement(golden):
    n, k = golden["lin3_shape"]
    cb = golden["lin3_cb16"].astype(np.float32)
    y = o.fused_matvec_3bit(golden["lin3_x"][0], golden["lin3_packed"], cb, 8, int(k))
    ref = golden["lin3_y"][0, :8]
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(golden["lin3_y"]).max()


def test_torch_baseline_mirror_equals_oracle(golden):
    torch = pytest.importorskip("torch")
    n, k = (int(v) for v in golden["lin3_shape"])
    x = torch.from_numpy(golden["lin3_x"])
    packed = torch.from_numpy(golden["lin3_packed"])
    cb = torch.from_numpy(golden["lin3_cb16"].astype(np.float32))
    y = o.torch_reference_forward(x, packed, cb, n, k).numpy()
    ref = golden["lin3_y"]
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()
    idx = torch.from_numpy(golden["lin3_idx"].astype(np.int64)).view(-1, 128)
    y2 = o.torch_gather_forward(x, idx, cb, n, k).numpy()
    assert np.abs(y2 - ref).max() <= 1e-5 * np.abs(ref).max()


def test_synthetic_inputs_are_deterministic_and_sorted():
    packed, cb, idx = o.make_packed_linear(32, 256, 3, seed=0)
    packed2, cb2, _ = o.make_packed_linear(32, 256, 3, seed=0)
    assert np.array_equal(packed, packed2) and np.array_equal(cb, cb2)
    assert cb.dtype == np.float16 and cb.shape == (64, 8)
    assert np.all(np.diff(cb.astype(np.float32), axis=1) >= 0)
    assert packed.size == 32 * 256 * 3 // 8
    x = o.make_activation(4, 256, 0)
    assert np.array_equal(o.round_to_bf16(x), x)
    assert o.algorithmic_bytes(1, 6912, 2560, 3) == 8_866_304
    assert o.algorithmic_bytes(16, 6912, 2560, 3) == 9_150_464
    assert o.algorithmic_bytes(1, 2560, 2560, 3) == 3_287_040
    assert o.algorithmic_bytes(1, 6912, 2560, 2) == 5_548_544


def test_quantiser_restatement_matches_the_reference_argmin(golden):
    """quantize_weight against the indices the reference's quantiser produced for the same weight, and
    against the index bytes its exporter stored for a whole training checkpoint."""
    idx = o.quantize_weight(golden["quant_w"], golden["lin3_cb16"].astype(np.float32), 128)
    assert np.array_equal(idx.reshape(-1, 128), golden["quant_idx"])
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    ck = torch.load(os.path.join(here, "tiny_bs8_ckpt.pt"), map_location="cpu", weights_only=False)["model_state_dict"]
    blob = torch.load(os.path.join(here, "tiny_bs8.nbpack"), map_location="cpu", weights_only=False)
    for name, d in blob["quantized_layers"].items():
        idx = o.quantize_weight(ck[name + ".weight"].numpy(), ck[name + ".codebook"].numpy(), 8)
        assert np.array_equal(o.pack_3bit(idx), d["packed_indices"].numpy()), name
