"""Generate the golden vectors in this folder by importing the reference's own Python.

Run once, in a container that has the reference checkout (it is not needed at test
time):   python tests/golden/make_golden.py /path/to/reference

Every array written here is the output of a reference function
(nativebit/pack.py, nativebit/inference.py, inference/triton_kernel.py,
inference/pack.py, inference/generate_torch.py) on seeded inputs that are stored
alongside, so the tests can replay the inputs through the oracle and through the
CUDA path and demand identical bytes / stated-tolerance floats.
"""
import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from nativebit.pack import (pack_3bit, unpack_3bit, pack_4bit, unpack_4bit, pack_nbits,
                                unpack_nbits, reconstruct_weight)
    from nativebit.inference import NativeBitInferenceLinear
    from nativebit.codebook_utils import init_codebook_percentile
    from inference.triton_kernel import PackedLinear, pack_indices_to_3bit
    from inference.pack import pack_indices_3bit, quantize_weight
    from inference.generate_torch import unpack_indices_3bit

    out = {}
    g = torch.Generator().manual_seed(0)

    # ---- 3-bit packing: the cases of the reference's tests/test_pack.py:25-67
    cases = {
        "arange8": torch.arange(8, dtype=torch.uint8),
        "zeros16": torch.zeros(16, dtype=torch.uint8),
        "sevens16": torch.full((16,), 7, dtype=torch.uint8),
        "rand1024": torch.randint(0, 8, (1024,), dtype=torch.uint8, generator=g),
    }
    for n in [1, 3, 7, 10, 13, 100, 1001]:
        cases[f"rand{n}"] = torch.randint(0, 8, (n,), dtype=torch.uint8, generator=g)
    out["p3_names"] = np.array(sorted(cases))
    for name, idx in cases.items():
        packed = pack_3bit(idx)
        assert torch.equal(unpack_3bit(packed, idx.numel()), idx)
        out[f"p3_idx_{name}"] = idx.numpy()
        out[f"p3_packed_{name}"] = packed.numpy()

    # ---- 4-bit, 2-bit and 5-bit (tests/test_pack.py:74-114)
    i4 = torch.randint(0, 16, (101,), dtype=torch.uint8, generator=g)
    out["p4_idx"], out["p4_packed"] = i4.numpy(), pack_4bit(i4).numpy()
    assert torch.equal(unpack_4bit(pack_4bit(i4), 101), i4)
    i2 = torch.randint(0, 4, (203,), dtype=torch.uint8, generator=g)
    out["p2_idx"], out["p2_packed"] = i2.numpy(), pack_nbits(i2, 2).numpy()
    assert torch.equal(unpack_nbits(pack_nbits(i2, 2), 203, 2), i2)
    i5 = torch.randint(0, 32, (50,), dtype=torch.uint8, generator=g)
    out["p5_idx"], out["p5_packed"] = i5.numpy(), pack_nbits(i5, 5).numpy()

    # ---- loader-side packers agree with pack_3bit
    r = cases["rand1024"]
    assert torch.equal(pack_indices_to_3bit(r), pack_3bit(r))
    assert np.array_equal(np.frombuffer(pack_indices_3bit(r.numpy()), np.uint8), pack_3bit(r).numpy())
    assert np.array_equal(unpack_indices_3bit(pack_3bit(r).numpy(), (8, 128)), r.numpy().reshape(8, 128))

    # ---- reconstruct_weight: block 8 basic + padding (tests/test_pack.py:121-151)
    cb_small = torch.randn(4, 8, generator=g)
    idx_small = torch.randint(0, 8, (32,), generator=g)
    out["rw_small_cb"], out["rw_small_idx"] = cb_small.numpy(), idx_small.numpy().astype(np.uint8)
    out["rw_small_w"] = reconstruct_weight(idx_small, cb_small, (4, 8), 8, 32).numpy()
    cb_pad = torch.randn(2, 8, generator=g)
    idx_pad = torch.randint(0, 8, (16,), generator=g)
    out["rw_pad_cb"], out["rw_pad_idx"] = cb_pad.numpy(), idx_pad.numpy().astype(np.uint8)
    out["rw_pad_w"] = reconstruct_weight(idx_pad, cb_pad, (2, 5), 8, 10).numpy()

    # ---- one packed linear at block 128: 3-bit (K=8) and 2-bit (K=4)
    for bits, n, k in [(3, 48, 384), (2, 32, 256)]:
        ne = 1 << bits
        nb = n * k // 128
        z = torch.randn(nb, 128, generator=g)
        scale = torch.empty(nb, 1).uniform_(0.01, 0.05, generator=g)
        cb = torch.stack([init_codebook_percentile(z[b], ne) for b in range(nb)]) * scale
        cb16 = cb.half()
        idx = torch.randint(0, ne, (nb * 128,), dtype=torch.uint8, generator=g)
        packed = pack_nbits(idx, bits)
        x = torch.randn(3, k, generator=g).bfloat16().float()
        w = reconstruct_weight(unpack_nbits(packed, nb * 128, bits), cb16.float(), (n, k), 128, n * k)
        lin = NativeBitInferenceLinear(k, n, cb16.float(), idx.view(nb, 128).long(), 128)
        y = lin(x)
        tag = f"lin{bits}"
        out[f"{tag}_shape"] = np.array([n, k])
        out[f"{tag}_idx"], out[f"{tag}_packed"] = idx.numpy(), packed.numpy()
        out[f"{tag}_cb16"] = cb16.numpy()
        out[f"{tag}_x"], out[f"{tag}_w"], out[f"{tag}_y"] = x.numpy(), w.numpy(), y.numpy()
        if bits == 3:
            # the reference's packed module, batched (M>1) path, run on CPU
            pl = PackedLinear(packed, cb16.float(), n, k)
            y_pl = pl(x)
            assert torch.equal(y_pl, x @ w.T)
            out[f"{tag}_y_packedlinear"] = y_pl.numpy()
            # the .nbpack.npz quantiser: nearest entry (squared distance) -> indices
            wq = (w + 0.001 * torch.randn(n, k, generator=g)).numpy()
            out["quant_w"] = wq
            out["quant_idx"] = quantize_weight(wq, cb16.float().numpy())

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} <path of the NativeBit reference checkout>")
    main(sys.argv[1])
