"""The tcgen05 prefill GEMM through the C ABI: the tensor-core kernel alone against an fp64
product of the same bf16 operands, and the packed entry point against the oracle (the weights
enter the tensor cores as the exact fp16 codebook entries, so the result matches the fp64 product
of the reference's weights to fp32-accumulation accuracy, far inside the stated 2e-3 gate)."""
import numpy as np
import pytest
import torch

from oracle import nb_oracle as o

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 128), (128, 256, 512), (256, 384, 2560), (200, 384, 256),
                                   (130, 200, 128), (1, 128, 64), (2048, 2560, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16_kernel(built_lib, m, n, k, out_dtype):
    from nativebit_b200 import ops
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(m + n + k)
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w = (torch.randn(n, k, device=dev, generator=g) * 0.05).bfloat16()
    y = ops.gemm_bf16(x, w, out_dtype=out_dtype)
    torch.cuda.synchronize()
    ref = x.double() @ w.double().T
    tol = 2e-5 if out_dtype == torch.float32 else 2.0 ** -8     # bf16 output: half an ulp of bf16
    assert (y.double() - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("bits,m,n,k", [(3, 128, 256, 384), (3, 300, 640, 1280), (2, 256, 256, 512), (3, 2048, 6912, 2560),
                                        (3, 2048, 2560, 6912)])
def test_gemm_prefill_packed(built_lib, bits, m, n, k):
    from nativebit_b200 import ops
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=m)
    x = o.make_activation(m, k, seed=m)                                  # bf16-representable
    xt = torch.from_numpy(x).to(dev)
    y = ops.gemm_prefill(xt.bfloat16(), torch.from_numpy(packed).to(dev), torch.from_numpy(cb).to(dev), bits, 128, n, k,
                         out_dtype=torch.float32)
    torch.cuda.synchronize()
    W = torch.from_numpy(o.dequant_packed(packed, cb.astype(np.float32), n, k, bits)).to(dev)
    ref_exact = xt.double() @ W.double().T                               # the reference's fp32 weights
    assert (y.double() - ref_exact).abs().max() <= 2e-5 * ref_exact.abs().max()


def test_packed_linear_uses_tensor_core_path_for_long_inputs(built_lib):
    import nativebit_b200 as nbt
    dev = _dev()
    n, k, m = 640, 1280, 512
    packed, cb, _ = o.make_packed_linear(n, k, 3, seed=3)
    lin = nbt.PackedLinear(torch.from_numpy(packed).to(dev), torch.from_numpy(cb).to(dev), n, k)
    x = torch.from_numpy(o.make_activation(m, k, 4)).to(dev).bfloat16()
    y = lin(x)
    assert y.dtype == torch.bfloat16 and y.shape == (m, n)
    ref = o.packed_linear_forward(x.float().cpu().numpy(), packed, cb.astype(np.float32), n, k, 3, acc_dtype=np.float64)
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 2.0 ** -8 * np.abs(ref).max()     # bf16 output: half an ulp


@pytest.mark.parametrize("bits,m,n,k", [(3, 128, 256, 384), (3, 300, 640, 1280), (2, 256, 256, 512), (4, 130, 200, 256), (3, 17, 1000, 640),
                                        (3, 64, 2560, 2560), (3, 1, 128, 128), (3, 2048, 6912, 2560), (3, 2048, 2560, 6912)])
@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float16, torch.float32])
def test_fused_dequant_gemm(built_lib, bits, m, n, k, xdt):
    """The kernel that dequantises inside the tensor-core pipeline, against the fp64 product with the
    reference's dense weights: ragged M and N, every packed format, all activation types."""
    from nativebit_b200 import ops, stream as S
    dev = _dev()
    if xdt != torch.bfloat16 and m == 2048 and k == 6912:
        pytest.skip("one activation type is enough at the largest shape")
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=m + 1)
    x = o.make_activation(m, k, seed=m)                                  # bf16-representable
    if xdt == torch.float32:
        x = (x.astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)   # needs both fp16 terms
    w = S.stream_pack(torch.from_numpy(packed).to(dev), torch.from_numpy(cb).to(dev), bits, n, k)
    xt = torch.from_numpy(x).to(dev).to(xdt)
    y = ops.gemm_prefill_fused(xt, w, bits, n, k, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ops.prefill_status(dev) == 0
    W = torch.from_numpy(o.dequant_packed(packed, cb.astype(np.float32), n, k, bits)).to(dev)
    ref = xt.double() @ W.double().T
    assert (y.double() - ref).abs().max() <= 2e-5 * ref.abs().max()
    yb = ops.gemm_prefill_fused(xt, w, bits, n, k, out_dtype=torch.bfloat16) if xdt != torch.float32 else None
    if yb is not None:
        assert (yb.double() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()     # bf16 output: half an ulp


@pytest.mark.parametrize("bits,m,n,k,xdt", [(3, 64, 2560, 6912, torch.float32), (3, 128, 2560, 2560, torch.bfloat16), (2, 32, 1000, 1280, torch.float16),
                                            (4, 40, 1002, 640, torch.float32), (3, 512, 2560, 6912, torch.bfloat16), (3, 18, 384, 7168, torch.float32)])
def test_fused_dequant_gemm_with_k_splits(built_lib, bits, m, n, k, xdt):
    """Short inputs: the k range of an output tile is cut into parts that run on different SMs and a second kernel adds
    their fp32 results in k order (1002 outputs per row cannot use the four-wide summing kernel and stay unsplit).  Against
    the fp64 product with the reference's dense weights, for both output types, and twice: bit-identical."""
    from nativebit_b200 import ops, stream as S
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(n, k, bits, seed=n + 7)
    x = o.make_activation(m, k, seed=m + 3)
    if xdt == torch.float32:
        x = (x.astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)   # needs both fp16 terms
    w = S.stream_pack(torch.from_numpy(packed).to(dev), torch.from_numpy(cb).to(dev), bits, n, k)
    xt = torch.from_numpy(x).to(dev).to(xdt)
    W = torch.from_numpy(o.dequant_packed(packed, cb.astype(np.float32), n, k, bits)).to(dev)
    ref = xt.double() @ W.double().T
    y1 = ops.gemm_prefill_fused(xt, w, bits, n, k, out_dtype=torch.float32)
    y2 = ops.gemm_prefill_fused(xt, w, bits, n, k, out_dtype=torch.float32)
    yb = ops.gemm_prefill_fused(xt, w, bits, n, k, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert ops.prefill_status(dev) == 0
    assert (y1.double() - ref).abs().max() <= 2e-5 * ref.abs().max()
    assert torch.equal(y1, y2)
    assert (yb.double() - ref).abs().max() <= 2.0 ** -8 * ref.abs().max()


@pytest.mark.parametrize("m,n,k", [(130, 200, 256), (1100, 640, 1280)])
def test_dequant_then_gemm_with_fp32_activations(built_lib, m, n, k):
    """The two-kernel form with fp32 activations: the library splits them into two fp16 terms in adjacent operand rows
    and the epilogue adds the pair's results; 1100 rows is also what PackedLinear sends this way."""
    import nativebit_b200 as nbt
    from nativebit_b200 import ops
    dev = _dev()
    packed, cb, _ = o.make_packed_linear(n, k, 3, seed=m)
    x = (o.make_activation(m, k, seed=m).astype(np.float64) * (1.0 + 1e-4 * np.arange(k))).astype(np.float32)
    xt = torch.from_numpy(x).to(dev)
    p, c = torch.from_numpy(packed).to(dev), torch.from_numpy(cb).to(dev)
    W = torch.from_numpy(o.dequant_packed(packed, cb.astype(np.float32), n, k, 3)).to(dev)
    ref = xt.double() @ W.double().T
    y = ops.gemm_prefill(xt, p, c, 3, 128, n, k, out_dtype=torch.float32)
    yl = nbt.PackedLinear(p, c, n, k)(xt)
    torch.cuda.synchronize()
    assert ops.prefill_status(dev) == 0
    assert (y.double() - ref).abs().max() <= 2e-5 * ref.abs().max()
    assert yl.dtype == torch.float32 and (yl.double() - ref).abs().max() <= 2e-5 * ref.abs().max()
